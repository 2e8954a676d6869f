// Torch operator registry of the fused-MoE path.
//
// Registers, on the CUDA dispatch key, the operator schemas that
// vllm-xpu-kernels registers on XPU for this path (csrc/moe/torch_bindings.cpp,
// csrc/torch_bindings.cpp, csrc/xpu/torch_bindings.cpp) in the same three
// library namespaces.  Each implementation validates its tensors, allocates
// scratch through torch's caching allocator and calls the C ABI of
// libb200moe.so on the current CUDA stream.  There is no other code path: if a
// tensor is not on a CUDA device the dispatcher has no kernel to run.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>
#include <torch/library.h>

#include <optional>
#include <string>
#include <tuple>

#include "b200moe.h"

#ifndef B200MOE_NS_C
#define B200MOE_NS_C _C
#endif
#ifndef B200MOE_NS_MOE_C
#define B200MOE_NS_MOE_C _moe_C
#endif
#ifndef B200MOE_NS_XPU_C
#define B200MOE_NS_XPU_C _xpu_C
#endif

namespace {

using at::Tensor;
using OptTensor = std::optional<Tensor>;

void* cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check(int status, const char* op) {
  TORCH_CHECK(status == B200MOE_OK, op, ": ", b200moe_status_string(status), " (",
              b200moe_last_error(), ")");
}

int float_code(const Tensor& t, const char* what) {
  switch (t.scalar_type()) {
    case at::kFloat: return B200MOE_F32;
    case at::kHalf: return B200MOE_F16;
    case at::kBFloat16: return B200MOE_BF16;
    default: TORCH_CHECK(false, what, ": unsupported dtype ", t.scalar_type());
  }
  return -1;
}

int index_code(const Tensor& t, const char* what) {
  switch (t.scalar_type()) {
    case at::kInt: return B200MOE_I32;
    case at::kLong: return B200MOE_I64;
    case at::kUInt32: return B200MOE_U32;
    default: TORCH_CHECK(false, what, ": index tensor must be int32, uint32 or int64");
  }
  return -1;
}

const void* opt_ptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }

Tensor workspace(size_t bytes, const Tensor& like) {
  return at::empty({static_cast<int64_t>(bytes ? bytes : 1)}, like.options().dtype(at::kByte));
}

// ---- routing ------------------------------------------------------------------

void topk_common(bool sigmoid, Tensor& topk_weights, Tensor& topk_indices,
                 Tensor& token_expert_indices, const Tensor& gating_output, bool renormalize,
                 const OptTensor& bias, double scale, const OptTensor& is_padding) {
  const char* op = sigmoid ? "topk_sigmoid" : "topk_softmax";
  TORCH_CHECK(gating_output.dim() >= 1 && gating_output.is_contiguous(), op,
              ": gating_output must be contiguous");
  const int64_t E = gating_output.size(-1);
  const int64_t T = gating_output.numel() / E;
  const int64_t k = topk_weights.size(-1);
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat, op, ": topk_weights must be float32");
  TORCH_CHECK(topk_weights.is_contiguous() && topk_indices.is_contiguous() &&
                  token_expert_indices.is_contiguous(),
              op, ": outputs must be contiguous");
  TORCH_CHECK(topk_indices.numel() == T * k && topk_weights.numel() == T * k, op,
              ": output shape mismatch");
  TORCH_CHECK(token_expert_indices.scalar_type() == at::kInt, op,
              ": token_expert_indices must be int32");
  Tensor bias_f;
  const float* bias_p = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->numel() == E, op, ": bias must have num_experts entries");
    bias_f = bias->to(at::kFloat).contiguous();
    bias_p = bias_f.data_ptr<float>();
  }
  Tensor pad_u8;
  const uint8_t* pad_p = nullptr;
  if (is_padding.has_value()) {
    TORCH_CHECK(is_padding->numel() == T, op, ": is_padding must have one entry per row");
    pad_u8 = is_padding->to(at::kBool).contiguous();
    pad_p = reinterpret_cast<const uint8_t*>(pad_u8.data_ptr());
  }
  c10::cuda::CUDAGuard guard(gating_output.device());
  const int in = float_code(gating_output, op);
  const int idt = index_code(topk_indices, op);
  int rc;
  if (sigmoid)
    rc = b200moe_topk_sigmoid(gating_output.data_ptr(), in, T, E, k, renormalize, bias_p,
                              static_cast<float>(scale), pad_p, topk_weights.data_ptr<float>(),
                              topk_indices.data_ptr(), idt, token_expert_indices.data_ptr<int>(),
                              cur_stream());
  else
    rc = b200moe_topk_softmax(gating_output.data_ptr(), in, T, E, k, renormalize, bias_p, pad_p,
                              topk_weights.data_ptr<float>(), topk_indices.data_ptr(), idt,
                              token_expert_indices.data_ptr<int>(), cur_stream());
  check(rc, op);
}

void topk_softmax(Tensor& w, Tensor& ids, Tensor& src, const Tensor& gating, bool renorm,
                  const OptTensor& bias, const OptTensor& is_padding) {
  topk_common(false, w, ids, src, gating, renorm, bias, 1.0, is_padding);
}

void topk_sigmoid(Tensor& w, Tensor& ids, Tensor& src, const Tensor& gating, bool renorm,
                  const OptTensor& bias, double scale, const OptTensor& is_padding) {
  topk_common(true, w, ids, src, gating, renorm, bias, scale, is_padding);
}

void topk_softplus_sqrt(Tensor& topk_weights, Tensor& topk_indices, Tensor& token_expert_indices,
                        const Tensor& gating_output, bool renormalize, double routed_scaling_factor,
                        const OptTensor& correction_bias, const OptTensor& input_ids,
                        const OptTensor& tid2eid, const OptTensor& is_padding) {
  const char* op = "topk_softplus_sqrt";
  TORCH_CHECK(gating_output.is_contiguous(), op, ": gating_output must be contiguous");
  const int64_t E = gating_output.size(-1);
  const int64_t T = gating_output.numel() / E;
  const int64_t k = topk_weights.size(-1);
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat && topk_weights.is_contiguous() &&
                  topk_indices.is_contiguous() && token_expert_indices.is_contiguous(),
              op, ": outputs must be contiguous, weights float32");
  TORCH_CHECK(token_expert_indices.scalar_type() == at::kInt, op, ": token_expert_indices must be int32");
  TORCH_CHECK(input_ids.has_value() == tid2eid.has_value(), op, ": input_ids and tid2eid go together");
  Tensor bias_f, pad_u8, table;
  const float* bias_p = nullptr;
  const uint8_t* pad_p = nullptr;
  if (correction_bias.has_value()) {
    TORCH_CHECK(correction_bias->numel() == E, op, ": bias must have num_experts entries");
    bias_f = correction_bias->to(at::kFloat).contiguous();
    bias_p = bias_f.data_ptr<float>();
  }
  if (is_padding.has_value()) {
    pad_u8 = is_padding->to(at::kBool).contiguous();
    pad_p = reinterpret_cast<const uint8_t*>(pad_u8.data_ptr());
  }
  const void* ids_in = nullptr;
  int ids_in_dtype = B200MOE_I32;
  const int32_t* table_p = nullptr;
  if (tid2eid.has_value()) {
    TORCH_CHECK(tid2eid->dim() == 2 && tid2eid->size(1) == k, op, ": tid2eid must be [vocab, topk]");
    TORCH_CHECK(input_ids->is_contiguous() && input_ids->numel() == T, op, ": one input id per token");
    table = tid2eid->to(at::kInt).contiguous();
    table_p = table.data_ptr<int>();
    ids_in = input_ids->data_ptr();
    ids_in_dtype = index_code(*input_ids, op);
  }
  c10::cuda::CUDAGuard guard(gating_output.device());
  check(b200moe_topk_softplus_sqrt(gating_output.data_ptr(), float_code(gating_output, op), T, E, k,
                                   renormalize, static_cast<float>(routed_scaling_factor), bias_p,
                                   ids_in, ids_in_dtype, table_p, pad_p,
                                   topk_weights.data_ptr<float>(), topk_indices.data_ptr(),
                                   index_code(topk_indices, op), token_expert_indices.data_ptr<int>(),
                                   cur_stream()),
        op);
}

std::tuple<Tensor, Tensor> grouped_topk(const Tensor& scores, int64_t n_group, int64_t topk_group,
                                        int64_t topk, bool renormalize, double scale,
                                        const Tensor& bias, int64_t scoring_func) {
  TORCH_CHECK(scores.dim() == 2 && scores.is_contiguous(), "grouped_topk: scores must be [T, E] contiguous");
  const int64_t T = scores.size(0), E = scores.size(1);
  TORCH_CHECK(bias.numel() == E && bias.is_contiguous(), "grouped_topk: bias must have num_experts entries");
  TORCH_CHECK(n_group > 0 && n_group <= 32, "grouped_topk: n_group must be in [1, 32]");
  TORCH_CHECK(topk > 0 && topk <= 32, "grouped_topk: topk must be in [1, 32]");
  TORCH_CHECK(E % n_group == 0, "grouped_topk: num_experts must be divisible by n_group");
  c10::cuda::CUDAGuard guard(scores.device());
  Tensor values = at::empty({T, topk}, scores.options().dtype(at::kFloat));
  Tensor ids = at::empty({T, topk}, scores.options().dtype(at::kInt));
  check(b200moe_grouped_topk(scores.data_ptr(), float_code(scores, "grouped_topk"), bias.data_ptr(),
                             float_code(bias, "grouped_topk"), T, E, n_group, topk_group, topk,
                             renormalize, static_cast<float>(scale), scoring_func,
                             values.data_ptr<float>(), ids.data_ptr<int>(), cur_stream()),
        "grouped_topk");
  return {values, ids};
}

// ---- permutation -----------------------------------------------------------------

void moe_align_block_size(const Tensor& topk_ids, int64_t num_experts, int64_t block_size,
                          Tensor& sorted_token_ids, Tensor& experts_ids,
                          Tensor& num_tokens_post_pad, const OptTensor& maybe_expert_map) {
  TORCH_CHECK(topk_ids.is_contiguous(), "moe_align_block_size: topk_ids must be contiguous");
  TORCH_CHECK(sorted_token_ids.scalar_type() == at::kInt && experts_ids.scalar_type() == at::kInt &&
                  num_tokens_post_pad.scalar_type() == at::kInt,
              "moe_align_block_size: outputs must be int32");
  TORCH_CHECK(num_experts <= 1024, "moe_align_block_size: at most 1024 experts");
  if (maybe_expert_map.has_value())
    TORCH_CHECK(maybe_expert_map->scalar_type() == at::kInt && maybe_expert_map->is_contiguous(),
                "moe_align_block_size: expert_map must be contiguous int32");
  c10::cuda::CUDAGuard guard(topk_ids.device());
  const size_t ws = b200moe_moe_align_block_size_workspace_bytes(topk_ids.numel(), num_experts);
  Tensor w = workspace(ws, topk_ids);
  check(b200moe_moe_align_block_size(
            topk_ids.data_ptr(), index_code(topk_ids, "moe_align_block_size"), topk_ids.numel(),
            num_experts, block_size,
            reinterpret_cast<const int32_t*>(opt_ptr(maybe_expert_map)),
            sorted_token_ids.data_ptr<int>(), sorted_token_ids.numel(), experts_ids.data_ptr<int>(),
            experts_ids.numel(), num_tokens_post_pad.data_ptr<int>(), w.data_ptr(), ws,
            cur_stream()),
        "moe_align_block_size");
}

void batched_moe_align_block_size(int64_t max_tokens_per_batch, int64_t block_size,
                                  const Tensor& expert_num_tokens, Tensor& sorted_token_ids,
                                  Tensor& experts_ids, Tensor& num_tokens_post_pad) {
  const int64_t B = expert_num_tokens.size(0);
  const int64_t blocks = (max_tokens_per_batch + block_size - 1) / block_size * B;
  TORCH_CHECK(expert_num_tokens.scalar_type() == at::kInt && expert_num_tokens.is_contiguous(),
              "batched_moe_align_block_size: expert_num_tokens must be contiguous int32");
  TORCH_CHECK(sorted_token_ids.size(0) == blocks * block_size);
  TORCH_CHECK(experts_ids.size(0) == blocks);
  TORCH_CHECK(num_tokens_post_pad.size(0) == 1);
  TORCH_CHECK(B <= 1024);
  c10::cuda::CUDAGuard guard(expert_num_tokens.device());
  check(b200moe_batched_moe_align_block_size(max_tokens_per_batch, block_size,
                                             expert_num_tokens.data_ptr<int>(), B,
                                             sorted_token_ids.data_ptr<int>(),
                                             experts_ids.data_ptr<int>(),
                                             num_tokens_post_pad.data_ptr<int>(), cur_stream()),
        "batched_moe_align_block_size");
}

void moe_lora_align_block_size(const Tensor& topk_ids, const Tensor& token_lora_mapping,
                               int64_t num_experts, int64_t block_size, int64_t max_loras,
                               int64_t max_num_tokens_padded, int64_t max_num_m_blocks,
                               Tensor& sorted_token_ids, Tensor& expert_ids,
                               Tensor& num_tokens_post_pad, Tensor& adapter_enabled,
                               Tensor& lora_ids, const std::optional<Tensor>& maybe_expert_map) {
  const char* op = "moe_lora_align_block_size";
  TORCH_CHECK(block_size > 0, "block_size should be greater than 0. ");
  TORCH_CHECK(topk_ids.dim() == 2 && topk_ids.is_contiguous(), op, ": topk_ids must be contiguous [T, k]");
  TORCH_CHECK(num_experts <= 1024, op, ": at most 1024 experts");
  const Tensor* int_tensors[] = {&token_lora_mapping, &sorted_token_ids, &expert_ids,
                                 &num_tokens_post_pad, &adapter_enabled, &lora_ids};
  for (const Tensor* t : int_tensors)
    TORCH_CHECK(t->scalar_type() == at::kInt && t->is_contiguous(), op, ": int32 contiguous tensors expected");
  TORCH_CHECK(token_lora_mapping.numel() == topk_ids.size(0), op, ": one adapter slot per token");
  TORCH_CHECK(sorted_token_ids.numel() >= max_loras * max_num_tokens_padded &&
                  expert_ids.numel() >= max_loras * max_num_m_blocks &&
                  num_tokens_post_pad.numel() >= max_loras && adapter_enabled.numel() >= max_loras &&
                  lora_ids.numel() >= max_loras + 1,
              op, ": output / slot tensors are too small for max_loras");
  if (maybe_expert_map)
    TORCH_CHECK(maybe_expert_map->scalar_type() == at::kInt && maybe_expert_map->numel() >= num_experts,
                op, ": expert_map must be int32 [num_experts]");
  c10::cuda::CUDAGuard guard(topk_ids.device());
  check(b200moe_moe_lora_align_block_size(
            topk_ids.data_ptr(), index_code(topk_ids, op), topk_ids.size(0), topk_ids.size(1),
            token_lora_mapping.data_ptr<int>(), num_experts, block_size, max_loras,
            max_num_tokens_padded, max_num_m_blocks, sorted_token_ids.data_ptr<int>(),
            expert_ids.data_ptr<int>(), num_tokens_post_pad.data_ptr<int>(),
            adapter_enabled.data_ptr<int>(), lora_ids.data_ptr<int>(),
            reinterpret_cast<const int32_t*>(opt_ptr(maybe_expert_map)), cur_stream()),
        op);
}

Tensor reorder_mxfp_scales(const Tensor& A_scales, const Tensor& rows_per_expert,
                           int64_t total_padded_rows) {
  TORCH_CHECK(A_scales.dim() == 2, "A_scales must be 2D [total_rows, scale_k]");
  TORCH_CHECK(A_scales.scalar_type() == at::kFloat8_e8m0fnu, "A_scales must be float8_e8m0fnu");
  TORCH_CHECK(A_scales.is_contiguous(), "A_scales must be contiguous");
  TORCH_CHECK(rows_per_expert.scalar_type() == at::kInt, "rows_per_expert must be int32");
  TORCH_CHECK(rows_per_expert.is_contiguous(), "rows_per_expert must be contiguous");
  c10::cuda::CUDAGuard guard(A_scales.device());
  Tensor out = at::empty({total_padded_rows, A_scales.size(1)}, A_scales.options());
  check(b200moe_reorder_mxfp_scales(reinterpret_cast<const uint8_t*>(A_scales.data_ptr()),
                                    rows_per_expert.data_ptr<int>(), rows_per_expert.size(0),
                                    A_scales.size(1), total_padded_rows,
                                    reinterpret_cast<uint8_t*>(out.data_ptr()), cur_stream()),
        "reorder_mxfp_scales");
  return out;
}

void init_expert_map(Tensor expert_map, int64_t num_experts, int64_t ep_rank, int64_t ep_size) {
  TORCH_CHECK(expert_map.scalar_type() == at::kInt && expert_map.is_contiguous(),
              "init_expert_map: expert_map must be contiguous int32");
  TORCH_CHECK(expert_map.numel() == num_experts * ep_size, "init_expert_map: size mismatch");
  c10::cuda::CUDAGuard guard(expert_map.device());
  check(b200moe_init_expert_map(expert_map.data_ptr<int>(), num_experts, ep_rank, ep_size,
                                cur_stream()),
        "init_expert_map");
}

void remap_hidden_states(const Tensor& hidden_states, const OptTensor& hidden_states_scales,
                         Tensor remapped_hidden_states, const OptTensor& remapped_scales,
                         const OptTensor& expert_map, Tensor rows_per_expert,
                         Tensor unpermuted_row_to_permuted_row, const Tensor& topk_ids,
                         int64_t total_experts_num, int64_t local_experts_num) {
  TORCH_CHECK(hidden_states.dim() == 2 && hidden_states.is_contiguous() &&
                  remapped_hidden_states.is_contiguous(),
              "remap_hidden_states: hidden states must be contiguous 2-D");
  TORCH_CHECK(topk_ids.dim() == 2 && topk_ids.is_contiguous(), "remap_hidden_states: topk_ids must be [T, k]");
  TORCH_CHECK(rows_per_expert.scalar_type() == at::kInt &&
                  unpermuted_row_to_permuted_row.scalar_type() == at::kInt,
              "remap_hidden_states: rows_per_expert and the row map must be int32");
  TORCH_CHECK(local_experts_num <= 1024, "remap_hidden_states: at most 1024 local experts");
  const int64_t T = hidden_states.size(0), k = topk_ids.size(1);
  const int64_t row_bytes = hidden_states.size(1) * hidden_states.element_size();
  TORCH_CHECK(row_bytes % 16 == 0, "remap_hidden_states: a row must be a multiple of 16 bytes");
  TORCH_CHECK(remapped_hidden_states.numel() * remapped_hidden_states.element_size() >= T * k * row_bytes,
              "remap_hidden_states: remapped buffer too small");
  int64_t scale_row_bytes = 0;
  if (hidden_states_scales.has_value()) {
    TORCH_CHECK(remapped_scales.has_value(), "remap_hidden_states: remapped scales missing");
    TORCH_CHECK(hidden_states_scales->is_contiguous() && remapped_scales->is_contiguous(),
                "remap_hidden_states: scales must be contiguous");
    scale_row_bytes = hidden_states_scales->size(1) * hidden_states_scales->element_size();
  }
  Tensor map32;
  const int32_t* map_p = nullptr;
  if (expert_map.has_value()) {
    map32 = expert_map->scalar_type() == at::kInt ? expert_map->contiguous()
                                                  : expert_map->to(at::kInt).contiguous();
    map_p = map32.data_ptr<int>();
  }
  c10::cuda::CUDAGuard guard(hidden_states.device());
  const size_t ws = b200moe_remap_hidden_states_workspace_bytes(T, k, local_experts_num);
  Tensor w = workspace(ws, topk_ids);
  check(b200moe_remap_hidden_states(
            hidden_states.data_ptr(), opt_ptr(hidden_states_scales),
            remapped_hidden_states.data_ptr(),
            remapped_scales.has_value() ? remapped_scales->data_ptr() : nullptr, row_bytes,
            scale_row_bytes, topk_ids.data_ptr(), index_code(topk_ids, "remap_hidden_states"),
            map_p, T, k, total_experts_num, local_experts_num, rows_per_expert.data_ptr<int>(),
            unpermuted_row_to_permuted_row.data_ptr<int>(), w.data_ptr(), ws, cur_stream()),
        "remap_hidden_states");
}

void b200_moe_gather_add(Tensor& output, const Tensor& moe_output, const Tensor& topk_weights,
                         const Tensor& row_map, const Tensor& addend) {
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat, "b200_moe_gather_add: topk_weights must be float32");
  TORCH_CHECK(output.scalar_type() == moe_output.scalar_type() && addend.scalar_type() == output.scalar_type(),
              "b200_moe_gather_add: dtype mismatch");
  TORCH_CHECK(output.is_contiguous() && moe_output.is_contiguous() && topk_weights.is_contiguous() &&
                  row_map.is_contiguous() && addend.is_contiguous() && addend.sizes() == output.sizes(),
              "b200_moe_gather_add: contiguous tensors, addend shaped like the output");
  TORCH_CHECK(row_map.scalar_type() == at::kInt, "b200_moe_gather_add: row map must be int32");
  const int64_t T = output.size(0), H = output.size(1), k = topk_weights.size(1);
  c10::cuda::CUDAGuard guard(output.device());
  check(b200moe_moe_gather_add(output.data_ptr(), moe_output.data_ptr(), float_code(output, "b200_moe_gather_add"),
                               topk_weights.data_ptr<float>(), row_map.data_ptr<int>(), addend.data_ptr(),
                               T, k, H, cur_stream()),
        "b200_moe_gather_add");
}

void b200_moe_gather_bounded(Tensor& output, const Tensor& moe_output, const Tensor& topk_weights,
                             const Tensor& row_map, const Tensor& valid_tokens) {
  const char* op = "b200_moe_gather_bounded";
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat, op, ": topk_weights must be float32");
  TORCH_CHECK(output.scalar_type() == moe_output.scalar_type(), op, ": dtype mismatch");
  TORCH_CHECK(output.is_contiguous() && moe_output.is_contiguous() && topk_weights.is_contiguous() &&
                  row_map.is_contiguous(), op, ": tensors must be contiguous");
  TORCH_CHECK(row_map.scalar_type() == at::kInt && valid_tokens.scalar_type() == at::kInt &&
                  valid_tokens.numel() >= 1 && valid_tokens.is_cuda(),
              op, ": row map and the valid-token count must be int32 on the device");
  const int64_t T = output.size(0), H = output.size(1), k = topk_weights.size(1);
  c10::cuda::CUDAGuard guard(output.device());
  check(b200moe_moe_gather_bounded(output.data_ptr(), moe_output.data_ptr(), float_code(output, op),
                                   topk_weights.data_ptr<float>(), row_map.data_ptr<int>(),
                                   valid_tokens.data_ptr<int>(), T, k, H, cur_stream()),
        op);
}

void moe_gather(Tensor& output, const Tensor& moe_output, const Tensor& topk_weights,
                const Tensor& unpermuted_row_to_permuted_row, int64_t /*num_experts*/) {
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat, "moe_gather: topk_weights must be float32");
  TORCH_CHECK(output.scalar_type() == moe_output.scalar_type(), "moe_gather: dtype mismatch");
  TORCH_CHECK(output.is_contiguous() && moe_output.is_contiguous() && topk_weights.is_contiguous() &&
                  unpermuted_row_to_permuted_row.is_contiguous(),
              "moe_gather: tensors must be contiguous");
  TORCH_CHECK(unpermuted_row_to_permuted_row.scalar_type() == at::kInt, "moe_gather: row map must be int32");
  const int64_t T = output.size(0), H = output.size(1), k = topk_weights.size(1);
  c10::cuda::CUDAGuard guard(output.device());
  check(b200moe_moe_gather(output.data_ptr(), moe_output.data_ptr(), float_code(output, "moe_gather"),
                           topk_weights.data_ptr<float>(),
                           unpermuted_row_to_permuted_row.data_ptr<int>(), T, k, H, cur_stream()),
        "moe_gather");
}

void moe_sum(const Tensor& input, Tensor& output, const OptTensor& topk_ids,
             const OptTensor& expert_map) {
  TORCH_CHECK(input.dim() == 3, "moe_sum: input must be [num_tokens, topk, hidden]");
  const int64_t num_tokens = input.size(0), topk = input.size(1), hidden = input.size(2);
  TORCH_CHECK(input.scalar_type() == output.scalar_type(),
              "moe_sum: input and output must have the same dtype");
  TORCH_CHECK(input.device() == output.device(), "moe_sum: input and output must be on the same device");
  TORCH_CHECK(input.is_contiguous() && output.is_contiguous(),
              "moe_sum expects contiguous input and output");
  TORCH_CHECK(input.numel() == output.numel() * topk,
              "moe_sum: input shape must be [num_tokens, topk, hidden] matching output "
              "[num_tokens, hidden]");
  TORCH_CHECK(!(expert_map.has_value() && !topk_ids.has_value()),
              "moe_sum: expert_map requires topk_ids to be provided");
  int idt = B200MOE_I32;
  if (topk_ids.has_value()) {
    const Tensor& tk = *topk_ids;
    TORCH_CHECK(tk.is_contiguous(), "moe_sum: topk_ids must be contiguous");
    TORCH_CHECK(tk.device() == input.device(), "moe_sum: topk_ids must be on the same device as input");
    TORCH_CHECK(tk.dim() == 2 && tk.size(0) == num_tokens && tk.size(1) == topk,
                "moe_sum: topk_ids must have shape [num_tokens, topk]");
    idt = index_code(tk, "moe_sum");
    if (expert_map.has_value()) {
      TORCH_CHECK(expert_map->scalar_type() == at::kInt, "moe_sum: expert_map must be int32");
      TORCH_CHECK(expert_map->is_contiguous(), "moe_sum: expert_map must be contiguous");
      TORCH_CHECK(expert_map->device() == input.device(),
                  "moe_sum: expert_map must be on the same device as input");
    }
  }
  c10::cuda::CUDAGuard guard(input.device());
  check(b200moe_moe_sum(input.data_ptr(), output.data_ptr(), float_code(input, "moe_sum"),
                        num_tokens, topk, hidden, opt_ptr(topk_ids), idt,
                        reinterpret_cast<const int32_t*>(opt_ptr(expert_map)), cur_stream()),
        "moe_sum");
}

// ---- activations / quantisation -----------------------------------------------------

void silu_and_mul(Tensor& result, const Tensor& input) {
  TORCH_CHECK(input.is_contiguous() && result.is_contiguous(), "silu_and_mul: tensors must be contiguous");
  TORCH_CHECK(input.scalar_type() == result.scalar_type(), "silu_and_mul: dtype mismatch");
  const int64_t d = input.size(-1) / 2;
  TORCH_CHECK(result.size(-1) == d, "silu_and_mul: output must have half the input's last dim");
  c10::cuda::CUDAGuard guard(input.device());
  check(b200moe_silu_and_mul(result.data_ptr(), input.data_ptr(), float_code(input, "silu_and_mul"),
                             input.numel() / (2 * d), d, cur_stream()),
        "silu_and_mul");
}

void swigluoai_and_mul(Tensor& out, const Tensor& input, double alpha, double limit) {
  TORCH_CHECK(input.is_contiguous() && out.is_contiguous(), "swigluoai_and_mul: tensors must be contiguous");
  TORCH_CHECK(input.scalar_type() == out.scalar_type(), "swigluoai_and_mul: dtype mismatch");
  const int64_t d = input.size(-1) / 2;
  c10::cuda::CUDAGuard guard(input.device());
  check(b200moe_swigluoai_and_mul(out.data_ptr(), input.data_ptr(),
                                  float_code(input, "swigluoai_and_mul"), input.numel() / (2 * d), d,
                                  static_cast<float>(alpha), static_cast<float>(limit), cur_stream()),
        "swigluoai_and_mul");
}

// Shared body of the other activations; `name` prefixes the error texts.
void act_and_mul_common(Tensor& out, const Tensor& input, int act, double p0, double p1,
                        double clamp_limit, const char* name) {
  TORCH_CHECK(input.dim() >= 1, name, " input must have at least one dimension");
  const bool gated = act != B200MOE_ACT_RELU2_NO_MUL;
  if (gated)
    TORCH_CHECK(input.size(-1) > 0 && input.size(-1) % 2 == 0, name,
                " input last dimension must be positive and even");
  TORCH_CHECK(input.is_contiguous(), name, " input must be contiguous");
  TORCH_CHECK(out.is_contiguous(), name, " output must be contiguous");
  TORCH_CHECK(out.device() == input.device(), name, " input and output must be on the same device");
  TORCH_CHECK(out.scalar_type() == input.scalar_type(), name,
              " input and output must have the same dtype");
  TORCH_CHECK(out.dim() == input.dim(), name,
              " input and output must have the same number of dimensions");
  for (int64_t dim = 0; dim < input.dim() - 1; ++dim)
    TORCH_CHECK(out.size(dim) == input.size(dim), name,
                " input and output leading dimensions must match");
  const int64_t d = gated ? input.size(-1) / 2 : input.size(-1);
  TORCH_CHECK(out.size(-1) == d, name,
              gated ? " output last dimension must be half the input last dimension"
                    : " output must have the input's shape");
  if (input.numel() == 0) return;
  c10::cuda::CUDAGuard guard(input.device());
  check(b200moe_act_and_mul(out.data_ptr(), input.data_ptr(), float_code(input, name),
                            input.numel() / input.size(-1), d, act, static_cast<float>(p0),
                            static_cast<float>(p1), static_cast<float>(clamp_limit), cur_stream()),
        name);
}

void gelu_and_mul(Tensor& out, const Tensor& input) {
  act_and_mul_common(out, input, B200MOE_ACT_GELU, 0, 0, 0, "gelu_and_mul:");
}
void gelu_tanh_and_mul(Tensor& out, const Tensor& input) {
  act_and_mul_common(out, input, B200MOE_ACT_GELU_TANH, 0, 0, 0, "gelu_tanh_and_mul:");
}
void relu2_no_mul(Tensor& out, Tensor& input) {
  act_and_mul_common(out, input, B200MOE_ACT_RELU2_NO_MUL, 0, 0, 0, "relu2_no_mul:");
}
void swiglustep_and_mul(Tensor& out, const Tensor& input, double limit) {
  act_and_mul_common(out, input, B200MOE_ACT_SWIGLUSTEP, limit, 0, 0, "swiglustep_and_mul:");
}
void situ_and_mul(Tensor& out, const Tensor& input, double beta, double linear_beta) {
  // same argument checks and texts as csrc/activation.cpp:777-780 of the reference
  TORCH_CHECK(std::isfinite(beta) && beta > 0.0, "SITU beta must be finite and greater than zero");
  TORCH_CHECK(std::isfinite(linear_beta), "SITU linear_beta must be finite");
  act_and_mul_common(out, input, B200MOE_ACT_SITU, beta, linear_beta, 0, "SITU");
}
// Extended: any of the activations with the layer's gemm1 clamp folded in.
void b200_act_and_mul(Tensor& out, const Tensor& input, int64_t act, double p0, double p1,
                      double clamp_limit) {
  act_and_mul_common(out, input, static_cast<int>(act), p0, p1, clamp_limit, "b200_act_and_mul:");
}

void scale_strides(const Tensor& s, int64_t rows, int64_t groups, int64_t* sr, int64_t* sg) {
  TORCH_CHECK(s.scalar_type() == at::kFloat, "group quant: scales must be float32");
  TORCH_CHECK(s.numel() == rows * groups, "group quant: scales must have one entry per group");
  if (s.dim() >= 2) {
    *sr = s.stride(-2);
    *sg = s.stride(-1);
  } else {
    *sr = groups;
    *sg = 1;
  }
}

void per_token_group_fp8_quant(const Tensor& input, Tensor& output_q, Tensor& output_s,
                               int64_t group_size, double eps, double fp8_min, double fp8_max,
                               bool scale_ue8m0, bool, bool) {
  TORCH_CHECK(input.is_contiguous() && output_q.is_contiguous(), "per_token_group_fp8_quant: contiguous tensors expected");
  TORCH_CHECK(output_q.scalar_type() == at::kFloat8_e4m3fn, "per_token_group_fp8_quant: output must be float8_e4m3fn");
  const int64_t N = input.size(-1);
  TORCH_CHECK(N % group_size == 0, "per_token_group_fp8_quant: hidden size must be divisible by group_size");
  const int64_t R = input.numel() / N;
  int64_t sr, sg;
  scale_strides(output_s, R, N / group_size, &sr, &sg);
  c10::cuda::CUDAGuard guard(input.device());
  check(b200moe_per_token_group_fp8_quant(
            input.data_ptr(), float_code(input, "per_token_group_fp8_quant"), output_q.data_ptr(),
            output_s.data_ptr<float>(), R, N, group_size, static_cast<float>(eps),
            static_cast<float>(fp8_min), static_cast<float>(fp8_max), scale_ue8m0, sr, sg,
            cur_stream()),
        "per_token_group_fp8_quant");
}

void per_token_group_quant_mxfp4(const Tensor& input, Tensor& output_q, Tensor& output_s,
                                 int64_t group_size, double eps) {
  TORCH_CHECK(input.is_contiguous() && output_q.is_contiguous(), "per_token_group_quant_mxfp4: contiguous tensors expected");
  TORCH_CHECK(group_size == 32, "per_token_group_quant_mxfp4: group_size must be 32");
  const int64_t N = input.size(-1);
  const int64_t R = input.numel() / N;
  TORCH_CHECK(output_q.numel() * output_q.element_size() == R * N / 2,
              "per_token_group_quant_mxfp4: output must hold two values per byte");
  int64_t sr, sg;
  scale_strides(output_s, R, N / 32, &sr, &sg);
  c10::cuda::CUDAGuard guard(input.device());
  check(b200moe_per_token_group_quant_mxfp4(
            input.data_ptr(), float_code(input, "per_token_group_quant_mxfp4"),
            reinterpret_cast<uint8_t*>(output_q.data_ptr()), output_s.data_ptr<float>(), R, N,
            group_size, static_cast<float>(eps), sr, sg, cur_stream()),
        "per_token_group_quant_mxfp4");
}

void silu_and_mul_per_block_quant(Tensor& out, const Tensor& input, Tensor& scales,
                                  int64_t group_size, const OptTensor& scale_ub,
                                  bool is_scale_transposed, bool scale_ue8m0) {
  TORCH_CHECK(input.is_contiguous() && out.is_contiguous(), "silu_and_mul_per_block_quant: contiguous tensors expected");
  TORCH_CHECK(out.scalar_type() == at::kFloat8_e4m3fn, "silu_and_mul_per_block_quant: output must be float8_e4m3fn");
  const int64_t d = input.size(-1) / 2;
  const int64_t R = input.numel() / (2 * d);
  TORCH_CHECK(d % group_size == 0, "silu_and_mul_per_block_quant: hidden size must be divisible by group_size");
  int64_t sr, sg;
  scale_strides(scales, R, d / group_size, &sr, &sg);
  if (is_scale_transposed && scales.dim() >= 2 && scales.size(0) != R) { sr = scales.stride(-1); sg = scales.stride(-2); }
  c10::cuda::CUDAGuard guard(input.device());
  check(b200moe_silu_mul_block_quant(
            input.data_ptr(), float_code(input, "silu_and_mul_per_block_quant"), out.data_ptr(),
            scales.data_ptr<float>(), R, d, group_size,
            scale_ub.has_value() ? scale_ub->data_ptr<float>() : nullptr, scale_ue8m0, sr, sg,
            cur_stream()),
        "silu_and_mul_per_block_quant");
}

void silu_and_mul_mxfp4_quant(Tensor& out, const Tensor& input, Tensor& scales, int64_t group_size,
                              double eps) {
  TORCH_CHECK(input.is_contiguous() && out.is_contiguous() && scales.is_contiguous(),
              "silu_and_mul_mxfp4_quant: contiguous tensors expected");
  TORCH_CHECK(scales.scalar_type() == at::kFloat, "silu_and_mul_mxfp4_quant: scales must be float32");
  const int64_t d = input.size(-1) / 2;
  const int64_t R = input.numel() / (2 * d);
  c10::cuda::CUDAGuard guard(input.device());
  check(b200moe_silu_mul_mxfp4_quant(input.data_ptr(), float_code(input, "silu_and_mul_mxfp4_quant"),
                                     reinterpret_cast<uint8_t*>(out.data_ptr()),
                                     scales.data_ptr<float>(), R, d, group_size,
                                     static_cast<float>(eps), cur_stream()),
        "silu_and_mul_mxfp4_quant");
}

// ---- grouped GEMM -----------------------------------------------------------------

int act_code(const Tensor& t, const char* op) {
  if (t.scalar_type() == at::kFloat8_e4m3fn) return B200MOE_E4M3;
  return float_code(t, op);
}

// Shared by the reference-named entry and the extended one.
Tensor grouped_gemm_impl(const Tensor& A, const OptTensor& A_scale, const Tensor& B,
                         const OptTensor& B_scale, const OptTensor& bias, Tensor D,
                         const Tensor& rows_per_expert, int64_t N, int64_t K, int64_t num_experts,
                         int64_t epilogue, int64_t b_layout, double alpha, double limit,
                         const OptTensor& D_scale = std::nullopt,
                         const OptTensor& D_row_ptr = std::nullopt, int64_t a_scale_layout = 0,
                         int64_t gated_act = 0, double act_param0 = 0.0, double act_param1 = 0.0,
                         double clamp_limit = 0.0, bool scales_pow2 = false) {
  const char* op = "cutlass_grouped_gemm_interface";
  TORCH_CHECK(A.is_contiguous() && B.is_contiguous() && D.is_contiguous(), op, ": A, B and D must be contiguous");
  TORCH_CHECK(rows_per_expert.scalar_type() == at::kInt && rows_per_expert.is_contiguous() &&
                  rows_per_expert.numel() >= num_experts,
              op, ": rows_per_expert must be int32 [num_experts]");
  TORCH_CHECK(N % 8 == 0, op, ": N must be a multiple of 8");
  b200moe_gemm_args a{};
  a.epilogue = static_cast<int>(epilogue);
  a.a_dtype = act_code(A, op);
  a.d_dtype = act_code(D, op);
  a.A = A.data_ptr();
  a.B = B.data_ptr();
  a.b_layout = static_cast<int>(b_layout);
  a.a_scale_layout = static_cast<int>(a_scale_layout);
  a.D = D.data_ptr();
  if (D_scale.has_value()) {
    TORCH_CHECK(D_scale->scalar_type() == at::kFloat && D_scale->is_contiguous(), op,
                ": output scales must be contiguous float32");
    a.d_scale = D_scale->data_ptr<float>();
  }
  if (D_row_ptr.has_value()) {
    TORCH_CHECK(D_row_ptr->scalar_type() == at::kLong && D_row_ptr->is_contiguous() &&
                    D_row_ptr->numel() >= A.numel() / K,
                op, ": the row address table must be int64 with one entry per row of A");
    a.d_row_ptr = D_row_ptr->data_ptr<int64_t>();
  }
  a.rows_per_expert = rows_per_expert.data_ptr<int>();
  a.R = A.numel() / K;
  a.N = N;
  a.K = K;
  a.E = num_experts;
  a.alpha = static_cast<float>(alpha);
  a.limit = static_cast<float>(limit);
  TORCH_CHECK(gated_act >= B200MOE_ACT_SILU && gated_act <= B200MOE_ACT_SITU, op,
              ": the fused gated activation is silu, gelu, gelu_tanh, swiglustep or situ");
  a.gated_act = static_cast<int>(gated_act);
  a.act_param0 = static_cast<float>(act_param0);
  a.act_param1 = static_cast<float>(act_param1);
  a.clamp_limit = static_cast<float>(clamp_limit);
  a.scales_pow2 = scales_pow2 ? 1 : 0;
  const auto bt = B.scalar_type();
  if (bt == at::kFloat8_e4m3fn && !B_scale.has_value() && !A_scale.has_value() &&
      a.a_dtype == B200MOE_E4M3) {
    // unit scales: the plain e4m3 x e4m3 contraction (throughput probe of the extended op)
    TORCH_CHECK(K % 128 == 0 && N % 128 == 0, op, ": FP8 needs K and N to be multiples of 128");
    a.recipe = B200MOE_RECIPE_FP8_BLOCK;
  } else if (bt == at::kFloat8_e4m3fn) {
    TORCH_CHECK(B_scale.has_value() && B_scale->scalar_type() == at::kFloat && B_scale->dim() == 3,
                op, ": float8 weights need float32 block scales [E, K/128, N/128]");
    TORCH_CHECK(B_scale->is_contiguous(), op, ": weight scales must be contiguous");
    TORCH_CHECK(K % 128 == 0 && N % 128 == 0, op, ": block-FP8 needs K and N to be multiples of 128");
    a.recipe = B200MOE_RECIPE_FP8_BLOCK;
    a.b_scale = B_scale->data_ptr();
    if (a.a_dtype == B200MOE_E4M3) {
      TORCH_CHECK(A_scale.has_value() && A_scale->scalar_type() == at::kFloat && A_scale->is_contiguous(),
                  op, ": float8 activations need float32 per-token-group-128 scales");
      a.a_scale = A_scale->data_ptr<float>();
    }
  } else if (bt == at::kChar) {
    // the reference's INT4 recipe (int8 pairs + 16-bit group scales,
    // csrc/xpu/grouped_gemm/xe_2/grouped_gemm_xe2_interface.hpp:193).  This operator keeps no
    // state between calls, so it does not widen such weights on every call behind the
    // caller's back: widen once and pass the result.
    TORCH_CHECK(false, op, ": INT4 weights are widened once with _xpu_C.b200_expand_weights(B, scales, "
                "\"int4\", dtype) (XpuFusedMoe(is_int4=True) does so at first use); pass the widened weights");
  } else if (bt == at::kFloat4_e2m1fn_x2 || (bt == at::kByte && B_scale.has_value())) {
    // uint8 is accepted as a view of packed e2m1 pairs only together with one-byte (e8m0)
    // scales; INT4 is int8 in the reference and never reaches this branch
    TORCH_CHECK(B_scale.has_value() && B_scale->element_size() == 1 && B_scale->is_contiguous(), op,
                ": MXFP4 weights need e8m0 scales [E, N, K/32] (uint8 weights with wider scales are "
                "not a recipe of this operator)");
    TORCH_CHECK(K % 32 == 0, op, ": MXFP4 needs K to be a multiple of 32");
    a.recipe = B200MOE_RECIPE_MXFP4;
    a.b_scale = B_scale->data_ptr();
  } else {
    TORCH_CHECK(bt == A.scalar_type(), op, ": 16-bit weights must have the activations' dtype");
    TORCH_CHECK(!B_scale.has_value(), op, ": 16-bit weights take no scales");
    a.recipe = B200MOE_RECIPE_BF16;
  }
  if (bias.has_value()) {
    TORCH_CHECK(bias->is_contiguous() && bias->numel() == num_experts * N, op, ": bias must be [E, N]");
    a.bias = bias->data_ptr();
    a.bias_dtype = float_code(*bias, op);
  }
  c10::cuda::CUDAGuard guard(A.device());
  const size_t ws = b200moe_grouped_gemm_workspace_bytes(&a);
  Tensor w = workspace(ws, rows_per_expert);
  check(b200moe_grouped_gemm(&a, w.data_ptr(), ws, cur_stream()), op);
  return D;
}

Tensor cutlass_grouped_gemm_interface(const Tensor& ptr_A, const OptTensor& ptr_A_scale,
                                      const Tensor& ptr_B, const OptTensor& ptr_B_scale,
                                      const OptTensor& ptr_bias, Tensor ptr_D,
                                      const Tensor& rows_per_expert, int64_t N, int64_t K,
                                      int64_t num_experts) {
  return grouped_gemm_impl(ptr_A, ptr_A_scale, ptr_B, ptr_B_scale, ptr_bias, ptr_D, rows_per_expert,
                           N, K, num_experts, B200MOE_EPI_STORE, B200MOE_B_LAYOUT_KN, 1.702, 7.0);
}

Tensor b200_grouped_gemm(const Tensor& A, const OptTensor& A_scale, const Tensor& B,
                         const OptTensor& B_scale, const OptTensor& bias, Tensor D,
                         const Tensor& rows_per_expert, int64_t N, int64_t K, int64_t num_experts,
                         int64_t epilogue, int64_t b_layout, double alpha, double limit,
                         const OptTensor& D_scale, const OptTensor& D_row_ptr,
                         int64_t a_scale_layout, int64_t gated_act, double act_param0,
                         double act_param1, double clamp_limit, bool scales_pow2) {
  return grouped_gemm_impl(A, A_scale, B, B_scale, bias, D, rows_per_expert, N, K, num_experts,
                           epilogue, b_layout, alpha, limit, D_scale, D_row_ptr, a_scale_layout,
                           gated_act, act_param0, act_param1, clamp_limit, scales_pow2);
}

Tensor b200_grouped_gemm_check(const Tensor& A, const OptTensor& A_scale, const Tensor& B,
                               const OptTensor& B_scale, const OptTensor& bias, Tensor D,
                               const Tensor& rows_per_expert, int64_t N, int64_t K,
                               int64_t num_experts, int64_t b_layout) {
  b200moe_gemm_args a{};
  a.a_dtype = act_code(A, "b200_grouped_gemm_check");
  a.d_dtype = float_code(D, "b200_grouped_gemm_check");
  a.A = A.data_ptr();
  a.a_scale = A_scale.has_value() ? A_scale->data_ptr<float>() : nullptr;
  a.B = B.data_ptr();
  a.b_scale = B_scale.has_value() ? B_scale->data_ptr() : nullptr;
  a.b_layout = static_cast<int>(b_layout);
  a.bias = bias.has_value() ? bias->data_ptr() : nullptr;
  a.bias_dtype = bias.has_value() ? float_code(*bias, "b200_grouped_gemm_check") : 0;
  a.D = D.data_ptr();
  a.rows_per_expert = rows_per_expert.data_ptr<int>();
  a.R = D.numel() / N;
  a.N = N;
  a.K = K;
  a.E = num_experts;
  a.recipe = B.scalar_type() == at::kFloat8_e4m3fn ? B200MOE_RECIPE_FP8_BLOCK
             : (B.element_size() == 1 ? B200MOE_RECIPE_MXFP4 : B200MOE_RECIPE_BF16);
  c10::cuda::CUDAGuard guard(A.device());
  check(b200moe_grouped_gemm_check(&a, cur_stream()), "b200_grouped_gemm_check");
  return D;
}

Tensor b200_dequant_weights(const Tensor& B, const Tensor& B_scale) {
  TORCH_CHECK(B.dim() == 3 && B.is_contiguous() && B_scale.is_contiguous(), "b200_dequant_weights: contiguous [E, ., .] weights expected");
  c10::cuda::CUDAGuard guard(B.device());
  Tensor out;
  int rc;
  if (B.scalar_type() == at::kFloat8_e4m3fn) {
    out = at::empty(B.sizes(), B.options().dtype(at::kBFloat16));
    rc = b200moe_dequant_weights(B200MOE_RECIPE_FP8_BLOCK, B.data_ptr(), B_scale.data_ptr(),
                                 out.data_ptr(), B.size(0), B.size(2), B.size(1), cur_stream());
  } else {
    out = at::empty({B.size(0), B.size(1), B.size(2) * 2}, B.options().dtype(at::kBFloat16));
    rc = b200moe_dequant_weights(B200MOE_RECIPE_MXFP4, B.data_ptr(), B_scale.data_ptr(),
                                 out.data_ptr(), B.size(0), B.size(1), B.size(2) * 2, cur_stream());
  }
  check(rc, "b200_dequant_weights");
  return out;
}

// recipe: "fp8" (per-expert f32 scale [E]), "mxfp8" (u8/e8m0 scale [E,K/32,N]) or "int4"
// (u8 [E,N,K/2], 16-bit/f32 scale [E,N,K/group]).  out_dtype: bf16 or f16.
Tensor b200_expand_weights(const Tensor& B, const Tensor& B_scale, const std::string& recipe,
                           at::ScalarType out_dtype) {
  TORCH_CHECK(B.dim() == 3 && B.is_contiguous() && B_scale.is_contiguous(),
              "b200_expand_weights: contiguous [E, ., .] weights expected");
  TORCH_CHECK(out_dtype == at::kBFloat16 || out_dtype == at::kHalf,
              "b200_expand_weights: bf16 or f16 output");
  c10::cuda::CUDAGuard guard(B.device());
  const int odt = out_dtype == at::kBFloat16 ? B200MOE_BF16 : B200MOE_F16;
  const int E = B.size(0);
  Tensor out;
  int rc;
  if (recipe == "int4") {
    TORCH_CHECK(B.scalar_type() == at::kByte, "b200_expand_weights: int4 weights are uint8 pairs");
    const int N = B.size(1), K = B.size(2) * 2;
    TORCH_CHECK(B_scale.dim() == 3 && B_scale.size(0) == E && B_scale.size(1) == N && B_scale.size(2) > 0 &&
                    K % B_scale.size(2) == 0,
                "b200_expand_weights: int4 scales must be [E, N, K/group]");
    const int sdt = B_scale.scalar_type() == at::kBFloat16 ? B200MOE_BF16
                    : B_scale.scalar_type() == at::kHalf   ? B200MOE_F16
                                                           : B200MOE_F32;
    TORCH_CHECK(sdt != B200MOE_F32 || B_scale.scalar_type() == at::kFloat,
                "b200_expand_weights: int4 scales must be bf16, f16 or f32");
    out = at::empty({E, N, K}, B.options().dtype(out_dtype));
    rc = b200moe_expand_weights(B200MOE_RECIPE_INT4, B.data_ptr(), B200MOE_U8, B_scale.data_ptr(), sdt,
                                K / B_scale.size(2), out.data_ptr(), odt, E, N, K, cur_stream());
  } else {
    const bool e5 = B.scalar_type() == at::kFloat8_e5m2;
    TORCH_CHECK(e5 || B.scalar_type() == at::kFloat8_e4m3fn, "b200_expand_weights: FP8 weights expected");
    const int K = B.size(1), N = B.size(2);
    out = at::empty({E, K, N}, B.options().dtype(out_dtype));
    if (recipe == "fp8") {
      TORCH_CHECK(B_scale.scalar_type() == at::kFloat && B_scale.numel() == E,
                  "b200_expand_weights: per-tensor FP8 takes one float32 scale per expert");
      rc = b200moe_expand_weights(B200MOE_RECIPE_FP8_TENSOR, B.data_ptr(), e5 ? B200MOE_E5M2 : B200MOE_E4M3,
                                  B_scale.data_ptr(), B200MOE_F32, 0, out.data_ptr(), odt, E, N, K,
                                  cur_stream());
    } else if (recipe == "mxfp8") {
      TORCH_CHECK(B_scale.element_size() == 1 && B_scale.dim() == 3 && B_scale.size(1) * 32 == K &&
                      B_scale.size(2) == N,
                  "b200_expand_weights: MXFP8 scales must be e8m0 [E, K/32, N]");
      rc = b200moe_expand_weights(B200MOE_RECIPE_MXFP8, B.data_ptr(), e5 ? B200MOE_E5M2 : B200MOE_E4M3,
                                  B_scale.data_ptr(), B200MOE_U8, 32, out.data_ptr(), odt, E, N, K,
                                  cur_stream());
    } else {
      TORCH_CHECK(false, "b200_expand_weights: unknown recipe ", recipe);
    }
  }
  check(rc, "b200_expand_weights");
  return out;
}

// ---- block-scaled (MX) grouped GEMM ------------------------------------------------

// e8m0 weight scales [E, N, K/32] -> the tensor-core order (one call per layer).
Tensor b200_mx_prepare_weight_scales(const Tensor& scales, int64_t K) {
  TORCH_CHECK(scales.dim() == 3 && scales.is_contiguous() && scales.element_size() == 1 &&
                  scales.size(2) * 32 == K,
              "b200_mx_prepare_weight_scales: e8m0 scales [E, N, K/32] expected");
  c10::cuda::CUDAGuard guard(scales.device());
  const int E = scales.size(0), N = scales.size(1);
  Tensor out = at::empty({static_cast<int64_t>(b200moe_mx_weight_scales_bytes(E, N, K))},
                         scales.options().dtype(at::kByte));
  check(b200moe_mx_prepare_weight_scales(reinterpret_cast<const uint8_t*>(scales.data_ptr()), E, N, K,
                                         out.data_ptr<uint8_t>(), cur_stream()),
        "b200_mx_prepare_weight_scales");
  return out;
}

// x [R, N] -> (e4m3 [R, N], e8m0 bytes [R, pitch]) with pitch = 16 * ceil(N / 512).
std::tuple<Tensor, Tensor> b200_quant_mxfp8(const Tensor& x) {
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.size(1) % 32 == 0,
              "b200_quant_mxfp8: contiguous [R, N] with N a multiple of 32 expected");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t R = x.size(0), N = x.size(1);
  const int64_t pitch = (N + 511) / 512 * 16;
  Tensor q = at::empty({R, N}, x.options().dtype(at::kFloat8_e4m3fn));
  Tensor sf = at::empty({R, pitch}, x.options().dtype(at::kByte));
  check(b200moe_quant_mxfp8(x.data_ptr(), float_code(x, "b200_quant_mxfp8"), q.data_ptr(),
                            sf.data_ptr<uint8_t>(), R, N, pitch, cur_stream()),
        "b200_quant_mxfp8");
  return {q, sf};
}

Tensor b200_grouped_gemm_mx(const Tensor& A, const Tensor& A_sf, const Tensor& B, const Tensor& B_sf,
                            const OptTensor& bias, Tensor D, const OptTensor& D_sf,
                            const Tensor& rows_per_expert, int64_t N, int64_t K, int64_t num_experts,
                            int64_t epilogue, double alpha, double limit) {
  const char* op = "b200_grouped_gemm_mx";
  TORCH_CHECK(A.is_contiguous() && A_sf.is_contiguous() && B.is_contiguous() && B_sf.is_contiguous() &&
                  D.is_contiguous(),
              op, ": contiguous tensors expected");
  TORCH_CHECK(A.scalar_type() == at::kFloat8_e4m3fn && A.dim() == 2 && A.size(1) == K, op,
              ": A must be float8_e4m3fn [R, K]");
  TORCH_CHECK(A_sf.element_size() == 1 && A_sf.dim() == 2 && A_sf.size(0) == A.size(0), op,
              ": A scales must be e8m0 bytes [R, pitch]");
  TORCH_CHECK(B.element_size() == 1 && B.numel() == num_experts * N * (K / 2), op,
              ": B must be packed e2m1 [E, N, K/2]");
  TORCH_CHECK(B_sf.numel() == static_cast<int64_t>(b200moe_mx_weight_scales_bytes(num_experts, N, K)), op,
              ": B scales must come from b200_mx_prepare_weight_scales");
  TORCH_CHECK(rows_per_expert.scalar_type() == at::kInt && rows_per_expert.is_contiguous() &&
                  rows_per_expert.numel() >= num_experts,
              op, ": rows_per_expert must be int32 [num_experts]");
  b200moe_mx_gemm_args a{};
  a.epilogue = static_cast<int>(epilogue);
  a.d_dtype = act_code(D, op);
  a.A = A.data_ptr();
  a.a_sf = reinterpret_cast<const uint8_t*>(A_sf.data_ptr());
  a.a_sf_pitch = A_sf.size(1);
  a.B = B.data_ptr();
  a.b_sf = reinterpret_cast<const uint8_t*>(B_sf.data_ptr());
  if (bias.has_value()) {
    TORCH_CHECK(bias->is_contiguous() && bias->numel() == num_experts * N, op, ": bias must be [E, N]");
    a.bias = bias->data_ptr();
    a.bias_dtype = float_code(*bias, op);
  }
  a.D = D.data_ptr();
  if (D_sf.has_value()) {
    TORCH_CHECK(D_sf->element_size() == 1 && D_sf->dim() == 2 && D_sf->is_contiguous() &&
                    D_sf->size(0) == A.size(0),
                op, ": output scales must be e8m0 bytes [R, pitch]");
    a.d_sf = reinterpret_cast<uint8_t*>(D_sf->data_ptr());
    a.d_sf_pitch = D_sf->size(1);
  }
  a.rows_per_expert = rows_per_expert.data_ptr<int>();
  a.R = A.size(0);
  a.N = N;
  a.K = K;
  a.E = num_experts;
  a.alpha = static_cast<float>(alpha);
  a.limit = static_cast<float>(limit);
  c10::cuda::CUDAGuard guard(A.device());
  check(b200moe_grouped_gemm_mx(&a, cur_stream()), op);
  return D;
}

int64_t b200_device_status() {
  int st = 0;
  check(b200moe_device_status(cur_stream(), &st), "b200_device_status");
  return st;
}

}  // namespace

TORCH_LIBRARY(B200MOE_NS_MOE_C, m) {
  m.def("moe_sum(Tensor input, Tensor! output, Tensor? topk_ids, Tensor? expert_map) -> ()");
  m.def(
      "moe_align_block_size(Tensor topk_ids, int num_experts, int block_size, Tensor! "
      "sorted_token_ids, Tensor! experts_ids, Tensor! num_tokens_post_pad, Tensor? "
      "maybe_expert_map) -> ()");
  m.def(
      "grouped_topk(Tensor scores, int n_group, int topk_group, int topk, bool renormalize, float "
      "routed_scaling_factor, Tensor bias, int scoring_func) -> (Tensor, Tensor)");
  m.def(
      "topk_softmax(Tensor! topk_weights, Tensor! topk_indices, Tensor! token_expert_indices, "
      "Tensor gating_output, bool renormalize, Tensor? bias, Tensor? is_padding) -> ()");
  m.def(
      "topk_sigmoid(Tensor! topk_weights, Tensor! topk_indices, Tensor! token_expert_indices, "
      "Tensor gating_output, bool renormalize, Tensor? bias, float routed_scaling_factor, Tensor? "
      "is_padding) -> ()");
  m.def(
      "moe_gather(Tensor! output, Tensor moe_output, Tensor topk_weights, Tensor "
      "unpermuted_row_to_permuted_row, int num_experts) -> ()");
  m.def(
      "b200_moe_gather_add(Tensor! output, Tensor moe_output, Tensor topk_weights, Tensor row_map, "
      "Tensor addend) -> ()");
  m.def(
      "b200_moe_gather_bounded(Tensor! output, Tensor moe_output, Tensor topk_weights, Tensor row_map, "
      "Tensor valid_tokens) -> ()");
  m.def("init_expert_map(Tensor expert_map, int num_experts, int ep_rank, int ep_size) -> ()");
  m.def(
      "moe_lora_align_block_size(Tensor topk_ids, Tensor token_lora_mapping, int num_experts, int "
      "block_size, int max_loras, int max_num_tokens_padded, int max_num_m_blocks, Tensor! "
      "sorted_token_ids, Tensor! experts_ids, Tensor! num_tokens_post_pad, Tensor! adapter_enabled, "
      "Tensor! lora_ids, Tensor? maybe_expert_map) -> ()");
  m.def(
      "batched_moe_align_block_size(int max_tokens_per_batch, int block_size, Tensor "
      "expert_num_tokens, Tensor! sorted_token_ids, Tensor! experts_ids, Tensor! "
      "num_tokens_post_pad) -> ()");
  m.def(
      "topk_softplus_sqrt(Tensor! topk_weights, Tensor! topk_indices, Tensor! "
      "token_expert_indices, Tensor gating_output, bool renormalize, float routed_scaling_factor, "
      "Tensor? correction_bias=None, Tensor? input_ids=None, Tensor? tid2eid=None, Tensor? "
      "is_padding=None) -> ()");
  m.def("reorder_mxfp_scales(Tensor A_scales, Tensor rows_per_expert, int total_padded_rows) -> Tensor");
  m.def(
      "remap_hidden_states(Tensor hidden_states, Tensor? hidden_states_scales, Tensor "
      "remapped_hidden_states, Tensor? remapped_hidden_states_scales, Tensor? expert_map, Tensor "
      "rows_per_expert, Tensor unpermuted_row_to_permuted_row, Tensor topk_ids, int "
      "total_experts_num, int local_experts_num) -> ()");
}

TORCH_LIBRARY_IMPL(B200MOE_NS_MOE_C, CUDA, m) {
  m.impl("moe_sum", &moe_sum);
  m.impl("moe_align_block_size", &moe_align_block_size);
  m.impl("grouped_topk", &grouped_topk);
  m.impl("topk_softmax", &topk_softmax);
  m.impl("topk_sigmoid", &topk_sigmoid);
  m.impl("moe_gather", &moe_gather);
  m.impl("b200_moe_gather_add", &b200_moe_gather_add);
  m.impl("b200_moe_gather_bounded", &b200_moe_gather_bounded);
  m.impl("init_expert_map", &init_expert_map);
  m.impl("batched_moe_align_block_size", &batched_moe_align_block_size);
  m.impl("moe_lora_align_block_size", &moe_lora_align_block_size);
  m.impl("topk_softplus_sqrt", &topk_softplus_sqrt);
  m.impl("reorder_mxfp_scales", &reorder_mxfp_scales);
  m.impl("remap_hidden_states", &remap_hidden_states);
}

TORCH_LIBRARY(B200MOE_NS_C, m) {
  m.def("silu_and_mul(Tensor! result, Tensor input) -> ()");
  m.def("swigluoai_and_mul(Tensor! out, Tensor input, float alpha=1.702, float limit=7.0) -> ()");
  m.def("gelu_and_mul(Tensor! out, Tensor input) -> ()");
  m.def("gelu_tanh_and_mul(Tensor! out, Tensor input) -> ()");
  m.def("situ_and_mul(Tensor! out, Tensor input, float beta=1.0, float linear_beta=-1.0) -> ()");
  m.def("relu2_no_mul(Tensor! out, Tensor! input) -> ()");
  m.def("swiglustep_and_mul(Tensor! out, Tensor input, float limit=7.0) -> ()");
  m.def(
      "b200_act_and_mul(Tensor! out, Tensor input, int act, float param0=0.0, float param1=0.0, "
      "float clamp_limit=0.0) -> ()");
  m.def(
      "per_token_group_fp8_quant(Tensor input, Tensor! output_q, Tensor! output_s, int group_size, "
      "float eps, float fp8_min, float fp8_max, bool scale_ue8m0, bool dummy_is_scale_transposed, "
      "bool dummy_is_tma_aligned) -> ()");
  m.def(
      "per_token_group_quant_mxfp4(Tensor input, Tensor! output_q, Tensor! output_s, int "
      "group_size, float eps) -> ()");
  m.def(
      "silu_and_mul_per_block_quant(Tensor! out, Tensor input, Tensor! scales, int group_size, "
      "Tensor? scale_ub=None, bool is_scale_transposed=False, bool scale_ue8m0=False) -> ()");
  m.def(
      "silu_and_mul_mxfp4_quant(Tensor! out, Tensor input, Tensor! scales, int group_size, float "
      "eps=1e-10) -> ()");
}

TORCH_LIBRARY_IMPL(B200MOE_NS_C, CUDA, m) {
  m.impl("silu_and_mul", &silu_and_mul);
  m.impl("swigluoai_and_mul", &swigluoai_and_mul);
  m.impl("gelu_and_mul", &gelu_and_mul);
  m.impl("gelu_tanh_and_mul", &gelu_tanh_and_mul);
  m.impl("situ_and_mul", &situ_and_mul);
  m.impl("relu2_no_mul", &relu2_no_mul);
  m.impl("swiglustep_and_mul", &swiglustep_and_mul);
  m.impl("b200_act_and_mul", &b200_act_and_mul);
  m.impl("per_token_group_fp8_quant", &per_token_group_fp8_quant);
  m.impl("per_token_group_quant_mxfp4", &per_token_group_quant_mxfp4);
  m.impl("silu_and_mul_per_block_quant", &silu_and_mul_per_block_quant);
  m.impl("silu_and_mul_mxfp4_quant", &silu_and_mul_mxfp4_quant);
}

TORCH_LIBRARY(B200MOE_NS_XPU_C, m) {
  m.def(
      "cutlass_grouped_gemm_interface(Tensor ptr_A, Tensor? ptr_A_scale, Tensor ptr_B, Tensor? "
      "ptr_B_scale, Tensor? ptr_bias, Tensor ptr_D, Tensor rows_per_expert, int N, int K, int "
      "num_experts) -> Tensor");
  // Extensions used by the fused layer: epilogue selection and a second weight layout.
  m.def(
      "b200_grouped_gemm(Tensor A, Tensor? A_scale, Tensor B, Tensor? B_scale, Tensor? bias, "
      "Tensor D, Tensor rows_per_expert, int N, int K, int num_experts, int epilogue, int "
      "b_layout, float alpha=1.702, float limit=7.0, Tensor? D_scale=None, Tensor? D_row_ptr=None, int "
      "a_scale_layout=0, int gated_act=0, float act_param0=0.0, float act_param1=0.0, float "
      "clamp_limit=0.0, bool scales_pow2=False) -> Tensor");
  m.def(
      "b200_grouped_gemm_check(Tensor A, Tensor? A_scale, Tensor B, Tensor? B_scale, Tensor? "
      "bias, Tensor D, Tensor rows_per_expert, int N, int K, int num_experts, int b_layout) -> "
      "Tensor");
  m.def("b200_dequant_weights(Tensor B, Tensor B_scale) -> Tensor");
  m.def("b200_expand_weights(Tensor B, Tensor B_scale, str recipe, ScalarType out_dtype) -> Tensor");
  m.def("b200_device_status() -> int");
  m.def("b200_mx_prepare_weight_scales(Tensor scales, int K) -> Tensor");
  m.def("b200_quant_mxfp8(Tensor x) -> (Tensor, Tensor)");
  m.def(
      "b200_grouped_gemm_mx(Tensor A, Tensor A_sf, Tensor B, Tensor B_sf, Tensor? bias, Tensor D, "
      "Tensor? D_sf, Tensor rows_per_expert, int N, int K, int num_experts, int epilogue, float "
      "alpha=1.702, float limit=7.0) -> Tensor");
}

TORCH_LIBRARY_IMPL(B200MOE_NS_XPU_C, CUDA, m) {
  m.impl("cutlass_grouped_gemm_interface", &cutlass_grouped_gemm_interface);
  m.impl("b200_grouped_gemm", &b200_grouped_gemm);
  m.impl("b200_grouped_gemm_check", &b200_grouped_gemm_check);
  m.impl("b200_dequant_weights", &b200_dequant_weights);
  m.impl("b200_expand_weights", &b200_expand_weights);
  m.impl("b200_mx_prepare_weight_scales", &b200_mx_prepare_weight_scales);
  m.impl("b200_quant_mxfp8", &b200_quant_mxfp8);
  m.impl("b200_grouped_gemm_mx", &b200_grouped_gemm_mx);
}

TORCH_LIBRARY_IMPL(B200MOE_NS_XPU_C, CompositeExplicitAutograd, m) {
  m.impl("b200_device_status", &b200_device_status);
}
