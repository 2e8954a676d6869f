/*
 * b200moe — C ABI of the B200 (sm_100a) fused Mixture-of-Experts kernels.
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless the
 * parameter name ends in `_host`; `stream` is a cudaStream_t passed as void*.
 * No call allocates, synchronises or creates streams.  Scratch memory is passed
 * in by the caller; its size comes from the matching *_workspace_bytes() query.
 *
 * Every function returns one of the B200MOE_* status codes below and never
 * throws or aborts.  Citations name the operator of vllm-xpu-kernels that an
 * entry point stands in for (path inside that project).
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_OK 0
#define B200MOE_INVALID_ARG (-1)
#define B200MOE_UNSUPPORTED (-2)
#define B200MOE_WORKSPACE_TOO_SMALL (-3)
#define B200MOE_CUDA_ERROR (-4)
#define B200MOE_TIMEOUT (-5)

/* element types */
#define B200MOE_F32 0
#define B200MOE_F16 1
#define B200MOE_BF16 2
#define B200MOE_E4M3 3
#define B200MOE_I32 4
#define B200MOE_I64 5
#define B200MOE_U32 6
#define B200MOE_U8 7
#define B200MOE_E2M1X2 8 /* two e2m1 per byte, low nibble = even element */
#define B200MOE_E5M2 9

/* weight recipes of the grouped GEMM */
#define B200MOE_RECIPE_BF16 0     /* B [E,K,N] bf16/f16, no scales                     */
#define B200MOE_RECIPE_FP8_BLOCK 1 /* B [E,K,N] e4m3, scales f32 [E,K/128,N/128]        */
                                   /* (a_scale and b_scale both NULL: unit scales, a plain
                                      e4m3 x e4m3 contraction; store epilogue only)      */
#define B200MOE_RECIPE_MXFP4 2    /* B [E,N,K/2] e2m1x2, scales e8m0 u8 [E,N,K/32]     */
/* 16-bit-activation recipes, taken by b200moe_expand_weights only: */
#define B200MOE_RECIPE_FP8_TENSOR 3 /* B [E,K,N] e4m3|e5m2, one f32 scale per expert [E] */
#define B200MOE_RECIPE_MXFP8 4      /* B [E,K,N] e4m3|e5m2, scales e8m0 u8 [E,K/32,N]    */
#define B200MOE_RECIPE_INT4 5       /* B [E,N,K/2] u8 (value = nibble - 8, low nibble =
                                       even k), scales bf16|f16|f32 [E,N,K/group]         */

#define B200MOE_B_LAYOUT_KN 0
#define B200MOE_B_LAYOUT_NK 1

/* layout of the per-token-group-128 activation scales of an e4m3 A */
#define B200MOE_A_SCALE_ROW_MAJOR 0    /* [R, K/128], what per_token_group_fp8_quant writes   */
#define B200MOE_A_SCALE_KBLOCK_MAJOR 1 /* [K/128, R]: also selects the decode-regime kernel
                                          (weights on the M side of the MMA, 32 tokens per
                                          tile); FP8_BLOCK recipe, EPI_STORE / EPI_SILU_MUL,
                                          16-bit output, or e4m3 + d_scale with SILU_MUL     */
#define B200MOE_A_SCALE_ROW_MAJOR_DECODE 2 /* [R, K/128] as ROW_MAJOR, and the decode-regime
                                          kernel as KBLOCK_MAJOR                              */

/* epilogues of the grouped GEMM */
#define B200MOE_EPI_STORE 0        /* D = acc (+bias), dtype of D                       */
#define B200MOE_EPI_SILU_MUL 1     /* D[:, j] = silu(acc[:, j]) * acc[:, N/2 + j]       */
#define B200MOE_EPI_SWIGLU_OAI 2   /* D[:, j] from acc[:, 2j] (gate), acc[:, 2j+1] (up) */

const char* b200moe_version(void);
/* Text for a status code. */
const char* b200moe_status_string(int status);
/* Last CUDA error text seen by this library on the calling thread. */
const char* b200moe_last_error(void);
/* Kernels this library has enqueued in this process so far (all threads, all
 * devices): a benchmark reads it before and after a timed region to report how
 * many of its launches were this library's. */
long long b200moe_launch_count(void);

/* ---- routing ---------------------------------------------------------- */

/* topk_softmax (csrc/moe/torch_bindings.cpp:62-66, csrc/moe/topk.cpp:889-941).
 * logits [T,E] of `in_dtype` (F32/F16/BF16); bias f32 [E] or NULL; is_padding
 * u8 [T] or NULL.  Outputs: weights f32 [T,k]; ids [T,k] of `ids_dtype`
 * (I32/U32/I64); src_rows i32 [T,k] (= j*T + t) or NULL. */
int b200moe_topk_softmax(const void* logits, int in_dtype, int T, int E, int k,
                         int renormalize, const float* bias,
                         const uint8_t* is_padding, float* weights, void* ids,
                         int ids_dtype, int32_t* src_rows, void* stream);

/* topk_sigmoid (csrc/moe/torch_bindings.cpp:68-72, csrc/moe/topk.cpp:943-997). */
int b200moe_topk_sigmoid(const void* logits, int in_dtype, int T, int E, int k,
                         int renormalize, const float* bias,
                         float routed_scaling_factor, const uint8_t* is_padding,
                         float* weights, void* ids, int ids_dtype,
                         int32_t* src_rows, void* stream);

/* grouped_topk (csrc/moe/torch_bindings.cpp:56-60, csrc/moe/grouped_topk.cpp:825-942).
 * scores [T,E] of `in_dtype`; bias [E] of `bias_dtype` (F32/F16/BF16);
 * scoring_func 0 = scores are already activated, 1 = sigmoid here.
 * Outputs: values f32 [T,k], ids i32 [T,k]. */
int b200moe_grouped_topk(const void* scores, int in_dtype, const void* bias,
                         int bias_dtype, int T, int E, int n_group,
                         int topk_group, int k, int renormalize,
                         float routed_scaling_factor, int scoring_func,
                         float* values, int32_t* ids, void* stream);

/* topk_softplus_sqrt (csrc/moe/torch_bindings.cpp:73-78,
 * csrc/moe/topk_softplus_sqrt_kernels.cpp:742-817): scores = sqrt(softplus(x)) in
 * fp32; selection and weights as topk_sigmoid.  With `tid2eid` (i32 [vocab, k])
 * and `input_ids` [T] the experts of row t are tid2eid[input_ids[t]] (hash
 * routing) and only the weights come from the scores. */
int b200moe_topk_softplus_sqrt(const void* logits, int in_dtype, int T, int E, int k,
                               int renormalize, float routed_scaling_factor,
                               const float* bias, const void* input_ids,
                               int input_ids_dtype, const int32_t* tid2eid,
                               const uint8_t* is_padding, float* weights, void* ids,
                               int ids_dtype, int32_t* src_rows, void* stream);

/* ---- permutation ------------------------------------------------------ */

/* moe_align_block_size (csrc/moe/torch_bindings.cpp:14-20,
 * csrc/moe/moe_align_sum_kernels.cpp:1034-1181).  topk_ids: `numel` entries of
 * `ids_dtype`; expert_map i32 [num_experts] or NULL.  sorted_token_ids has
 * `sorted_capacity` entries, expert_ids `blocks_capacity`.  Order inside an
 * expert is ascending flat index (stable), so the result is reproducible. */
size_t b200moe_moe_align_block_size_workspace_bytes(int64_t numel, int num_experts);
int b200moe_moe_align_block_size(const void* topk_ids, int ids_dtype,
                                 int64_t numel, int num_experts, int block_size,
                                 const int32_t* expert_map,
                                 int32_t* sorted_token_ids, int64_t sorted_capacity,
                                 int32_t* expert_ids, int64_t blocks_capacity,
                                 int32_t* num_tokens_post_pad, void* workspace,
                                 size_t workspace_bytes, void* stream);

/* moe_align_block_size for hosts that are not allowed to allocate device memory
 * around the call: an inference server that handed all of HBM to its own pools at
 * start-up, a plug-in interface whose contract forbids cudaMalloc on the request
 * path, a C host with no allocator to lend a workspace from.  It has no
 * counterpart in vllm-xpu-kernels (whose operator allocates its scratch with
 * torch).  Same arguments and results as b200moe_moe_align_block_size minus the
 * workspace: the scratch is a 256 KiB array built into the library (every GPU
 * that loads the library carries it until the process ends).
 *   Limit: ceil(numel / 2048) * num_experts <= 65536; larger problems get
 *   B200MOE_WORKSPACE_TOO_SMALL and a message in b200moe_last_error().
 *   The first call on each device looks the array's device address up once, with
 *   that device current; make that first call before any stream capture.
 *   All calls on a device share the array: two calls whose kernels can overlap
 *   on the GPU (different streams) race; calls on one stream are safe, and
 *   nothing needs clearing between them.
 * Calls no cudaMalloc / cudaFree or allocating library routine. */
int b200moe_moe_align_block_size_static(const void* topk_ids, int ids_dtype,
                                        int64_t numel, int num_experts,
                                        int block_size, const int32_t* expert_map,
                                        int32_t* sorted_token_ids,
                                        int64_t sorted_capacity, int32_t* expert_ids,
                                        int64_t blocks_capacity,
                                        int32_t* num_tokens_post_pad, void* stream);

/* batched_moe_align_block_size (csrc/moe/torch_bindings.cpp:24-33,
 * csrc/moe/moe_align_sum_kernels.cpp:1183-1222): batch b owns token slots
 * [b*max_tokens, b*max_tokens + n_b); sorted_ids has ceil(max_tokens/bs)*bs*B
 * entries (sentinel B*max_tokens), block_ids one entry per block (-1 unused). */
int b200moe_batched_moe_align_block_size(int max_tokens_per_batch, int block_size,
                                         const int32_t* batch_num_tokens,
                                         int num_batches, int32_t* sorted_ids,
                                         int32_t* block_ids,
                                         int32_t* num_tokens_post_pad, void* stream);

/* reorder_mxfp_scales (csrc/moe/torch_bindings.cpp:103-106,
 * csrc/moe/reorder_mxfp_scales.cpp:174-234): e8m0 scales [total_rows, scale_k],
 * experts back to back -> per expert [scale_k, rows padded to 4], written into
 * `out` (total_padded_rows * scale_k bytes; the tail is zero-filled). */
int b200moe_reorder_mxfp_scales(const uint8_t* scales, const int32_t* rows_per_expert,
                                int num_experts, int scale_k, int64_t total_padded_rows,
                                uint8_t* out, void* stream);

/* init_expert_map (csrc/moe/torch_bindings.cpp:86-91, csrc/moe/init_expert_map.cpp:78-95). */
int b200moe_init_expert_map(int32_t* expert_map, int num_local_experts,
                            int ep_rank, int ep_size, void* stream);

/* remap_hidden_states (csrc/moe/torch_bindings.cpp:92-101,
 * csrc/moe/remap_hidden_states.cpp:415-568).  Copies row t of `hidden`
 * (row_bytes bytes, a multiple of 16) and of `scales` (scale_row_bytes, may be
 * 0/NULL) to the permuted row of every local (t, j); rows_per_expert i32
 * [local_experts] is ADDED to (the caller zeroes it, as the reference's caller
 * does); row_map i32 [T,k] gets the permuted row or -1.  Stable. */
size_t b200moe_remap_hidden_states_workspace_bytes(int T, int k, int local_experts);
int b200moe_remap_hidden_states(const void* hidden, const void* scales,
                                void* remapped, void* remapped_scales,
                                int64_t row_bytes, int64_t scale_row_bytes,
                                const void* topk_ids, int ids_dtype,
                                const int32_t* expert_map, int T, int k,
                                int total_experts, int local_experts,
                                int32_t* rows_per_expert, int32_t* row_map,
                                void* workspace, size_t workspace_bytes,
                                void* stream);

/* moe_gather (csrc/moe/torch_bindings.cpp:81-85, csrc/moe/moe_gather.cpp:162-205).
 * out[t,:] = sum_j w[t,j] * y[row_map[t,j],:] (fp32 accumulate, -1 skipped). */
int b200moe_moe_gather(void* out, const void* y, int dtype, const float* weights,
                       const int32_t* row_map, int T, int k, int H, void* stream);

/* moe_gather with one more source row per token, weight 1: out[t,:] = addend[t,:] +
 * sum_j w[t,j] * y[row_map[t,j],:], one rounding.  The combine of a layer with a
 * shared expert (every token goes through it, as in the DeepSeek-V3 layer); the
 * reference project has no shared-expert operator, its moe_gather
 * (csrc/moe/moe_gather.cpp:162-205) is the routed part of this.  `out` may be
 * `addend`. */
int b200moe_moe_gather_add(void* out, const void* y, int dtype, const float* weights,
                           const int32_t* row_map, const void* addend, int T, int k,
                           int H, void* stream);

/* moe_gather over a token buffer sized for the worst case: only the first
 * *num_valid_tokens (i32 on the device) rows of `out` are computed and written;
 * the rest of `out` is left as it was.  Used on the receiving side of the
 * expert-parallel token exchange, where the number of tokens that arrived is
 * known on the device only. */
int b200moe_moe_gather_bounded(void* out, const void* y, int dtype, const float* weights,
                               const int32_t* row_map, const int32_t* num_valid_tokens,
                               int T, int k, int H, void* stream);

/* moe_sum (csrc/moe/torch_bindings.cpp:7-10, csrc/moe/moe_align_sum_kernels.cpp:1224-1372).
 * out[t,:] = sum_j in[t,j,:]; with topk_ids, slots with id < 0 or
 * expert_map[id] < 0 are skipped. */
int b200moe_moe_sum(const void* in, void* out, int dtype, int T, int k, int H,
                    const void* topk_ids, int ids_dtype,
                    const int32_t* expert_map, void* stream);

/* moe_lora_align_block_size (csrc/moe/torch_bindings.cpp:36-50,
 * csrc/moe/moe_align_sum_kernels.cpp:1374-1549; slot guards :806-812): one
 * alignment per LoRA adapter slot.  For every entry s of lora_ids[max_loras+1]
 * that is in [0, max_loras) and has adapter_enabled[s] != 0, the tokens t with
 * token_lora_mapping[t] == s are grouped by expert exactly like
 * moe_align_block_size into row s of sorted_token_ids [max_loras,
 * max_num_tokens_padded] (padding value num_tokens*topk), expert_ids
 * [max_loras, max_num_m_blocks] (-1 after the last used block) and
 * num_tokens_post_pad [max_loras].  Rows of other slots are not written.
 * expert_map, when given, maps the id before grouping (-1 drops the entry). */
int b200moe_moe_lora_align_block_size(
    const void* topk_ids, int ids_dtype, int64_t num_tokens, int topk,
    const int32_t* token_lora_mapping, int num_experts, int block_size,
    int max_loras, int64_t max_num_tokens_padded, int64_t max_num_m_blocks,
    int32_t* sorted_token_ids, int32_t* expert_ids, int32_t* num_tokens_post_pad,
    const int32_t* adapter_enabled, const int32_t* lora_ids,
    const int32_t* expert_map, void* stream);

/* ---- gated activations and activation quantisation --------------------- */

/* silu_and_mul (csrc/torch_bindings.cpp:80-81, csrc/activation.cpp:546-553). in [R,2d] -> out [R,d]. */
int b200moe_silu_and_mul(void* out, const void* in, int dtype, int64_t R, int d,
                         void* stream);
/* swigluoai_and_mul (csrc/torch_bindings.cpp:192-196, csrc/activation.cpp:737-743). */
int b200moe_swigluoai_and_mul(void* out, const void* in, int dtype, int64_t R,
                              int d, float alpha, float limit, void* stream);

/* The remaining activations the layer can be built with
 * (vllm_xpu_kernels/fused_moe_interface.py:133-154): gelu_and_mul,
 * gelu_tanh_and_mul (csrc/torch_bindings.cpp:112-116, csrc/activation.cpp:51-72),
 * swiglustep_and_mul(limit = param0) (:202-206, activation.cpp:297-311),
 * situ_and_mul(beta = param0, linear_beta = param1; <= 0 leaves `up` linear)
 * (:118-121, activation.cpp:313-323, argument checks :777-780),
 * relu2_no_mul (:198-200, activation.cpp:44-49).  Gated forms: in [R,2d] ->
 * out [R,d], gate = first half.  RELU2_NO_MUL: in [R,d] -> out [R,d].
 * clamp_limit > 0 first clamps gate to <= limit and up to [-limit, limit], the
 * layer's gemm1_clamp_limit (fused_moe_interface.py:436-441) without a pass of
 * its own; for RELU2_NO_MUL the first d/2 columns count as gate. */
#define B200MOE_ACT_SILU 0
#define B200MOE_ACT_GELU 1
#define B200MOE_ACT_GELU_TANH 2
#define B200MOE_ACT_SWIGLUSTEP 3
#define B200MOE_ACT_SITU 4
#define B200MOE_ACT_RELU2_NO_MUL 5
int b200moe_act_and_mul(void* out, const void* in, int dtype, int64_t R, int d,
                        int act, float param0, float param1, float clamp_limit,
                        void* stream);

/* per_token_group_fp8_quant (csrc/torch_bindings.cpp:175-182,
 * csrc/quantization/fp8/fp8_quant.cpp:724-849).  scales f32, element (r, g) at
 * r*scale_stride_row + g*scale_stride_group. */
int b200moe_per_token_group_fp8_quant(const void* in, int dtype, void* out_q,
                                      float* out_s, int64_t R, int N,
                                      int group_size, float eps, float fp8_min,
                                      float fp8_max, int scale_ue8m0,
                                      int64_t scale_stride_row,
                                      int64_t scale_stride_group, void* stream);

/* per_token_group_quant_mxfp4 (csrc/torch_bindings.cpp:185-189,
 * csrc/quantization/fp4/mxfp4_quant.cpp:24-126).  group_size must be 32. */
int b200moe_per_token_group_quant_mxfp4(const void* in, int dtype, uint8_t* out_q,
                                        float* out_s, int64_t R, int N,
                                        int group_size, float eps,
                                        int64_t scale_stride_row,
                                        int64_t scale_stride_group, void* stream);

/* silu_and_mul_per_block_quant (csrc/torch_bindings.cpp:89-101,
 * csrc/quantization/fused_kernels/fused_silu_mul_block_quant.cpp). in [R,2d]. */
int b200moe_silu_mul_block_quant(const void* in, int dtype, void* out_q,
                                 float* out_s, int64_t R, int d, int group_size,
                                 const float* scale_ub, int scale_ue8m0,
                                 int64_t scale_stride_row,
                                 int64_t scale_stride_group, void* stream);

/* silu_and_mul_mxfp4_quant (csrc/torch_bindings.cpp:103-107,
 * csrc/quantization/fused_kernels/fused_silu_mul_mxfp4_quant.cpp). */
int b200moe_silu_mul_mxfp4_quant(const void* in, int dtype, uint8_t* out_q,
                                 float* out_s, int64_t R, int d, int group_size,
                                 float eps, void* stream);

/* ---- grouped GEMM ------------------------------------------------------ */

typedef struct b200moe_gemm_args {
  int recipe;        /* B200MOE_RECIPE_*                                        */
  int epilogue;      /* B200MOE_EPI_*                                           */
  int a_dtype;       /* BF16/F16 (any recipe) or E4M3 (FP8_BLOCK with a_scale)  */
  int d_dtype;       /* BF16/F16, or E4M3 with d_scale (fused group-128 quant)  */
  const void* A;     /* [R,K] rows grouped by expert, back to back              */
  const float* a_scale; /* [R,K/128] f32 when a_dtype == E4M3, else NULL        */
  const void* B;     /* per recipe                                              */
  int b_layout;      /* BF16 recipe only: B200MOE_B_LAYOUT_KN [E,K,N] (the operator's
                        layout) or B200MOE_B_LAYOUT_NK [E,N,K]                    */
  const void* b_scale;
  const void* bias;  /* [E,N] of bias_dtype or NULL                             */
  int bias_dtype;
  void* D;           /* [R,N] or [R,N/2] for the gated epilogues                */
  float* d_scale;    /* [R,(N/2)/128] f32 when d_dtype == E4M3 (FP8_BLOCK recipe
                        with EPI_SILU_MUL only: the activation leaves the GEMM
                        already quantised per token per 128 columns)             */
  const int32_t* rows_per_expert; /* i32 [E], device                           */
  int64_t R;         /* rows of A (upper bound on sum(rows_per_expert))         */
  int N, K, E;
  float alpha, limit; /* SWIGLU_OAI parameters                                  */
  const int64_t* d_row_ptr; /* optional, EPI_STORE only: device table with one
                        address per row of A; row r of the result is stored at
                        that address (N elements) instead of D + r*N.  The
                        addresses may be peer-mapped memory of other GPUs: this
                        is how the expert-parallel combine leaves the GEMM.      */
  int a_scale_layout; /* B200MOE_A_SCALE_*                                       */
  int gated_act;     /* EPI_SILU_MUL only: B200MOE_ACT_SILU (0, the default), GELU,
                        GELU_TANH, SWIGLUSTEP (act_param0 = its limit) or SITU
                        (act_param0 = beta, act_param1 = linear beta or <= 0) applied to the
                        gate half in the epilogue, fp32, one rounding at the store   */
  float act_param0, act_param1;
  float clamp_limit; /* > 0: the layer's gemm1 clamp (gate <= limit, |up| <= limit,
                        fused_moe_interface.py:436-441 of the reference) applied to the
                        accumulators before either gated epilogue; 0 = none          */
  int scales_pow2;   /* FP8_BLOCK recipe with E4M3 activations only.  1: every a_scale and
                        b_scale value is an exact power of two (what
                        per_token_group_fp8_quant(..., scale_ue8m0=True) produces, and how
                        UE8M0-scaled checkpoints store their 128x128 block scales).  The
                        scales are then applied by the tensor core itself (block-scaled MMA,
                        one accumulation phase per tile) instead of once per 128 of K in
                        registers, and the quantising epilogue writes power-of-two d_scale
                        values, so its output can feed the next GEMM the same way.  A scale
                        that is not a power of two leaves B200MOE_INVALID_ARG in the device
                        status word (b200moe_device_status).  STORE and SILU_MUL epilogues. */
} b200moe_gemm_args;

/* cutlass_grouped_gemm_interface (csrc/xpu/torch_bindings.cpp:58-67,
 * csrc/xpu/grouped_gemm/grouped_gemm_interface.cpp:12-64): for expert e with
 * rows [off_e, off_e + rows_e): D = A * B_e (+ bias_e), fp32 accumulate. */
/* Environment read per call (no effect on results): B200MOE_GEMM_SMS=n caps the persistent grid
 * (a caller overlapping other kernels with the GEMM); B200MOE_STORE_OFFLOAD=0/1 forces where
 * the block-FP8 store GEMM on CTA pairs writes its tiles from (reader warps / the two spare
 * warps through a shared-memory staging tile; default: the latter for K <= 4096);
 * B200MOE_PAIR, B200MOE_TILE_N force a tile shape (tests). */
size_t b200moe_grouped_gemm_workspace_bytes(const b200moe_gemm_args* args);
int b200moe_grouped_gemm(const b200moe_gemm_args* args, void* workspace,
                         size_t workspace_bytes, void* stream);

/* Expands quantised expert weights to bf16 once, so that later grouped-GEMM
 * calls can take the 16-bit path without a per-call workspace: FP8_BLOCK
 * [E,K,N] -> bf16 [E,K,N]; MXFP4 [E,N,K/2] -> bf16 [E,N,K] (exact).
 * Stands in for the in-register up-conversion of
 * csrc/xpu/grouped_gemm/xe_2/gemm_xe2.hpp:399-483. */
int b200moe_dequant_weights(int recipe, const void* B, const void* b_scale,
                            void* out_bf16, int E, int N, int K, void* stream);

/* One-time widening of the weight formats the reference runs with 16-bit
 * activations (W8A16 per-tensor FP8 and MXFP8, W4A16 INT4; recipe detection in
 * vllm_xpu_kernels/fused_moe_interface.py:48-83, dequantisation rules in
 * vllm_xpu_kernels/moe_utils.py:206-217 and tests/fused_moe/test_fused_moe.py:37-50):
 * out = round_to_out_dtype(value * scale), bf16 or f16, in the layout of the
 * input ([E,K,N] for the FP8 forms, [E,N,K] for INT4).  The result is the B
 * operand of a B200MOE_RECIPE_BF16 grouped GEMM.  Stands in for the in-kernel
 * up-conversion of csrc/xpu/grouped_gemm/xe_2/grouped_gemm_xe2_interface.hpp:368-523;
 * tcgen05 needs both operands in one element width. */
int b200moe_expand_weights(int recipe, const void* B, int b_dtype,
                           const void* b_scale, int scale_dtype, int group_size,
                           void* out, int out_dtype, int E, int N, int K,
                           void* stream);

/* ---- block-scaled (MX) grouped GEMM -------------------------------------------
 * The tensor-core form of the reference's MXFP4 weight recipe
 * (csrc/xpu/grouped_gemm/xe_2/gemm_xe2.hpp:249-504 `xe_gemm_4bits`, scale decode
 * :426-434; weight layout csrc/xpu/grouped_gemm/xe_2/grouped_gemm_xe2_interface.hpp:281-301):
 * B stays e2m1 [E,N,K/2] in memory; A is MXFP8 (e4m3 with one e8m0 scale per 32
 * of K, the quantisation vllm_xpu_kernels/moe_utils.py:84-109 applies to
 * activations: per_token_group_fp8_quant with group 32 and scale_ue8m0); both
 * scale sets are applied inside tcgen05.mma kind::mxf8f6f4.block_scale. */

/* Bytes of the rearranged weight scales for b200moe_grouped_gemm_mx. */
size_t b200moe_mx_weight_scales_bytes(int E, int N, int K);
/* scales: e8m0 bytes [E,N,K/32] as the operator takes them -> `out` in the order
 * the tensor core reads them (once per layer).  Plays the part of
 * reorder_mxfp_scales (csrc/moe/reorder_mxfp_scales.cpp:174-234) for the weight
 * side. */
int b200moe_mx_prepare_weight_scales(const uint8_t* scales, int E, int N, int K,
                                     uint8_t* out, void* stream);

/* MXFP8 quantisation of activations: out_q e4m3 [R,N]; out_sf e8m0 bytes, scale
 * of columns [32g, 32g+32) of row r at out_sf[r*sf_pitch + g] (sf_pitch a multiple
 * of 16 and >= 16*ceil(N/512); bytes past N/32 are not written).
 * scale = 2^ceil(log2(max(max(amax,1e-10)/448, 1/(448*512)))), q = e4m3(x / scale):
 * per_token_group_fp8_quant(group 32, scale_ue8m0) with the scale stored as its
 * exponent byte (vllm_xpu_kernels/moe_utils.py:84-109). */
int b200moe_quant_mxfp8(const void* in, int dtype, void* out_q, uint8_t* out_sf,
                        int64_t R, int N, int64_t sf_pitch, void* stream);

typedef struct b200moe_mx_gemm_args {
  int epilogue;      /* B200MOE_EPI_STORE or B200MOE_EPI_SWIGLU_OAI                 */
  int d_dtype;       /* BF16/F16; or E4M3 with d_sf (SWIGLU_OAI only): the result
                        leaves the GEMM as MXFP8, ready to be the next A          */
  const void* A;     /* e4m3 [R,K], rows grouped by expert                         */
  const uint8_t* a_sf; /* e8m0 [R, a_sf_pitch]                                      */
  int64_t a_sf_pitch;  /* multiple of 16, >= 16*ceil(K/512)                          */
  const void* B;     /* e2m1 pairs [E,N,K/2], 32-byte aligned                      */
  const uint8_t* b_sf; /* from b200moe_mx_prepare_weight_scales                      */
  const void* bias;  /* [E,N] of bias_dtype or NULL                                */
  int bias_dtype;
  void* D;           /* [R,N], or [R,N/2] for SWIGLU_OAI                           */
  uint8_t* d_sf;     /* e8m0 [R, d_sf_pitch] when d_dtype == E4M3                  */
  int64_t d_sf_pitch;
  const int32_t* rows_per_expert; /* i32 [E], device                               */
  int64_t R;
  int N, K, E;       /* K a multiple of 64, >= 128                                 */
  float alpha, limit;
} b200moe_mx_gemm_args;

int b200moe_grouped_gemm_mx(const b200moe_mx_gemm_args* args, void* stream);

/* Plain CUDA-core evaluation of the same contract, one thread per output
 * element, for checking the tensor-core path on sizes a CPU cannot reach. */
int b200moe_grouped_gemm_check(const b200moe_gemm_args* args, void* stream);

/* Launches one warp that waits, for at most `budget_cycles`, on a barrier nobody
 * arrives at: the wait gives up, B200MOE_TIMEOUT lands in the device status word
 * and the kernel returns.  A check of the give-up path without a hung GPU. */
int b200moe_selftest_wait_timeout(long long budget_cycles, void* stream);

/* Reads (and clears) the sticky device status word that bounded waits inside
 * the tensor-core kernels set when they give up; 0 = none.  Synchronises. */
int b200moe_device_status(void* stream, int* status_host);

/* ---- expert-parallel exchange over peer-mapped memory -------------------------
 * vllm-xpu-kernels has no exchange step (its expert-parallel mode masks
 * non-local experts, csrc/moe/init_expert_map.cpp:45-52, and leaves the
 * all-to-all to vLLM); these four entry points are that step for GPUs of one
 * NVLink/NVSwitch domain.  `peer_bases_host` is a HOST array of `world` device
 * addresses: the base of every rank's symmetric allocation, mapped into this
 * process.  Offsets are byte offsets inside that allocation, the same on every
 * rank.  The data entry points only enqueue kernels that write or read; the
 * cross-rank ordering between them is b200moe_ep_barrier on the same stream. */

/* Barrier over the ranks of the symmetric allocation, as one small kernel on
 * `stream`: orders everything this rank's earlier kernels on the stream wrote to
 * peer memory before the peers' later kernels, and the other way round.  The
 * allocation holds B200MOE_EP_BARRIER_CHANNELS x 16 u32 flag words at
 * `flags_offset` (zero before the first barrier, never written by the host
 * afterwards); `epochs` is this rank's own device array u32
 * [B200MOE_EP_BARRIER_CHANNELS], zero at first.  Every rank must call the
 * barriers of one channel in the same order.  The wait polls local memory and is
 * bounded: after `budget_ns` (<= 0: B200MOE_EP_BARRIER_TIMEOUT_MS from the
 * environment, default 30 s) the kernel leaves B200MOE_TIMEOUT in the device
 * status word (b200moe_device_status) and returns; later kernels then run on
 * whatever the peers have delivered so far, inside their buffers. */
#define B200MOE_EP_BARRIER_CHANNELS 4
int b200moe_ep_barrier(const int64_t* peer_bases_host, int64_t flags_offset,
                       int my_rank, int world, int channel, uint32_t* epochs,
                       int64_t budget_ns, void* stream);

/* The same protocol with all `world` ranks played by the CTAs of one
 * cooperative launch on one device (rank r's flag words at flags + r * CHANNELS *
 * 16, its epochs at epochs + r * CHANNELS), for exercising it where each rank
 * cannot have a GPU of its own; ranks in `absent_mask` never arrive. */
int b200moe_ep_barrier_emulated(uint32_t* flags, uint32_t* epochs, int world,
                                int channel, uint32_t absent_mask, int64_t budget_ns,
                                void* stream);

/* Token-level exchange (a token crosses to a rank ONCE, however many of its
 * experts live there; the receiving rank runs its local layer on the tokens it
 * got and returns one partial sum per token).  It reuses the entry points below
 * with experts_per_rank = 1 and top-k = world on the matrix this one builds:
 * hits i32 [num_tokens, world], hits[t,r] = r if any expert of token t lives on
 * rank r (ids in [r*experts_per_rank, (r+1)*experts_per_rank)), else -1. */
int b200moe_ep_rank_hits(const void* topk_ids, int ids_dtype, int num_tokens, int topk,
                         int experts_per_rank, int world, int32_t* hits, void* stream);

/* What travels with a token: side i32 [num_tokens, side_stride] = its expert ids
 * as i32, then its routing weights (f32 bits); side_stride >= 2*topk words (rounded
 * up to a multiple of 4 so that the row is a whole number of 16-byte pieces). */
int b200moe_ep_pack_routing(const void* topk_ids, int ids_dtype, const float* topk_weights,
                            int num_tokens, int topk, int side_stride, int32_t* side,
                            void* stream);

/* On the receiving rank: for the recv_total[0] (device) tokens that arrived,
 * ids_local i32 [capacity_tokens, topk] = local expert id, or -1 where the expert
 * lives on another rank, and weights f32 (0 there); rows past recv_total get -1,
 * so stale rows of the worst-case buffer are never routed. */
int b200moe_ep_unpack_routing(const int32_t* side, const int32_t* recv_total,
                              int64_t capacity_tokens, int topk, int side_stride, int my_rank,
                              int experts_per_rank, int32_t* ids_local, float* weights,
                              void* stream);

/* Writes my rows-per-global-expert (i32 [num_counts], num_counts = world *
 * experts_per_rank) into row `my_rank` of every rank's i32 [world, num_counts]
 * matrix at `counts_offset`. */
int b200moe_ep_put_counts(const int32_t* send_counts, int num_counts,
                          const int64_t* peer_bases_host, int64_t counts_offset,
                          int my_rank, int world, void* stream);

/* From the complete matrix (local copy): my_prefix i32 [E+1] (prefix of my own
 * counts = my send order), dst_start i32 [E] (first row of my rows for expert e
 * inside its owner's expert-grouped receive buffer), rows_per_expert i32
 * [experts_per_rank] (what each of my experts receives; feed it to the grouped
 * GEMMs), recv_total i32 [1]. */
int b200moe_ep_offsets(const int32_t* counts, int my_rank, int world,
                       int experts_per_rank, int32_t* my_prefix, int32_t* dst_start,
                       int32_t* rows_per_expert, int32_t* recv_total, void* stream);

/* Stores my send rows (grouped by global expert, as remap_hidden_states with no
 * expert map leaves them) and their scale rows at their final place in the
 * owners' receive buffers, and per row an i64 (my_rank << 32 | row) at
 * meta_offset. */
int b200moe_ep_push(const void* send_rows, const void* send_scales, int64_t num_rows,
                    int64_t row_bytes, int64_t scale_row_bytes, int my_rank, int world,
                    int experts_per_rank, const int32_t* my_prefix,
                    const int32_t* dst_start, const int64_t* peer_bases_host,
                    int64_t rows_offset, int64_t scales_offset, int64_t meta_offset,
                    int64_t capacity, void* stream);

/* The same placement straight from the token-major inputs, without a local
 * copy grouped by expert: for every (token t, slot s) with row_map[t,s] = i >= 0
 * and expert e = topk_ids[t,s], row t of `hidden` (and of `scales`) goes to row
 * dst_start[e] + (i - my_prefix[e]) of e's owner.  row_map and the per-expert
 * counts behind my_prefix come from b200moe_remap_hidden_states called with
 * hidden = NULL.  Rows travel as bulk asynchronous copies. */
int b200moe_ep_dispatch(const void* hidden, const void* scales, int64_t row_bytes,
                        int64_t scale_row_bytes, const void* topk_ids, int ids_dtype,
                        const int32_t* row_map, int num_tokens, int topk, int my_rank,
                        int world, int experts_per_rank, const int32_t* my_prefix,
                        const int32_t* dst_start, const int64_t* peer_bases_host,
                        int64_t rows_offset, int64_t scales_offset, int64_t meta_offset,
                        int64_t capacity, void* stream);

/* dst_addr[j] = address, in the return buffer of the rank that sent received row
 * j, of the row it came from; feed it to b200moe_gemm_args.d_row_ptr of the
 * second grouped GEMM. */
int b200moe_ep_return_table(const int64_t* meta, const int32_t* recv_total, int world,
                            const int64_t* peer_bases_host, int64_t return_offset,
                            int64_t row_bytes, int64_t* dst_addr, void* stream);

/* The other way round ("pull" combine): src_addr[i] = address, in the output
 * buffer of the rank that owns send row i's expert, where that rank's second
 * grouped GEMM leaves the row's result (row j of the buffer at out_offset, j as
 * in b200moe_ep_push; 0 if j is beyond capacity). */
int b200moe_ep_source_table(const int32_t* my_prefix, const int32_t* dst_start,
                            int64_t num_rows, int world, int experts_per_rank,
                            const int64_t* peer_bases_host, int64_t out_offset,
                            int64_t row_bytes, int64_t capacity, int64_t* src_addr,
                            void* stream);

/* moe_gather (csrc/moe/torch_bindings.cpp:81-85) over rows that live in peers'
 * memory: out[t] = sum_j weights[t,j] * row at src_addr[row_map[t,j]], fp32
 * accumulation in slot order, entries with row_map < 0 or a null address
 * skipped.  Call after a barrier that follows every rank's second GEMM. */
int b200moe_ep_gather(void* out, int dtype, const float* weights,
                      const int32_t* row_map, const int64_t* src_addr, int T, int k,
                      int H, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
