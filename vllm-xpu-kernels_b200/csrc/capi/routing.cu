// Routing kernels: softmax / sigmoid top-k and DeepSeek grouped top-k.
//
// All three are warp-level: a row's scores live in registers (expert
// e = lane + LANES*i), the k winners are found by k rounds of a butterfly
// arg-max whose order is (key descending, expert index ascending) — the order
// a stable descending sort gives — and nothing touches shared memory or a
// workspace.  Scores are computed with IEEE division and the accurate expf so
// that they agree with a plain fp32 evaluation of the same formula.
#include <math_constants.h>

#include <type_traits>

#include "common.cuh"

namespace b200moe {
namespace {

struct Best {
  float key;
  int idx;
};

__device__ __forceinline__ bool better(float ka, int ia, float kb, int ib) {
  return (ka > kb) || (ka == kb && ia < ib);
}

template <int LANES>
__device__ __forceinline__ Best group_argmax(Best b, float& payload) {
#pragma unroll
  for (int off = LANES / 2; off > 0; off >>= 1) {
    float ok = __shfl_xor_sync(0xffffffffu, b.key, off, LANES);
    int oi = __shfl_xor_sync(0xffffffffu, b.idx, off, LANES);
    float op = __shfl_xor_sync(0xffffffffu, payload, off, LANES);
    if (better(ok, oi, b.key, b.idx)) {
      b.key = ok;
      b.idx = oi;
      payload = op;
    }
  }
  return b;
}

template <int LANES>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int off = LANES / 2; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off, LANES));
  return v;
}

template <int LANES>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int off = LANES / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off, LANES);
  return v;
}

constexpr int kInvalidIdx = 0x7fffffff;

enum : int { SCORE_SOFTMAX = 0, SCORE_SIGMOID = 1, SCORE_SOFTPLUS_SQRT = 2 };

// One row per LANES threads.  SCORE selects the scoring function.  With a hash table
// (`tid2eid`, [vocab, k] expert ids) the experts of a row are looked up by its input id
// instead of being selected, and only the weights come from the scores.
template <typename T, int LANES, int VPT, int SCORE>
__global__ void __launch_bounds__(128) topk_gating_kernel(
    const T* __restrict__ logits, int num_rows, int E, int k, bool renorm,
    const float* __restrict__ bias, float scale, const uint8_t* __restrict__ is_padding,
    float* __restrict__ weights, void* __restrict__ ids, int ids_dtype,
    int32_t* __restrict__ src_rows, const void* __restrict__ input_ids, int input_ids_dtype,
    const int32_t* __restrict__ tid2eid) {
  const int rows_per_block = blockDim.x / LANES;
  const int sub = threadIdx.x % LANES;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * rows_per_block + threadIdx.x / LANES;
  const bool live = row < num_rows;
  const int64_t r = live ? row : 0;

  float s[VPT];  // unbiased score
  float key[VPT];
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int e = sub + LANES * i;
    const float x = (e < E) ? Elem<T>::to_f32(logits[r * E + e]) : -CUDART_INF_F;
    s[i] = x;
    mx = fmaxf(mx, x);
  }
  if (SCORE == SCORE_SIGMOID) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) s[i] = round_through<T>(1.0f / (1.0f + expf(-s[i])));
  } else if (SCORE == SCORE_SOFTPLUS_SQRT) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) s[i] = sqrtf(s[i] > 20.0f ? s[i] : log1pf(expf(s[i])));
  } else {
    mx = group_max<LANES>(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int e = sub + LANES * i;
      s[i] = (e < E) ? expf(s[i] - mx) : 0.f;
      sum += s[i];
    }
    sum = group_sum<LANES>(sum);
#pragma unroll
    for (int i = 0; i < VPT; ++i) s[i] = s[i] / sum;
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int e = sub + LANES * i;
    key[i] = (e < E) ? (bias ? s[i] + bias[e] : s[i]) : -CUDART_INF_F;
  }

  uint32_t taken = 0;
  float my_w = 0.f;
  int my_id = 0;
  float wsum = 0.f;
  const int64_t hash_row = tid2eid ? load_index(input_ids, input_ids_dtype, r) * k : 0;
  for (int j = 0; j < k; ++j) {
    Best b{-CUDART_INF_F, kInvalidIdx};
    float pay = 0.f;
    if (tid2eid) {
      b.idx = tid2eid[hash_row + j];
#pragma unroll
      for (int i = 0; i < VPT; ++i)
        if (sub + LANES * i == b.idx) pay = s[i];
      pay = group_sum<LANES>(pay);  // exactly one lane holds the expert's score
    } else {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int e = sub + LANES * i;
        if (e < E && !((taken >> i) & 1u) && better(key[i], e, b.key, b.idx)) {
          b.key = key[i];
          b.idx = e;
          pay = s[i];
        }
      }
      b = group_argmax<LANES>(b, pay);
      if (b.idx != kInvalidIdx && (b.idx % LANES) == sub) taken |= 1u << (b.idx / LANES);
    }
    wsum += pay;
    if (j == sub) {  // k <= LANES always holds: k <= E <= LANES when VPT == 1, k <= 32 otherwise
      my_w = pay;
      my_id = b.idx == kInvalidIdx ? 0 : b.idx;
    }
  }
  if (!live) return;
  const bool pad = is_padding != nullptr && is_padding[r] != 0;
  const float denom = (renorm && wsum > 0.f) ? wsum : 1.f;
  if (sub < k) {
    float w = renorm ? my_w / denom : my_w;
    if (SCORE != SCORE_SOFTMAX) w *= scale;
    weights[r * k + sub] = pad ? 0.f : w;
    store_index(ids, ids_dtype, r * k + sub, pad ? -1 : my_id);
    if (src_rows) src_rows[r * k + sub] = static_cast<int32_t>(sub * num_rows + r);
  }
}

template <typename T, int SCORE>
int launch_topk(const void* logits, int T_, int E, int k, int renorm, const float* bias,
                float scale, const uint8_t* pad, float* w, void* ids, int ids_dtype,
                int32_t* src_rows, cudaStream_t st, const void* input_ids = nullptr,
                int input_ids_dtype = B200MOE_I32, const int32_t* tid2eid = nullptr) {
  const T* in = reinterpret_cast<const T*>(logits);
#define LAUNCH(LANES, VPT)                                                              \
  do {                                                                                  \
    const int rows_per_block = 128 / LANES;                                             \
    const int grid = (T_ + rows_per_block - 1) / rows_per_block;                        \
    topk_gating_kernel<T, LANES, VPT, SCORE><<<grid, 128, 0, st>>>(                     \
        in, T_, E, k, renorm != 0, bias, scale, pad, w, ids, ids_dtype, src_rows,       \
        input_ids, input_ids_dtype, tid2eid);                                           \
    return launch_status("topk_gating_kernel");                                         \
  } while (0)
  if (E <= 4) LAUNCH(4, 1);
  if (E <= 8) LAUNCH(8, 1);
  if (E <= 16) LAUNCH(16, 1);
  if (E <= 32) LAUNCH(32, 1);
  if (E <= 64) LAUNCH(32, 2);
  if (E <= 128) LAUNCH(32, 4);
  if (E <= 256) LAUNCH(32, 8);
  if (E <= 512) LAUNCH(32, 16);
  if (E <= 1024) LAUNCH(32, 32);
#undef LAUNCH
  return B200MOE_UNSUPPORTED;
}

// ---- grouped top-k ---------------------------------------------------------

// One warp per token.  Expert e = lane + 32*i.  A group is a run of `per`
// consecutive experts.
template <typename T, typename TB, int VPT>
__global__ void __launch_bounds__(128) grouped_topk_kernel(
    const T* __restrict__ scores, const TB* __restrict__ bias, int num_rows, int E,
    int n_group, int topk_group, int k, bool renorm, float scale, int scoring_func,
    float* __restrict__ values, int32_t* __restrict__ ids) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= num_rows) return;  // whole warp leaves together
  const int per = E / n_group;
  constexpr bool kSameHalfType = sizeof(T) == 2 && std::is_same<T, TB>::value;

  float s[VPT];
  float key[VPT];
  uint32_t inf_in = 0;  // experts whose raw score is +-inf: they count for their group's score
                        // but are never selected (grouped_topk.cpp:659-662 of the reference)
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int e = lane + 32 * i;
    float x = 0.f, b = 0.f;
    if (e < E) {
      x = Elem<T>::to_f32(scores[row * E + e]);
      b = Elem<TB>::to_f32(bias[e]);
      if (isinf(x)) inf_in |= 1u << i;
      if (scoring_func == 1) x = round_through<T>(1.0f / (1.0f + expf(-x)));
    }
    s[i] = x;
    float kv = x + b;
    if (kSameHalfType) kv = round_through<T>(kv);
    key[i] = (e < E) ? kv : -CUDART_INF_F;
  }

  // Group score = sum of the two largest keys in the group; lane g ends up
  // holding group g's score.
  float my_group_score = -CUDART_INF_F;
  for (int g = 0; g < n_group; ++g) {
    const int lo = g * per, hi = lo + per;
    float m1 = -CUDART_INF_F, m2 = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int e = lane + 32 * i;
      if (e >= lo && e < hi) {
        const float v = key[i];
        if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float o1 = __shfl_xor_sync(0xffffffffu, m1, off);
      const float o2 = __shfl_xor_sync(0xffffffffu, m2, off);
      const float n1 = fmaxf(m1, o1);
      const float n2 = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
      m1 = n1;
      m2 = n2;
    }
    float gs = m1 + m2;
    if (kSameHalfType) gs = round_through<T>(gs);
    if (lane == g) my_group_score = gs;
  }

  // Stable top-`topk_group` over the n_group (<= 32) group scores.
  uint32_t group_mask = 0;
  float last_group_score = -CUDART_INF_F;
  {
    bool taken = lane >= n_group;
    for (int j = 0; j < topk_group; ++j) {
      Best b{taken ? -CUDART_INF_F : my_group_score, taken ? kInvalidIdx : lane};
      float pay = 0.f;
      b = group_argmax<32>(b, pay);
      last_group_score = b.idx == kInvalidIdx ? -CUDART_INF_F : b.key;
      if (b.idx == kInvalidIdx) break;
      group_mask |= 1u << b.idx;
      if (b.idx == lane) taken = true;
    }
  }
  // Fewer than `topk_group` groups with a finite score: the reference kernel gives up on the
  // row and returns experts 0..k-1 with weight 1/k each, unscaled (grouped_topk.cpp:608-624).
  if (topk_group > 0 && last_group_score == -CUDART_INF_F) {
    if (lane < k) {
      values[row * k + lane] = 1.0f / static_cast<float>(k);
      ids[row * k + lane] = lane;
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int e = lane + 32 * i;
    if (e < E && (!((group_mask >> (e / per)) & 1u) || ((inf_in >> i) & 1u))) key[i] = -CUDART_INF_F;
  }

  uint32_t taken = 0;
  float my_w = 0.f;
  int my_id = 0;
  float wsum = 0.f;
  for (int j = 0; j < k; ++j) {
    Best b{-CUDART_INF_F, kInvalidIdx};
    float pay = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int e = lane + 32 * i;
      if (e < E && !((taken >> i) & 1u) && better(key[i], e, b.key, b.idx)) {
        b.key = key[i];
        b.idx = e;
        pay = s[i];
      }
    }
    b = group_argmax<32>(b, pay);
    if (b.idx != kInvalidIdx && (b.idx & 31) == lane) taken |= 1u << (b.idx >> 5);
    wsum += pay;
    if (j == lane) {
      my_w = pay;
      my_id = b.idx == kInvalidIdx ? 0 : b.idx;
    }
  }
  if (lane < k) {
    // the reference kernel's denominator carries 1e-20 (grouped_topk.cpp:678-687): selected
    // scores that are all zero give weight 0, not NaN; invisible in fp32 otherwise
    float w = renorm ? my_w / (wsum + 1e-20f) : my_w;
    w *= scale;
    values[row * k + lane] = w;
    ids[row * k + lane] = my_id;
  }
}

template <typename T, typename TB>
int launch_grouped(const void* scores, const void* bias, int T_, int E, int n_group,
                   int topk_group, int k, int renorm, float scale, int scoring_func,
                   float* values, int32_t* ids, cudaStream_t st) {
  const int grid = (T_ + 3) / 4;
#define LAUNCH(VPT)                                                                        \
  do {                                                                                     \
    grouped_topk_kernel<T, TB, VPT><<<grid, 128, 0, st>>>(                                 \
        reinterpret_cast<const T*>(scores), reinterpret_cast<const TB*>(bias), T_, E,      \
        n_group, topk_group, k, renorm != 0, scale, scoring_func, values, ids);            \
    return launch_status("grouped_topk_kernel");                                           \
  } while (0)
  if (E <= 32) LAUNCH(1);
  if (E <= 64) LAUNCH(2);
  if (E <= 128) LAUNCH(4);
  if (E <= 256) LAUNCH(8);
  if (E <= 512) LAUNCH(16);
  if (E <= 1024) LAUNCH(32);
#undef LAUNCH
  return B200MOE_UNSUPPORTED;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_topk_softmax(const void* logits, int in_dtype, int T, int E, int k,
                                    int renormalize, const float* bias,
                                    const uint8_t* is_padding, float* weights, void* ids,
                                    int ids_dtype, int32_t* src_rows, void* stream) {
  if (T < 0 || E <= 0 || k <= 0 || k > E || !is_index_dtype(ids_dtype)) return B200MOE_INVALID_ARG;
  if (T == 0) return B200MOE_OK;
  if (!logits || !weights || !ids) return B200MOE_INVALID_ARG;
  if (k > 32 && E > 32) return B200MOE_UNSUPPORTED;
  return B200MOE_DISPATCH_FLOAT(in_dtype, [&] {
    return launch_topk<scalar_t, SCORE_SOFTMAX>(logits, T, E, k, renormalize, bias, 1.f, is_padding,
                                        weights, ids, ids_dtype, src_rows, as_stream(stream));
  });
}

extern "C" int b200moe_topk_sigmoid(const void* logits, int in_dtype, int T, int E, int k,
                                    int renormalize, const float* bias,
                                    float routed_scaling_factor, const uint8_t* is_padding,
                                    float* weights, void* ids, int ids_dtype,
                                    int32_t* src_rows, void* stream) {
  if (T < 0 || E <= 0 || k <= 0 || k > E || !is_index_dtype(ids_dtype)) return B200MOE_INVALID_ARG;
  if (T == 0) return B200MOE_OK;
  if (!logits || !weights || !ids) return B200MOE_INVALID_ARG;
  if (k > 32 && E > 32) return B200MOE_UNSUPPORTED;
  return B200MOE_DISPATCH_FLOAT(in_dtype, [&] {
    return launch_topk<scalar_t, SCORE_SIGMOID>(logits, T, E, k, renormalize, bias, routed_scaling_factor,
                                       is_padding, weights, ids, ids_dtype, src_rows,
                                       as_stream(stream));
  });
}

extern "C" int b200moe_grouped_topk(const void* scores, int in_dtype, const void* bias,
                                    int bias_dtype, int T, int E, int n_group, int topk_group,
                                    int k, int renormalize, float routed_scaling_factor,
                                    int scoring_func, float* values, int32_t* ids, void* stream) {
  if (T < 0 || E <= 0 || n_group <= 0 || n_group > 32 || E % n_group != 0 || topk_group <= 0 ||
      topk_group > n_group || k <= 0 || k > 32 || k > E || scoring_func < 0 || scoring_func > 1)
    return B200MOE_INVALID_ARG;
  if (T == 0) return B200MOE_OK;
  if (!scores || !bias || !values || !ids) return B200MOE_INVALID_ARG;
  cudaStream_t st = as_stream(stream);
  return B200MOE_DISPATCH_FLOAT(in_dtype, [&] {
    using in_t = scalar_t;
    return B200MOE_DISPATCH_FLOAT(bias_dtype, [&] {
      return launch_grouped<in_t, scalar_t>(scores, bias, T, E, n_group, topk_group, k,
                                            renormalize, routed_scaling_factor, scoring_func,
                                            values, ids, st);
    });
  });
}

extern "C" int b200moe_topk_softplus_sqrt(const void* logits, int in_dtype, int T, int E, int k,
                                          int renormalize, float routed_scaling_factor,
                                          const float* bias, const void* input_ids,
                                          int input_ids_dtype, const int32_t* tid2eid,
                                          const uint8_t* is_padding, float* weights, void* ids,
                                          int ids_dtype, int32_t* src_rows, void* stream) {
  if (T < 0 || E <= 0 || k <= 0 || k > E || !is_index_dtype(ids_dtype)) return B200MOE_INVALID_ARG;
  if ((tid2eid != nullptr) != (input_ids != nullptr)) return B200MOE_INVALID_ARG;
  if (tid2eid && !is_index_dtype(input_ids_dtype)) return B200MOE_INVALID_ARG;
  if (T == 0) return B200MOE_OK;
  if (!logits || !weights || !ids) return B200MOE_INVALID_ARG;
  if (k > 32 && E > 32) return B200MOE_UNSUPPORTED;
  return B200MOE_DISPATCH_FLOAT(in_dtype, [&] {
    return launch_topk<scalar_t, SCORE_SOFTPLUS_SQRT>(
        logits, T, E, k, renormalize, bias, routed_scaling_factor, is_padding, weights, ids,
        ids_dtype, src_rows, as_stream(stream), input_ids, input_ids_dtype, tid2eid);
  });
}
