// Gated activations and per-token-group activation quantisation (FP8 e4m3 and
// MXFP4 e2m1), stand-alone and fused.
//
// All kernels stream: a thread owns 8 consecutive elements (one or two 16-byte
// loads), a quantisation group is 4..32 neighbouring lanes of one warp, and the
// group maximum is a segmented xor-shuffle — no shared memory, no second pass
// over the data.  Math is plain IEEE fp32 (no fast-math) so the scale formulas
// give the same bits as a straightforward fp32 evaluation.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kVec = 8;

__device__ __forceinline__ float silu_f32(float g) { return g / (1.0f + expf(-g)); }

template <typename T>
__global__ void __launch_bounds__(256) silu_and_mul_kernel(T* __restrict__ out,
                                                           const T* __restrict__ in, int64_t R,
                                                           int d) {
  constexpr int V = 16 / sizeof(T);
  const int64_t chunks_per_row = d / V;
  const int64_t total = R * chunks_per_row;
  for (int64_t c = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; c < total;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = c / chunks_per_row, col = (c % chunks_per_row) * V;
    float g[V], u[V], o[V];
    load_f32<T, V>(in + r * 2 * d + col, g);
    load_f32<T, V>(in + r * 2 * d + d + col, u);
#pragma unroll
    for (int i = 0; i < V; ++i) o[i] = round_through<T>(silu_f32(g[i])) * u[i];
    store_f32<T, V>(out + r * d + col, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) silu_and_mul_scalar_kernel(T* __restrict__ out,
                                                                  const T* __restrict__ in,
                                                                  int64_t R, int d) {
  const int64_t total = R * d;
  for (int64_t c = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; c < total;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = c / d, col = c % d;
    const float g = Elem<T>::to_f32(in[r * 2 * d + col]);
    const float u = Elem<T>::to_f32(in[r * 2 * d + d + col]);
    out[c] = Elem<T>::from_f32(round_through<T>(silu_f32(g)) * u);
  }
}

__device__ __forceinline__ float swiglu_oai(float g, float u, float alpha, float limit) {
  g = fminf(g, limit);
  u = fmaxf(fminf(u, limit), -limit);
  return (u + 1.0f) * (g * (1.0f / (1.0f + expf(-g * alpha))));
}

template <typename T>
__global__ void __launch_bounds__(256) swigluoai_kernel(T* __restrict__ out,
                                                        const T* __restrict__ in, int64_t R, int d,
                                                        float alpha, float limit) {
  // 2 outputs per thread from one 4-element (or 2x2) read when possible.
  const int64_t total = R * d;
  for (int64_t c = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; c < total;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float v[2];
    load_f32<T, 2>(in + 2 * c, v);
    out[c] = Elem<T>::from_f32(swiglu_oai(v[0], v[1], alpha, limit));
  }
}

// ---- the other activations of the fused-MoE layer -----------------------------
// One kernel for every "act(first half) * second half" flavour, with the optional
// clamp the layer applies to the first GEMM's output (gate <= limit, |up| <= limit)
// folded in, so the clamp is not a separate pass over [R, 2d].
//   SILU, GELU, GELU_TANH  act(gate) is rounded to T before the product (the reference
//                          evaluates act in T and multiplies in T)
//   SWIGLUSTEP, SITU       fp32 throughout, one rounding
//   RELU2_NO_MUL           not gated: out[r, c] = relu(in[r, c])^2 over all `d` columns
template <typename T>
__device__ __forceinline__ float gated_act(int act, float g, float u, float p0, float p1) {
  switch (act) {
    case B200MOE_ACT_SILU:
      return round_through<T>(silu_f32(g)) * u;
    case B200MOE_ACT_GELU:
      return round_through<T>(g * 0.5f * (1.0f + erff(g * 0.70710678118654752440f))) * u;
    case B200MOE_ACT_GELU_TANH: {
      const float inner = 0.79788456080286535588f * (g + 0.044715f * (g * g * g));
      return round_through<T>(0.5f * g * (1.0f + tanhf(inner))) * u;
    }
    case B200MOE_ACT_SWIGLUSTEP: {
      const float sg = fminf(silu_f32(g), p0);
      return sg * fmaxf(fminf(u, p0), -p0);
    }
    case B200MOE_ACT_SITU: {
      const float ag = p0 * tanhf(g / p0) / (1.0f + expf(-g));
      const float au = p1 > 0.0f ? p1 * tanhf(u / p1) : u;
      return ag * au;
    }
    default:
      return 0.0f;
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256) act_and_mul_kernel(T* __restrict__ out,
                                                          const T* __restrict__ in, int64_t R,
                                                          int d, int act, float p0, float p1,
                                                          float clamp) {
  const int64_t chunks_per_row = d / V;
  const int64_t total = R * chunks_per_row;
  for (int64_t c = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; c < total;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = c / chunks_per_row, col = (c % chunks_per_row) * V;
    float g[V], u[V], o[V];
    load_f32<T, V>(in + r * 2 * d + col, g);
    load_f32<T, V>(in + r * 2 * d + d + col, u);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      if (clamp > 0.0f) {
        g[i] = round_through<T>(fminf(g[i], clamp));
        u[i] = round_through<T>(fmaxf(fminf(u[i], clamp), -clamp));
      }
      o[i] = gated_act<T>(act, g[i], u[i], p0, p1);
    }
    store_f32<T, V>(out + r * d + col, o);
  }
}

// relu(x)^2 over [R, d]; columns below `split` take the gate clamp, the rest the up clamp.
template <typename T, int V>
__global__ void __launch_bounds__(256) relu2_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                    int64_t R, int d, float clamp, int split) {
  const int64_t chunks_per_row = d / V;
  const int64_t total = R * chunks_per_row;
  for (int64_t c = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; c < total;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = c / chunks_per_row, col = (c % chunks_per_row) * V;
    float x[V], o[V];
    load_f32<T, V>(in + r * d + col, x);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float v = x[i];
      if (clamp > 0.0f) {
        v = fminf(v, clamp);
        if (col + i >= split) v = fmaxf(v, -clamp);
        v = round_through<T>(v);
      }
      const float rl = v > 0.0f ? v : 0.0f;
      o[i] = rl * rl;
    }
    store_f32<T, V>(out + r * d + col, o);
  }
}

// ---- group quantisation ---------------------------------------------------

__device__ __forceinline__ float round_up_pow2(float s) {
  return exp2f(ceilf(log2f(fmaxf(fabsf(s), 1e-10f))));
}

template <int LANES>
__device__ __forceinline__ float seg_max(float v) {
#pragma unroll
  for (int off = 1; off < LANES; off <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

__device__ __forceinline__ float seg_max_dyn(float v, int lanes) {
  for (int off = 1; off < lanes; off <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

__device__ __forceinline__ uint8_t e2m1_code(float x) {
  const float a = fabsf(x);
  const int code = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) +
                   (a > 3.5f) + (a > 5.0f);
  return static_cast<uint8_t>(code | (x < 0.0f ? 8 : 0));
}

// Source of 8 fp32 values for chunk c: either a plain tensor or silu(g)*u.
template <typename T, bool SILU>
__device__ __forceinline__ void fetch8(const T* __restrict__ in, int64_t r, int col, int N,
                                       float (&x)[kVec]) {
  if (SILU) {
    float g[kVec], u[kVec];
    if (sizeof(T) == 4) {
      load_f32<T, 4>(in + r * 2 * N + col, *reinterpret_cast<float(*)[4]>(g));
      load_f32<T, 4>(in + r * 2 * N + col + 4, *reinterpret_cast<float(*)[4]>(g + 4));
      load_f32<T, 4>(in + r * 2 * N + N + col, *reinterpret_cast<float(*)[4]>(u));
      load_f32<T, 4>(in + r * 2 * N + N + col + 4, *reinterpret_cast<float(*)[4]>(u + 4));
    } else {
      load_f32<T, kVec>(in + r * 2 * N + col, g);
      load_f32<T, kVec>(in + r * 2 * N + N + col, u);
    }
#pragma unroll
    for (int i = 0; i < kVec; ++i) x[i] = silu_f32(g[i]) * u[i];
  } else {
    if (sizeof(T) == 4) {
      load_f32<T, 4>(in + r * N + col, *reinterpret_cast<float(*)[4]>(x));
      load_f32<T, 4>(in + r * N + col + 4, *reinterpret_cast<float(*)[4]>(x + 4));
    } else {
      load_f32<T, kVec>(in + r * N + col, x);
    }
  }
}

// FP8 e4m3 group quantisation.  DIVIDE selects q = x / s (fused SiLU op)
// versus q = x * (1/s) (stand-alone op).
template <typename T, bool SILU, bool DIVIDE>
__global__ void __launch_bounds__(256) group_quant_fp8_kernel(
    const T* __restrict__ in, uint8_t* __restrict__ out_q, float* __restrict__ out_s, int64_t R,
    int N, int group_size, float eps, float fp8_min, float fp8_max, bool ue8m0,
    const float* __restrict__ scale_ub, int64_t ss_row, int64_t ss_group) {
  const int lanes = group_size / kVec;
  const int64_t chunks_per_row = N / kVec;
  const int64_t total = R * chunks_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const float min_scale = 1.0f / (fp8_max * 512.0f);
  for (int64_t base = blockIdx.x * static_cast<int64_t>(blockDim.x); base < total; base += stride) {
    const int64_t c = base + threadIdx.x;
    const bool live = c < total;
    const int64_t r = live ? c / chunks_per_row : 0;
    const int col = live ? static_cast<int>(c % chunks_per_row) * kVec : 0;
    float x[kVec];
    float amax = 0.f;
    if (live) {
      fetch8<T, SILU>(in, r, col, N, x);
#pragma unroll
      for (int i = 0; i < kVec; ++i) amax = fmaxf(amax, fabsf(x[i]));
    }
    amax = seg_max_dyn(amax, lanes);
    float s = SILU ? amax / fp8_max : fmaxf(amax, eps) / fp8_max;
    s = fmaxf(s, min_scale);
    if (scale_ub) s = fmaxf(fminf(s, *scale_ub), min_scale);
    if (ue8m0) s = round_up_pow2(s);
    if (!live) continue;
    if ((threadIdx.x & 31) % lanes == 0) out_s[r * ss_row + (col / group_size) * ss_group] = s;
    const float inv = 1.0f / s;
    uint8_t q[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      float y = DIVIDE ? x[i] / s : x[i] * inv;
      y = fmaxf(fp8_min, fminf(y, fp8_max));
      q[i] = f32_to_e4m3(y);
    }
    *reinterpret_cast<uint2*>(out_q + r * N + col) = *reinterpret_cast<uint2*>(q);
  }
}

// MXFP4 (group of 32 = 4 lanes).
template <typename T, bool SILU>
__global__ void __launch_bounds__(256) group_quant_mxfp4_kernel(
    const T* __restrict__ in, uint8_t* __restrict__ out_q, float* __restrict__ out_s, int64_t R,
    int N, float eps, int64_t ss_row, int64_t ss_group) {
  const int64_t chunks_per_row = N / kVec;
  const int64_t total = R * chunks_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t base = blockIdx.x * static_cast<int64_t>(blockDim.x); base < total; base += stride) {
    const int64_t c = base + threadIdx.x;
    const bool live = c < total;
    const int64_t r = live ? c / chunks_per_row : 0;
    const int col = live ? static_cast<int>(c % chunks_per_row) * kVec : 0;
    float x[kVec];
    float amax = SILU ? 0.f : eps;
    if (live) {
      fetch8<T, SILU>(in, r, col, N, x);
#pragma unroll
      for (int i = 0; i < kVec; ++i) amax = fmaxf(amax, fabsf(x[i]));
    }
    amax = seg_max<4>(amax);
    const float s = exp2f(ceilf(log2f(fmaxf(fabsf(amax / 6.0f), eps))));
    if (!live) continue;
    if ((threadIdx.x & 3) == 0) out_s[r * ss_row + (col / 32) * ss_group] = s;
    const float inv = 1.0f / s;
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const float y = fmaxf(-6.0f, fminf(x[i] * inv, 6.0f));
      packed |= static_cast<uint32_t>(e2m1_code(y)) << (4 * i);
    }
    *reinterpret_cast<uint32_t*>(out_q + (r * N + col) / 2) = packed;
  }
}

// MXFP8: e4m3 values with one e8m0 scale per 32 columns (4 lanes of 8 values).  The scale is
// the smallest power of two >= max(amax, 1e-10) / 448 (not below 1 / (448 * 512)), found on
// the bits of the float, and stored as its biased exponent.
template <typename T>
__global__ void __launch_bounds__(256) quant_mxfp8_kernel(const T* __restrict__ in,
                                                           uint8_t* __restrict__ out_q,
                                                           uint8_t* __restrict__ out_sf, int64_t R,
                                                           int N, int64_t sf_pitch) {
  const int64_t chunks_per_row = N / kVec;
  const int64_t total = R * chunks_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t base = blockIdx.x * static_cast<int64_t>(blockDim.x); base < total; base += stride) {
    const int64_t c = base + threadIdx.x;
    const bool live = c < total;
    const int64_t r = live ? c / chunks_per_row : 0;
    const int col = live ? static_cast<int>(c % chunks_per_row) * kVec : 0;
    float x[kVec];
    float amax = 0.f;
    if (live) {
      fetch8<T, false>(in, r, col, N, x);
#pragma unroll
      for (int i = 0; i < kVec; ++i) amax = fmaxf(amax, fabsf(x[i]));
    }
    amax = seg_max<4>(amax);
    const float s0 = fmaxf(fmaxf(amax, 1e-10f) * (1.0f / 448.0f), 1.0f / (448.0f * 512.0f));
    uint32_t bits = __float_as_uint(s0);
    uint32_t e = bits >> 23;
    if (bits & 0x7FFFFFu) ++e;
    if (!live) continue;
    if ((threadIdx.x & 3) == 0) out_sf[r * sf_pitch + col / 32] = static_cast<uint8_t>(e);
    const float inv = 1.0f / __uint_as_float(e << 23);
    uint8_t q[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) q[i] = f32_to_e4m3(fmaxf(-448.f, fminf(x[i] * inv, 448.f)));
    *reinterpret_cast<uint2*>(out_q + r * N + col) = *reinterpret_cast<uint2*>(q);
  }
}

inline int stream_grid(int64_t work_items, int threads) {
  int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(kNumSMs) * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

inline bool pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_silu_and_mul(void* out, const void* in, int dtype, int64_t R, int d,
                                    void* stream) {
  if (R < 0 || d <= 0) return B200MOE_INVALID_ARG;
  if (R == 0) return B200MOE_OK;
  if (!out || !in) return B200MOE_INVALID_ARG;
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    constexpr int V = 16 / sizeof(scalar_t);
    cudaStream_t st = as_stream(stream);
    if (d % V == 0) {
      silu_and_mul_kernel<scalar_t><<<stream_grid(R * (d / V), 256), 256, 0, st>>>(
          reinterpret_cast<scalar_t*>(out), reinterpret_cast<const scalar_t*>(in), R, d);
    } else {
      silu_and_mul_scalar_kernel<scalar_t><<<stream_grid(R * d, 256), 256, 0, st>>>(
          reinterpret_cast<scalar_t*>(out), reinterpret_cast<const scalar_t*>(in), R, d);
    }
    return launch_status("silu_and_mul_kernel");
  });
}

extern "C" int b200moe_swigluoai_and_mul(void* out, const void* in, int dtype, int64_t R, int d,
                                         float alpha, float limit, void* stream) {
  if (R < 0 || d <= 0) return B200MOE_INVALID_ARG;
  if (R == 0) return B200MOE_OK;
  if (!out || !in) return B200MOE_INVALID_ARG;
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    swigluoai_kernel<scalar_t><<<stream_grid(R * d, 256), 256, 0, as_stream(stream)>>>(
        reinterpret_cast<scalar_t*>(out), reinterpret_cast<const scalar_t*>(in), R, d, alpha, limit);
    return launch_status("swigluoai_kernel");
  });
}

extern "C" int b200moe_act_and_mul(void* out, const void* in, int dtype, int64_t R, int d, int act,
                                   float param0, float param1, float clamp_limit, void* stream) {
  if (R < 0 || d <= 0 || act < B200MOE_ACT_SILU || act > B200MOE_ACT_RELU2_NO_MUL)
    return B200MOE_INVALID_ARG;
  if (act == B200MOE_ACT_SITU && !(isfinite(param0) && param0 > 0.0f && isfinite(param1)))
    return B200MOE_INVALID_ARG;  // beta finite and > 0, linear_beta finite
  if (R == 0) return B200MOE_OK;
  if (!out || !in) return B200MOE_INVALID_ARG;
  const float clamp = clamp_limit > 0.0f ? clamp_limit : 0.0f;
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    constexpr int V = 16 / sizeof(scalar_t);
    cudaStream_t st = as_stream(stream);
    scalar_t* o = reinterpret_cast<scalar_t*>(out);
    const scalar_t* x = reinterpret_cast<const scalar_t*>(in);
    if (act == B200MOE_ACT_RELU2_NO_MUL) {
      if (d % V == 0)
        relu2_kernel<scalar_t, V><<<stream_grid(R * (d / V), 256), 256, 0, st>>>(o, x, R, d, clamp, d / 2);
      else
        relu2_kernel<scalar_t, 1><<<stream_grid(R * d, 256), 256, 0, st>>>(o, x, R, d, clamp, d / 2);
      return launch_status("relu2_kernel");
    }
    if (d % V == 0)
      act_and_mul_kernel<scalar_t, V><<<stream_grid(R * (d / V), 256), 256, 0, st>>>(
          o, x, R, d, act, param0, param1, clamp);
    else
      act_and_mul_kernel<scalar_t, 1><<<stream_grid(R * d, 256), 256, 0, st>>>(
          o, x, R, d, act, param0, param1, clamp);
    return launch_status("act_and_mul_kernel");
  });
}

static int check_group(int64_t R, int N, int group_size) {
  if (R < 0 || N <= 0 || group_size <= 0 || N % group_size != 0) return B200MOE_INVALID_ARG;
  if (!pow2(group_size) || group_size < kVec || group_size > 256) return B200MOE_UNSUPPORTED;
  return B200MOE_OK;
}

extern "C" int b200moe_per_token_group_fp8_quant(const void* in, int dtype, void* out_q,
                                                 float* out_s, int64_t R, int N, int group_size,
                                                 float eps, float fp8_min, float fp8_max,
                                                 int scale_ue8m0, int64_t ss_row, int64_t ss_group,
                                                 void* stream) {
  int rc = check_group(R, N, group_size);
  if (rc != B200MOE_OK) return rc;
  if (R == 0) return B200MOE_OK;
  if (!in || !out_q || !out_s) return B200MOE_INVALID_ARG;
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    group_quant_fp8_kernel<scalar_t, false, false>
        <<<stream_grid(R * (N / kVec), 256), 256, 0, as_stream(stream)>>>(
            reinterpret_cast<const scalar_t*>(in), reinterpret_cast<uint8_t*>(out_q), out_s, R, N,
            group_size, eps, fp8_min, fp8_max, scale_ue8m0 != 0, nullptr, ss_row, ss_group);
    return launch_status("group_quant_fp8_kernel");
  });
}

extern "C" int b200moe_silu_mul_block_quant(const void* in, int dtype, void* out_q, float* out_s,
                                            int64_t R, int d, int group_size,
                                            const float* scale_ub, int scale_ue8m0, int64_t ss_row,
                                            int64_t ss_group, void* stream) {
  int rc = check_group(R, d, group_size);
  if (rc != B200MOE_OK) return rc;
  if (R == 0) return B200MOE_OK;
  if (!in || !out_q || !out_s) return B200MOE_INVALID_ARG;
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    group_quant_fp8_kernel<scalar_t, true, true>
        <<<stream_grid(R * (d / kVec), 256), 256, 0, as_stream(stream)>>>(
            reinterpret_cast<const scalar_t*>(in), reinterpret_cast<uint8_t*>(out_q), out_s, R, d,
            group_size, 0.f, -448.f, 448.f, scale_ue8m0 != 0, scale_ub, ss_row, ss_group);
    return launch_status("silu_mul_block_quant_kernel");
  });
}

extern "C" int b200moe_per_token_group_quant_mxfp4(const void* in, int dtype, uint8_t* out_q,
                                                   float* out_s, int64_t R, int N, int group_size,
                                                   float eps, int64_t ss_row, int64_t ss_group,
                                                   void* stream) {
  if (group_size != 32) return B200MOE_UNSUPPORTED;
  if (R < 0 || N <= 0 || N % 32 != 0) return B200MOE_INVALID_ARG;
  if (R == 0) return B200MOE_OK;
  if (!in || !out_q || !out_s) return B200MOE_INVALID_ARG;
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    group_quant_mxfp4_kernel<scalar_t, false>
        <<<stream_grid(R * (N / kVec), 256), 256, 0, as_stream(stream)>>>(
            reinterpret_cast<const scalar_t*>(in), out_q, out_s, R, N, eps, ss_row, ss_group);
    return launch_status("group_quant_mxfp4_kernel");
  });
}

extern "C" int b200moe_silu_mul_mxfp4_quant(const void* in, int dtype, uint8_t* out_q,
                                            float* out_s, int64_t R, int d, int group_size,
                                            float eps, void* stream) {
  if (group_size != 32) return B200MOE_UNSUPPORTED;
  if (R < 0 || d <= 0 || d % 32 != 0) return B200MOE_INVALID_ARG;
  if (R == 0) return B200MOE_OK;
  if (!in || !out_q || !out_s) return B200MOE_INVALID_ARG;
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    group_quant_mxfp4_kernel<scalar_t, true>
        <<<stream_grid(R * (d / kVec), 256), 256, 0, as_stream(stream)>>>(
            reinterpret_cast<const scalar_t*>(in), out_q, out_s, R, d, eps, d / 32, 1);
    return launch_status("silu_mul_mxfp4_quant_kernel");
  });
}

extern "C" int b200moe_quant_mxfp8(const void* in, int dtype, void* out_q, uint8_t* out_sf,
                                   int64_t R, int N, int64_t sf_pitch, void* stream) {
  if (R < 0 || N <= 0 || N % 32 || sf_pitch < N / 32) return B200MOE_INVALID_ARG;
  if (R == 0) return B200MOE_OK;
  if (!in || !out_q || !out_sf) return B200MOE_INVALID_ARG;
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    quant_mxfp8_kernel<scalar_t><<<stream_grid(R * (N / kVec), 256), 256, 0, as_stream(stream)>>>(
        reinterpret_cast<const scalar_t*>(in), reinterpret_cast<uint8_t*>(out_q), out_sf, R, N,
        sf_pitch);
    return launch_status("quant_mxfp8_kernel");
  });
}
