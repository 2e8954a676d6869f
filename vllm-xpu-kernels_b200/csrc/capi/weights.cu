// One-time expansion of the weight formats whose activations stay 16-bit
// (W8A16 / W4A16 recipes) into the 16-bit operand the tcgen05 kind::f16 path
// consumes.  The tensor cores take both operands in one element width, so a
// weight narrower than the activation has to be widened somewhere; doing it
// once when the layer is built keeps the per-call path a plain 16-bit grouped
// GEMM and costs 2 bytes per weight of HBM.
//
//   per-tensor FP8   [E,K,N] e4m3|e5m2, one f32 scale per expert  -> [E,K,N]
//   MXFP8            [E,K,N] e4m3|e5m2, e8m0 scale [E,K/32,N]     -> [E,K,N]
//   INT4             [E,N,K/2] u8 (low nibble = even k, value = nibble - 8),
//                    16-bit or f32 scale [E,N,K/group]            -> [E,N,K]
//
// Every output is round_to_T(value * scale): exact for MXFP8 (power-of-two
// scale) and one rounding for the other two, the same rounding the reference's
// own dequantise-then-matmul oracles apply.
#include "common.cuh"

namespace b200moe {
namespace {

__device__ __forceinline__ float fp8_to_f32(uint8_t v, bool e5m2) {
  __half_raw h =
      __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(v), e5m2 ? __NV_E5M2 : __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

__device__ __forceinline__ float e8m0_to_f32(uint8_t s) {
  // 2^(s-127); s = 0 is the subnormal 2^-127, s = 255 is NaN
  const uint32_t bits = s == 0 ? 0x00400000u : (s == 255 ? 0x7fc00000u : static_cast<uint32_t>(s) << 23);
  return __uint_as_float(bits);
}

__device__ __forceinline__ float load_scale(const void* s, int dtype, int64_t i) {
  if (dtype == B200MOE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(s)[i]);
  if (dtype == B200MOE_F16) return __half2float(reinterpret_cast<const __half*>(s)[i]);
  return reinterpret_cast<const float*>(s)[i];
}

// mode 0: scale[e]; mode 1: e8m0 scale[e, k/32, n].  8 consecutive n per thread.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) expand_fp8_kernel(const uint8_t* __restrict__ w, bool e5m2,
                                                         const void* __restrict__ scale,
                                                         T* __restrict__ out, int64_t E, int K,
                                                         int N) {
  const int64_t total = E * K * static_cast<int64_t>(N) / 8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t at = i * 8;
    const int n = static_cast<int>(at % N);
    const int64_t ek = at / N;
    const int k = static_cast<int>(ek % K);
    const int64_t e = ek / K;
    const uint2 raw = *reinterpret_cast<const uint2*>(w + at);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
    float sc[8];
    if (MODE == 0) {
      const float s = reinterpret_cast<const float*>(scale)[e];
#pragma unroll
      for (int j = 0; j < 8; ++j) sc[j] = s;
    } else {
      const uint2 sraw = *reinterpret_cast<const uint2*>(
          reinterpret_cast<const uint8_t*>(scale) + (e * (K / 32) + k / 32) * N + n);
      const uint8_t* sb = reinterpret_cast<const uint8_t*>(&sraw);
#pragma unroll
      for (int j = 0; j < 8; ++j) sc[j] = e8m0_to_f32(sb[j]);
    }
    Vec<T, 8> o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = Elem<T>::from_f32(fp8_to_f32(b[j], e5m2) * sc[j]);
    *reinterpret_cast<Vec<T, 8>*>(out + at) = o;
  }
}

// 4 packed bytes = 8 consecutive k per thread.
template <typename T>
__global__ void __launch_bounds__(256) expand_int4_kernel(const uint8_t* __restrict__ w,
                                                          const void* __restrict__ scale,
                                                          int scale_dtype, T* __restrict__ out,
                                                          int64_t rows, int K, int group) {
  const int64_t total = rows * (K / 8);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / (K / 8);
    const int k0 = static_cast<int>(i % (K / 8)) * 8;
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(w + row * (K / 2) + k0 / 2);
    const float sc = load_scale(scale, scale_dtype, row * (K / group) + k0 / group);
    Vec<T, 8> o;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int q = static_cast<int>((raw >> (4 * j)) & 0xF) - 8;
      o.v[j] = Elem<T>::from_f32(static_cast<float>(q) * sc);
    }
    *reinterpret_cast<Vec<T, 8>*>(out + row * K + k0) = o;
  }
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_expand_weights(int recipe, const void* B, int b_dtype, const void* b_scale,
                                      int scale_dtype, int group_size, void* out, int out_dtype,
                                      int E, int N, int K, void* stream) {
  if (!B || !b_scale || !out || E <= 0 || N <= 0 || K <= 0) return B200MOE_INVALID_ARG;
  if (out_dtype != B200MOE_BF16 && out_dtype != B200MOE_F16) return B200MOE_UNSUPPORTED;
  cudaStream_t st = as_stream(stream);
  const int grid = kNumSMs * 8;
  const uint8_t* w = reinterpret_cast<const uint8_t*>(B);
  const bool bf = out_dtype == B200MOE_BF16;
  if (recipe == B200MOE_RECIPE_FP8_TENSOR || recipe == B200MOE_RECIPE_MXFP8) {
    if (b_dtype != B200MOE_E4M3 && b_dtype != B200MOE_E5M2) return B200MOE_UNSUPPORTED;
    if (N % 8) return B200MOE_INVALID_ARG;
    const bool e5 = b_dtype == B200MOE_E5M2;
    if (recipe == B200MOE_RECIPE_FP8_TENSOR) {
      if (scale_dtype != B200MOE_F32) return B200MOE_UNSUPPORTED;
      if (bf) expand_fp8_kernel<__nv_bfloat16, 0><<<grid, 256, 0, st>>>(w, e5, b_scale, reinterpret_cast<__nv_bfloat16*>(out), E, K, N);
      else expand_fp8_kernel<__half, 0><<<grid, 256, 0, st>>>(w, e5, b_scale, reinterpret_cast<__half*>(out), E, K, N);
    } else {
      if (scale_dtype != B200MOE_U8 || K % 32) return B200MOE_INVALID_ARG;
      if (bf) expand_fp8_kernel<__nv_bfloat16, 1><<<grid, 256, 0, st>>>(w, e5, b_scale, reinterpret_cast<__nv_bfloat16*>(out), E, K, N);
      else expand_fp8_kernel<__half, 1><<<grid, 256, 0, st>>>(w, e5, b_scale, reinterpret_cast<__half*>(out), E, K, N);
    }
  } else if (recipe == B200MOE_RECIPE_INT4) {
    if (group_size <= 0 || group_size % 8 || K % group_size) return B200MOE_INVALID_ARG;
    if (scale_dtype != B200MOE_BF16 && scale_dtype != B200MOE_F16 && scale_dtype != B200MOE_F32)
      return B200MOE_UNSUPPORTED;
    const int64_t rows = static_cast<int64_t>(E) * N;
    if (bf) expand_int4_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(w, b_scale, scale_dtype, reinterpret_cast<__nv_bfloat16*>(out), rows, K, group_size);
    else expand_int4_kernel<__half><<<grid, 256, 0, st>>>(w, b_scale, scale_dtype, reinterpret_cast<__half*>(out), rows, K, group_size);
  } else {
    return B200MOE_UNSUPPORTED;
  }
  return launch_status("expand_weights");
}
