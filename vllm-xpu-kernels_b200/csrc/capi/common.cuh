// Shared helpers of the b200moe kernels: status handling, element-type
// dispatch and 16-byte vector access.  Pure CUDA, no torch headers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "b200moe.h"

namespace b200moe {

constexpr int kNumSMs = 148;  // B200: two dies of 74 SMs

void set_last_error(const char* what, cudaError_t err);
// Device address of the status word that kernels raise when a bounded wait runs out
// (read and cleared by b200moe_device_status); null if it cannot be resolved.
int* device_status_word();

// Kernels this library has enqueued in this process (every launch goes through
// launch_status); read by b200moe_launch_count.
void count_launch();

// Checks the launch that was just enqueued and maps a failure to a status.
inline int launch_status(const char* what) {
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_last_error(what, err);
    return B200MOE_CUDA_ERROR;
  }
  return B200MOE_OK;
}

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Raises a kernel's dynamic shared-memory limit.  The attribute belongs to the (kernel,
// device) pair, so it is set once per device this process launches on, under a lock.
// `Tag` separates the bookkeeping of kernels that share one function-pointer type.
template <typename Tag, typename Kernel>
int ensure_dynamic_smem(Kernel kernel, size_t bytes, const char* what) {
  constexpr int kMaxDev = 64;
  static std::mutex mu;
  static bool done[kMaxDev] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) dev = -1;
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && done[dev]) return B200MOE_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(bytes));
  if (e != cudaSuccess) {
    set_last_error(what, e);
    return B200MOE_CUDA_ERROR;
  }
  if (dev >= 0) done[dev] = true;
  return B200MOE_OK;
}

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

// Rounds an fp32 value through T and back (what "compute in the input dtype" means).
template <typename T>
__device__ __forceinline__ float round_through(float v) {
  return Elem<T>::to_f32(Elem<T>::from_f32(v));
}

// N elements of T moved as 16-byte (or smaller) chunks.
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
  T v[N];
};

template <typename T, int N>
__device__ __forceinline__ void load_f32(const T* p, float (&out)[N]) {
  Vec<T, N> tmp = *reinterpret_cast<const Vec<T, N>*>(p);
#pragma unroll
  for (int i = 0; i < N; ++i) out[i] = Elem<T>::to_f32(tmp.v[i]);
}

template <typename T, int N>
__device__ __forceinline__ void store_f32(T* p, const float (&in)[N]) {
  Vec<T, N> tmp;
#pragma unroll
  for (int i = 0; i < N; ++i) tmp.v[i] = Elem<T>::from_f32(in[i]);
  *reinterpret_cast<Vec<T, N>*>(p) = tmp;
}

__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(v), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// Integer index tensors arrive as i32, u32 or i64.
__device__ __forceinline__ int64_t load_index(const void* p, int dtype, int64_t i) {
  if (dtype == B200MOE_I64) return reinterpret_cast<const int64_t*>(p)[i];
  if (dtype == B200MOE_U32) return static_cast<int64_t>(reinterpret_cast<const uint32_t*>(p)[i]);
  return static_cast<int64_t>(reinterpret_cast<const int32_t*>(p)[i]);
}

__device__ __forceinline__ void store_index(void* p, int dtype, int64_t i, int64_t v) {
  if (dtype == B200MOE_I64) reinterpret_cast<int64_t*>(p)[i] = v;
  else if (dtype == B200MOE_U32) reinterpret_cast<uint32_t*>(p)[i] = static_cast<uint32_t>(v);
  else reinterpret_cast<int32_t*>(p)[i] = static_cast<int32_t>(v);
}

inline bool is_index_dtype(int d) { return d == B200MOE_I32 || d == B200MOE_I64 || d == B200MOE_U32; }
inline bool is_float_dtype(int d) { return d == B200MOE_F32 || d == B200MOE_F16 || d == B200MOE_BF16; }
inline int dtype_size(int d) {
  switch (d) {
    case B200MOE_F32: case B200MOE_I32: case B200MOE_U32: return 4;
    case B200MOE_F16: case B200MOE_BF16: return 2;
    case B200MOE_I64: return 8;
    default: return 1;
  }
}

// Calls f(T{}) with T the C++ type of a floating dtype code.
#define B200MOE_DISPATCH_FLOAT(dtype, ...)                                   \
  [&]() -> int {                                                             \
    switch (dtype) {                                                         \
      case B200MOE_F32: { using scalar_t = float; return __VA_ARGS__(); }    \
      case B200MOE_F16: { using scalar_t = __half; return __VA_ARGS__(); }   \
      case B200MOE_BF16: { using scalar_t = __nv_bfloat16; return __VA_ARGS__(); } \
      default: return B200MOE_UNSUPPORTED;                                   \
    }                                                                        \
  }()

}  // namespace b200moe
