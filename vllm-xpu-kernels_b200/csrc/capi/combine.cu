// Combine kernels: moe_gather (weighted un-permute) and moe_sum.
//
// Both are pure streaming: every thread owns 16-byte columns of one output
// row, pulls the same columns of the k source rows, accumulates in fp32 and
// stores once.  Two tokens' worth of CTAs per SM keep HBM busy; there is no
// reuse to exploit, so no shared memory is used for data.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kMaxTopK = 64;

template <typename T>
__global__ void __launch_bounds__(256) moe_gather_kernel(
    T* __restrict__ out, const T* __restrict__ y, const float* __restrict__ weights,
    const int32_t* __restrict__ row_map, const T* __restrict__ addend,
    const int32_t* __restrict__ num_valid, int k, int H) {
  constexpr int V = 16 / sizeof(T);
  const int64_t t = blockIdx.x;
  if (num_valid && t >= *num_valid) return;  // rows of a worst-case buffer nobody will read
  __shared__ int rows[kMaxTopK];
  __shared__ float w[kMaxTopK];
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    rows[j] = row_map[t * k + j];
    w[j] = weights[t * k + j];
  }
  __syncthreads();
  for (int c = threadIdx.x * V; c < H; c += blockDim.x * V) {
    float acc[V];
    if (addend) {  // e.g. the shared expert's row of this token, weight 1
      load_f32<T, V>(addend + t * H + c, acc);
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = 0.f;
    }
    for (int j = 0; j < k; ++j) {
      const int r = rows[j];
      if (r < 0) continue;
      float v[V];
      load_f32<T, V>(y + static_cast<int64_t>(r) * H + c, v);
      const float wj = w[j];
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] += wj * v[i];
    }
    store_f32<T, V>(out + t * H + c, acc);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256) moe_sum_kernel(
    T* __restrict__ out, const T* __restrict__ in, int k, int H, const void* __restrict__ ids,
    int ids_dtype, const int32_t* __restrict__ expert_map) {
  const int64_t t = blockIdx.x;
  __shared__ int keep[kMaxTopK];
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    int kp = 1;
    if (ids) {
      const int64_t id = load_index(ids, ids_dtype, t * k + j);
      kp = id >= 0 && (!expert_map || expert_map[id] >= 0);
    }
    keep[j] = kp;
  }
  __syncthreads();
  for (int c = threadIdx.x * V; c < H; c += blockDim.x * V) {
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    for (int j = 0; j < k; ++j) {
      if (!keep[j]) continue;
      float v[V];
      load_f32<T, V>(in + (t * k + j) * H + c, v);
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] += v[i];
    }
    store_f32<T, V>(out + t * H + c, acc);
  }
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

static int gather_impl(void* out, const void* y, int dtype, const float* weights,
                       const int32_t* row_map, const void* addend, const int32_t* num_valid, int T,
                       int k, int H, void* stream) {
  if (T < 0 || k <= 0 || k > kMaxTopK || H <= 0) return B200MOE_INVALID_ARG;
  if (T == 0) return B200MOE_OK;
  if (!out || !y || !weights || !row_map) return B200MOE_INVALID_ARG;
  if ((H * dtype_size(dtype)) % 16 != 0) return B200MOE_INVALID_ARG;
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    constexpr int V = 16 / sizeof(scalar_t);
    int threads = (H / V + 31) / 32 * 32;
    threads = threads > 256 ? 256 : threads;
    moe_gather_kernel<scalar_t><<<T, threads, 0, as_stream(stream)>>>(
        reinterpret_cast<scalar_t*>(out), reinterpret_cast<const scalar_t*>(y), weights, row_map,
        reinterpret_cast<const scalar_t*>(addend), num_valid, k, H);
    return launch_status("moe_gather_kernel");
  });
}

extern "C" int b200moe_moe_gather(void* out, const void* y, int dtype, const float* weights,
                                  const int32_t* row_map, int T, int k, int H, void* stream) {
  return gather_impl(out, y, dtype, weights, row_map, nullptr, nullptr, T, k, H, stream);
}

extern "C" int b200moe_moe_gather_add(void* out, const void* y, int dtype, const float* weights,
                                      const int32_t* row_map, const void* addend, int T, int k,
                                      int H, void* stream) {
  if (!addend) return B200MOE_INVALID_ARG;
  return gather_impl(out, y, dtype, weights, row_map, addend, nullptr, T, k, H, stream);
}

extern "C" int b200moe_moe_gather_bounded(void* out, const void* y, int dtype, const float* weights,
                                          const int32_t* row_map, const int32_t* num_valid_tokens,
                                          int T, int k, int H, void* stream) {
  if (!num_valid_tokens) return B200MOE_INVALID_ARG;
  return gather_impl(out, y, dtype, weights, row_map, nullptr, num_valid_tokens, T, k, H, stream);
}

extern "C" int b200moe_moe_sum(const void* in, void* out, int dtype, int T, int k, int H,
                               const void* topk_ids, int ids_dtype, const int32_t* expert_map,
                               void* stream) {
  if (T < 0 || k <= 0 || k > kMaxTopK || H <= 0) return B200MOE_INVALID_ARG;
  if (topk_ids && !is_index_dtype(ids_dtype)) return B200MOE_INVALID_ARG;
  if (T == 0) return B200MOE_OK;
  if (!in || !out) return B200MOE_INVALID_ARG;
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    constexpr int VMAX = 16 / sizeof(scalar_t);
    cudaStream_t st = as_stream(stream);
    const scalar_t* i = reinterpret_cast<const scalar_t*>(in);
    scalar_t* o = reinterpret_cast<scalar_t*>(out);
    if (H % VMAX == 0) {
      int threads = (H / VMAX + 31) / 32 * 32;
      threads = threads > 256 ? 256 : threads;
      moe_sum_kernel<scalar_t, VMAX><<<T, threads, 0, st>>>(o, i, k, H, topk_ids, ids_dtype, expert_map);
    } else {
      int threads = (H + 31) / 32 * 32;
      threads = threads > 256 ? 256 : threads;
      moe_sum_kernel<scalar_t, 1><<<T, threads, 0, st>>>(o, i, k, H, topk_ids, ids_dtype, expert_map);
    }
    return launch_status("moe_sum_kernel");
  });
}
