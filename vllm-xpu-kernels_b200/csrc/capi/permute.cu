// Token permutation: moe_align_block_size, remap_hidden_states, init_expert_map.
//
// Both permutations are one stable counting sort of the flat (token, slot)
// indices by expert, done with integers only so the result is reproducible and
// equal to what a stable sort gives:
//   1. count   — each CTA histograms a contiguous chunk of flat indices into
//                 shared memory and writes its row of per-CTA counts;
//   2. scan    — one CTA turns the [n_cta, E] counts into, for every
//                 (cta, expert), the output position of that CTA's first
//                 element of that expert (expert starts padded to the block
//                 size for align), and writes the per-expert results;
//   3. place   — each CTA walks its chunk again in index order; an element's
//                 rank among equal experts comes from a warp match plus
//                 per-warp running offsets, never from atomics.
// Inputs that fit one chunk take a single fused launch.
#include <stdio.h>

#include <mutex>

#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kChunk = 2048;  // flat indices per CTA: 8 warps x 8 steps x 32 lanes
constexpr int kMaxExperts = 1024;

struct GroupParams {
  const void* ids;
  int ids_dtype;
  int64_t numel;
  int num_keys;        // number of output groups' key space (experts before mapping for align)
  int id_limit;        // ids >= id_limit are ignored
  const int32_t* map;  // optional id -> key (remap) or id -> keep? (align)
  int map_is_filter;   // 1: map only decides validity (align); 0: map gives the key (remap)
  int block_size;      // padding unit of each group's run (1 = none)
  // optional per-token filter (multi-LoRA): only tokens with token_tag[i / topk] == tag count
  const int32_t* token_tag = nullptr;
  int tag = 0;
  int topk = 1;
};

__device__ __forceinline__ int key_of(const GroupParams& p, int64_t i) {
  const int64_t id = load_index(p.ids, p.ids_dtype, i);
  if (id < 0 || id >= p.id_limit) return -1;
  if (p.token_tag && p.token_tag[i / p.topk] != p.tag) return -1;
  if (p.map) {
    const int m = p.map[id];
    if (m < 0) return -1;
    if (p.map_is_filter) return static_cast<int>(id);
    return m < p.num_keys ? m : -1;  // a map value outside the key space is dropped, not binned
  }
  return static_cast<int>(id);
}

// Histogram of this CTA's chunk into smem hist[num_keys].
__device__ __forceinline__ void chunk_histogram(const GroupParams& p, int64_t base, int* hist) {
  for (int e = threadIdx.x; e < p.num_keys; e += kThreads) hist[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < kChunk; i += kThreads) {
    const int64_t idx = base + i;
    if (idx < p.numel) {
      const int key = key_of(p, idx);
      if (key >= 0) atomicAdd(&hist[key], 1);  // integer counts: order does not matter
    }
  }
  __syncthreads();
}

// Walks the chunk in index order.  warp w owns indices [w*256, w*256+256) of
// the chunk; per-warp counts are prefix-summed across warps so that positions
// follow ascending flat index.  `emit(idx, key, pos)` is called once per valid
// element with pos = cta_base[key] + rank inside the CTA.
template <typename Emit>
__device__ __forceinline__ void chunk_place(const GroupParams& p, int64_t base,
                                            const int* cta_base, int* warp_off, Emit emit) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kPerWarp = kChunk / kWarps;
  for (int e = threadIdx.x; e < p.num_keys * kWarps; e += kThreads) warp_off[e] = 0;
  __syncthreads();
  int keys[kPerWarp / 32];
#pragma unroll
  for (int s = 0; s < kPerWarp / 32; ++s) {
    const int64_t idx = base + warp * kPerWarp + s * 32 + lane;
    keys[s] = idx < p.numel ? key_of(p, idx) : -1;
    if (keys[s] >= 0) atomicAdd(&warp_off[warp * p.num_keys + keys[s]], 1);
  }
  __syncthreads();
  // exclusive prefix over warps, per key
  for (int e = threadIdx.x; e < p.num_keys; e += kThreads) {
    int run = cta_base[e];
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const int c = warp_off[w * p.num_keys + e];
      warp_off[w * p.num_keys + e] = run;
      run += c;
    }
  }
  __syncthreads();
  int* mine = warp_off + warp * p.num_keys;
#pragma unroll
  for (int s = 0; s < kPerWarp / 32; ++s) {
    const int key = keys[s];
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    if (key >= 0) {
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int pos = mine[key] + rank;
      emit(base + warp * kPerWarp + s * 32 + lane, key, pos);
    }
    __syncwarp();
    if (key >= 0 && lane == (31 - __clz(peers))) mine[key] += __popc(peers);
    __syncwarp();
  }
}

__global__ void __launch_bounds__(kThreads) count_kernel(GroupParams p, int* __restrict__ counts) {
  extern __shared__ int smem[];
  chunk_histogram(p, static_cast<int64_t>(blockIdx.x) * kChunk, smem);
  for (int e = threadIdx.x; e < p.num_keys; e += kThreads)
    counts[static_cast<int64_t>(blockIdx.x) * p.num_keys + e] = smem[e];
}

// Per-key totals -> padded starts (exclusive scan over keys, any num_keys <=
// 1024 by a block-wide scan of 1024 slots).  Returns this thread's key start
// in `start` for key = threadIdx.x + 256*j via smem arrays.
__device__ __forceinline__ void scan_keys(int num_keys, int block_size, const int* total,
                                          int* start, int* grand_total) {
  // total/start are smem arrays of kMaxExperts ints.  Sequential-in-warp scan:
  // thread t handles 4 consecutive keys.
  __shared__ int warp_sums[kWarps];
  const int t = threadIdx.x;
  int v[4], pad[4];
  int local = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = t * 4 + j;
    v[j] = e < num_keys ? total[e] : 0;
    pad[j] = (v[j] + block_size - 1) / block_size * block_size;
    local += pad[j];
  }
  int incl = local;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, off);
    if ((t & 31) >= off) incl += o;
  }
  if ((t & 31) == 31) warp_sums[t >> 5] = incl;
  __syncthreads();
  int warp_base = 0;
  for (int w = 0; w < (t >> 5); ++w) warp_base += warp_sums[w];
  int run = warp_base + incl - local;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = t * 4 + j;
    if (e < num_keys) start[e] = run;
    run += pad[j];
  }
  if (t == kThreads - 1) *grand_total = run;
  __syncthreads();
}

struct AlignOut {
  int32_t* sorted_ids;
  int64_t sorted_capacity;
  int32_t* expert_ids;
  int64_t blocks_capacity;
  int32_t* total;
  const int32_t* expert_map;
  int32_t tail_label = 0;  // expert_ids value of the blocks after the last used one
};

__device__ __forceinline__ void write_align_meta(const AlignOut& o, int num_keys, int block_size,
                                                 const int* total, const int* start,
                                                 int grand_total) {
  for (int e = threadIdx.x; e < num_keys; e += kThreads) {
    const int nb = (total[e] + block_size - 1) / block_size;
    const int b0 = start[e] / block_size;
    const int label = o.expert_map ? o.expert_map[e] : e;
    for (int b = 0; b < nb; ++b)
      if (b0 + b < o.blocks_capacity) o.expert_ids[b0 + b] = label;
  }
  for (int64_t b = grand_total / block_size + threadIdx.x; b < o.blocks_capacity; b += kThreads)
    o.expert_ids[b] = o.tail_label;
  if (threadIdx.x == 0) o.total[0] = grand_total;
}

// counts [n_cta, E] -> in place: position of each CTA's first element per key.
__global__ void __launch_bounds__(kThreads) scan_kernel(GroupParams p, int n_cta,
                                                        int* __restrict__ counts, AlignOut ao,
                                                        int32_t* __restrict__ rows_per_key) {
  __shared__ int total[kMaxExperts];
  __shared__ int start[kMaxExperts];
  __shared__ int grand;
  for (int e = threadIdx.x; e < p.num_keys; e += kThreads) {
    int run = 0;
    for (int c = 0; c < n_cta; ++c) run += counts[static_cast<int64_t>(c) * p.num_keys + e];
    total[e] = run;
  }
  __syncthreads();
  scan_keys(p.num_keys, p.block_size, total, start, &grand);
  for (int e = threadIdx.x; e < p.num_keys; e += kThreads) {
    int run = start[e];
    for (int c = 0; c < n_cta; ++c) {
      const int64_t at = static_cast<int64_t>(c) * p.num_keys + e;
      const int cnt = counts[at];
      counts[at] = run;
      run += cnt;
    }
    if (rows_per_key) rows_per_key[e] += total[e];
  }
  if (ao.sorted_ids) write_align_meta(ao, p.num_keys, p.block_size, total, start, grand);
}

__global__ void fill_kernel(int32_t* __restrict__ dst, int64_t n, int32_t value) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    dst[i] = value;
}

__global__ void __launch_bounds__(kThreads) place_align_kernel(GroupParams p,
                                                               const int* __restrict__ bases,
                                                               AlignOut ao) {
  extern __shared__ int smem[];
  int* cta_base = smem;
  int* warp_off = smem + p.num_keys;
  for (int e = threadIdx.x; e < p.num_keys; e += kThreads)
    cta_base[e] = bases[static_cast<int64_t>(blockIdx.x) * p.num_keys + e];
  __syncthreads();
  chunk_place(p, static_cast<int64_t>(blockIdx.x) * kChunk, cta_base, warp_off,
              [&](int64_t idx, int, int pos) {
                if (pos < ao.sorted_capacity) ao.sorted_ids[pos] = static_cast<int32_t>(idx);
              });
}

__global__ void __launch_bounds__(kThreads) place_remap_kernel(GroupParams p,
                                                               const int* __restrict__ bases,
                                                               int32_t* __restrict__ row_map) {
  extern __shared__ int smem[];
  int* cta_base = smem;
  int* warp_off = smem + p.num_keys;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kChunk;
  for (int e = threadIdx.x; e < p.num_keys; e += kThreads)
    cta_base[e] = bases[static_cast<int64_t>(blockIdx.x) * p.num_keys + e];
  for (int i = threadIdx.x; i < kChunk; i += kThreads)
    if (base + i < p.numel) row_map[base + i] = -1;
  __syncthreads();
  chunk_place(p, base, cta_base, warp_off,
              [&](int64_t idx, int, int pos) { row_map[idx] = pos; });
}

// Whole permutation in one CTA when numel <= kChunk.
__global__ void __launch_bounds__(kThreads) fused_small_kernel(GroupParams p, AlignOut ao,
                                                               int32_t* __restrict__ rows_per_key,
                                                               int32_t* __restrict__ row_map) {
  extern __shared__ int smem[];
  __shared__ int total[kMaxExperts];
  __shared__ int start[kMaxExperts];
  __shared__ int grand;
  int* warp_off = smem;
  chunk_histogram(p, 0, total);
  scan_keys(p.num_keys, p.block_size, total, start, &grand);
  if (ao.sorted_ids) {
    write_align_meta(ao, p.num_keys, p.block_size, total, start, grand);
    for (int64_t i = threadIdx.x; i < ao.sorted_capacity; i += kThreads)
      ao.sorted_ids[i] = static_cast<int32_t>(p.numel);
  }
  if (rows_per_key)
    for (int e = threadIdx.x; e < p.num_keys; e += kThreads) rows_per_key[e] += total[e];
  if (row_map)
    for (int i = threadIdx.x; i < p.numel; i += kThreads) row_map[i] = -1;
  __syncthreads();
  chunk_place(p, 0, start, warp_off, [&](int64_t idx, int, int pos) {
    if (ao.sorted_ids) {
      if (pos < ao.sorted_capacity) ao.sorted_ids[pos] = static_cast<int32_t>(idx);
    } else {
      row_map[idx] = pos;
    }
  });
}

// Multi-LoRA alignment: CTA x handles the adapter slot lora_ids[x] and builds that slot's
// own (sorted_token_ids, expert_ids, num_tokens_post_pad) from the tokens mapped to it.
// Slots that are -1, out of range or disabled are left untouched.  One CTA walks the whole
// index list twice (count, then place chunk by chunk in index order), so the order inside
// an expert's run is ascending flat index.
__global__ void __launch_bounds__(kThreads) lora_align_kernel(
    GroupParams p, const int32_t* __restrict__ lora_ids,
    const int32_t* __restrict__ adapter_enabled, int max_loras, int32_t* __restrict__ sorted_ids,
    int64_t max_padded, int32_t* __restrict__ expert_ids, int64_t max_blocks,
    int32_t* __restrict__ post_pad) {
  extern __shared__ int smem[];
  __shared__ int total[kMaxExperts];
  __shared__ int start[kMaxExperts];
  __shared__ int grand;
  const int lora_id = lora_ids[blockIdx.x];
  if (lora_id < 0 || lora_id >= max_loras || adapter_enabled[lora_id] == 0) return;
  p.tag = lora_id;
  int* warp_off = smem;
  for (int e = threadIdx.x; e < p.num_keys; e += kThreads) total[e] = 0;
  __syncthreads();
  for (int64_t i = threadIdx.x; i < p.numel; i += kThreads) {
    const int key = key_of(p, i);
    if (key >= 0) atomicAdd(&total[key], 1);
  }
  __syncthreads();
  scan_keys(p.num_keys, p.block_size, total, start, &grand);
  AlignOut ao{sorted_ids + lora_id * max_padded, max_padded, expert_ids + lora_id * max_blocks,
              max_blocks, post_pad + lora_id, nullptr, -1};
  write_align_meta(ao, p.num_keys, p.block_size, total, start, grand);
  for (int64_t i = threadIdx.x; i < max_padded; i += kThreads)
    ao.sorted_ids[i] = static_cast<int32_t>(p.numel);
  __syncthreads();
  for (int64_t base = 0; base < p.numel; base += kChunk) {
    chunk_place(p, base, start, warp_off, [&](int64_t idx, int, int pos) {
      if (pos < max_padded) ao.sorted_ids[pos] = static_cast<int32_t>(idx);
    });
    __syncthreads();
    // the last warp's cursors now stand behind everything this chunk placed
    for (int e = threadIdx.x; e < p.num_keys; e += kThreads)
      start[e] = warp_off[(kWarps - 1) * p.num_keys + e];
    __syncthreads();
  }
}

int run_grouping(const GroupParams& p, const AlignOut& ao, int32_t* rows_per_key,
                 int32_t* row_map, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (p.num_keys > kMaxExperts) return B200MOE_UNSUPPORTED;
  const int64_t n_cta64 = (p.numel + kChunk - 1) / kChunk;
  const size_t place_smem = static_cast<size_t>(p.num_keys) * (1 + kWarps) * sizeof(int);
  if (n_cta64 <= 1) {
    fused_small_kernel<<<1, kThreads, p.num_keys * kWarps * sizeof(int), st>>>(p, ao, rows_per_key,
                                                                              row_map);
    return launch_status("fused_small_kernel");
  }
  const int n_cta = static_cast<int>(n_cta64);
  const size_t need = static_cast<size_t>(n_cta) * p.num_keys * sizeof(int);
  if (!ws || ws_bytes < need) return B200MOE_WORKSPACE_TOO_SMALL;
  int* counts = reinterpret_cast<int*>(ws);
  if (ao.sorted_ids) {
    const int blocks = static_cast<int>((ao.sorted_capacity + 4095) / 4096);
    fill_kernel<<<blocks < 592 ? blocks : 592, 256, 0, st>>>(ao.sorted_ids, ao.sorted_capacity,
                                                             static_cast<int32_t>(p.numel));
  }
  count_kernel<<<n_cta, kThreads, p.num_keys * sizeof(int), st>>>(p, counts);
  scan_kernel<<<1, kThreads, 0, st>>>(p, n_cta, counts, ao, rows_per_key);
  if (ao.sorted_ids)
    place_align_kernel<<<n_cta, kThreads, place_smem, st>>>(p, counts, ao);
  else
    place_remap_kernel<<<n_cta, kThreads, place_smem, st>>>(p, counts, row_map);
  for (int i = 0; i < (ao.sorted_ids ? 3 : 2); ++i) count_launch();  // launch_status counts the last one
  return launch_status("stable grouping");
}

// ---- row copy of remap_hidden_states ------------------------------------------

// One CTA per token: the row is read once and written to each of its k
// permuted positions in 16-byte pieces.
__global__ void __launch_bounds__(256) copy_rows_kernel(
    const uint4* __restrict__ src, const uint8_t* __restrict__ src_scale,
    uint4* __restrict__ dst, uint8_t* __restrict__ dst_scale, int64_t row_vecs,
    int64_t scale_row_bytes, const int32_t* __restrict__ row_map, int k) {
  const int64_t t = blockIdx.x;
  __shared__ int rows[64];
  for (int j = threadIdx.x; j < k; j += blockDim.x) rows[j] = row_map[t * k + j];
  __syncthreads();
  const uint4* s = src + t * row_vecs;
  for (int64_t v = threadIdx.x; v < row_vecs; v += blockDim.x) {
    const uint4 val = s[v];
    for (int j = 0; j < k; ++j) {
      const int r = rows[j];
      if (r >= 0) dst[static_cast<int64_t>(r) * row_vecs + v] = val;
    }
  }
  if (src_scale) {
    const uint8_t* ss = src_scale + t * scale_row_bytes;
    if ((scale_row_bytes & 3) == 0) {
      for (int64_t v = threadIdx.x; v < scale_row_bytes / 4; v += blockDim.x) {
        const uint32_t val = reinterpret_cast<const uint32_t*>(ss)[v];
        for (int j = 0; j < k; ++j)
          if (rows[j] >= 0)
            reinterpret_cast<uint32_t*>(dst_scale + static_cast<int64_t>(rows[j]) * scale_row_bytes)[v] = val;
      }
    } else {
      for (int64_t v = threadIdx.x; v < scale_row_bytes; v += blockDim.x) {
        const uint8_t val = ss[v];
        for (int j = 0; j < k; ++j)
          if (rows[j] >= 0) dst_scale[static_cast<int64_t>(rows[j]) * scale_row_bytes + v] = val;
      }
    }
  }
}

__global__ void init_expert_map_kernel(int32_t* map, int num_local, int ep_rank, int total) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int lo = ep_rank * num_local;
  map[i] = (i >= lo && i < lo + num_local) ? i - lo : -1;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

size_t grouping_workspace(int64_t numel, int num_keys) {
  const int64_t n_cta = (numel + kChunk - 1) / kChunk;
  return n_cta <= 1 ? 0 : static_cast<size_t>(n_cta) * num_keys * sizeof(int);
}

extern "C" size_t b200moe_moe_align_block_size_workspace_bytes(int64_t numel, int num_experts) {
  return grouping_workspace(numel, num_experts);
}

extern "C" int b200moe_moe_align_block_size(const void* topk_ids, int ids_dtype, int64_t numel,
                                            int num_experts, int block_size,
                                            const int32_t* expert_map, int32_t* sorted_token_ids,
                                            int64_t sorted_capacity, int32_t* expert_ids,
                                            int64_t blocks_capacity, int32_t* num_tokens_post_pad,
                                            void* workspace, size_t workspace_bytes,
                                            void* stream) {
  if (numel < 0 || num_experts <= 0 || block_size <= 0 || !is_index_dtype(ids_dtype) ||
      !sorted_token_ids || !expert_ids || !num_tokens_post_pad || (numel > 0 && !topk_ids))
    return B200MOE_INVALID_ARG;
  if (numel >= (1ll << 31)) return B200MOE_UNSUPPORTED;
  // With an expert map the runs are keyed and ordered by the MAPPED (local) id, as the
  // reference kernel does (expert_id = expert_map[expert_id] before counting,
  // csrc/moe/moe_align_sum_kernels.cpp:201-205), so a map that is not monotone reorders the
  // runs; expert_ids then holds the keys themselves.
  GroupParams p{topk_ids, ids_dtype, numel, num_experts, num_experts, expert_map, 0, block_size};
  AlignOut ao{sorted_token_ids, sorted_capacity, expert_ids, blocks_capacity, num_tokens_post_pad,
              nullptr};
  return run_grouping(p, ao, nullptr, nullptr, workspace, workspace_bytes, as_stream(stream));
}

extern "C" int b200moe_init_expert_map(int32_t* expert_map, int num_local_experts, int ep_rank,
                                       int ep_size, void* stream) {
  if (!expert_map || num_local_experts <= 0 || ep_size <= 0 || ep_rank < 0 || ep_rank >= ep_size)
    return B200MOE_INVALID_ARG;
  const int total = num_local_experts * ep_size;
  init_expert_map_kernel<<<(total + 255) / 256, 256, 0, as_stream(stream)>>>(
      expert_map, num_local_experts, ep_rank, total);
  return launch_status("init_expert_map_kernel");
}

extern "C" size_t b200moe_remap_hidden_states_workspace_bytes(int T, int k, int local_experts) {
  return grouping_workspace(static_cast<int64_t>(T) * k, local_experts);
}

extern "C" int b200moe_remap_hidden_states(const void* hidden, const void* scales, void* remapped,
                                           void* remapped_scales, int64_t row_bytes,
                                           int64_t scale_row_bytes, const void* topk_ids,
                                           int ids_dtype, const int32_t* expert_map, int T, int k,
                                           int total_experts, int local_experts,
                                           int32_t* rows_per_expert, int32_t* row_map,
                                           void* workspace, size_t workspace_bytes,
                                           void* stream) {
  if (T < 0 || k <= 0 || k > 64 || local_experts <= 0 || total_experts <= 0 ||
      !is_index_dtype(ids_dtype) || !rows_per_expert || !row_map)
    return B200MOE_INVALID_ARG;
  if (row_bytes % 16 != 0) return B200MOE_INVALID_ARG;
  if (T == 0) return B200MOE_OK;
  if (!topk_ids || (hidden && !remapped) || (scales && !remapped_scales)) return B200MOE_INVALID_ARG;
  cudaStream_t st = as_stream(stream);
  GroupParams p{topk_ids, ids_dtype, static_cast<int64_t>(T) * k, local_experts,
                expert_map ? total_experts : local_experts, expert_map, 0, 1};
  AlignOut none{nullptr, 0, nullptr, 0, nullptr, nullptr};
  int rc = run_grouping(p, none, rows_per_expert, row_map, workspace, workspace_bytes, st);
  if (rc != B200MOE_OK) return rc;
  if (hidden) {
    copy_rows_kernel<<<T, 256, 0, st>>>(reinterpret_cast<const uint4*>(hidden),
                                        reinterpret_cast<const uint8_t*>(scales),
                                        reinterpret_cast<uint4*>(remapped),
                                        reinterpret_cast<uint8_t*>(remapped_scales),
                                        row_bytes / 16, scale_row_bytes, row_map, k);
    rc = launch_status("copy_rows_kernel");
  }
  return rc;
}

// ---- moe_align_block_size for callers that cannot allocate ----------------------

namespace b200moe {
namespace {

// Scratch of the allocation-free entry point: 64 Ki ints = 256 KiB of every GPU
// that loads this library, held until the process exits.
constexpr int kStaticScratchInts = 64 * 1024;
static __device__ __align__(256) int g_align_static_scratch[kStaticScratchInts];

constexpr int kMaxDevices = 64;

// Device address of the array above on the current device.  In host code the
// array's name is only a handle for the runtime, never a pointer a kernel could
// use, so the address is looked up once per device (with that device current).
int* static_scratch_on_current_device() {
  static std::mutex mu;
  static int* cached[kMaxDevices] = {};
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_last_error("moe_align_block_size_static: cudaGetDevice", err);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_align_static_scratch);
    if (err != cudaSuccess || !ptr) {
      set_last_error("moe_align_block_size_static: cudaGetSymbolAddress", err);
      return nullptr;
    }
    cached[dev] = static_cast<int*>(ptr);
  }
  return cached[dev];
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_moe_align_block_size_static(const void* topk_ids, int ids_dtype,
                                                   int64_t numel, int num_experts, int block_size,
                                                   const int32_t* expert_map,
                                                   int32_t* sorted_token_ids,
                                                   int64_t sorted_capacity, int32_t* expert_ids,
                                                   int64_t blocks_capacity,
                                                   int32_t* num_tokens_post_pad, void* stream) {
  if (numel < 0 || num_experts <= 0) return B200MOE_INVALID_ARG;
  const size_t need = grouping_workspace(numel, num_experts);
  if (need > sizeof(int) * static_cast<size_t>(kStaticScratchInts)) {
    static thread_local char msg[160];
    snprintf(msg, sizeof(msg),
             "moe_align_block_size_static: ceil(numel/2048)*num_experts = %zu ints exceeds the "
             "built-in scratch of %d ints; use b200moe_moe_align_block_size with a workspace",
             need / sizeof(int), kStaticScratchInts);
    set_last_error(msg, cudaErrorInvalidValue);
    return B200MOE_WORKSPACE_TOO_SMALL;
  }
  int* scratch = nullptr;
  if (need > 0) {
    scratch = static_scratch_on_current_device();
    if (!scratch) return B200MOE_CUDA_ERROR;
  }
  // Nothing in the scratch has to start at zero: the count pass overwrites every
  // entry the scan and placement passes read.
  return b200moe_moe_align_block_size(topk_ids, ids_dtype, numel, num_experts, block_size,
                                      expert_map, sorted_token_ids, sorted_capacity, expert_ids,
                                      blocks_capacity, num_tokens_post_pad, scratch,
                                      sizeof(int) * static_cast<size_t>(kStaticScratchInts), stream);
}

// ---- batched_moe_align_block_size and reorder_mxfp_scales ------------------------------

namespace b200moe {
namespace {

// One CTA: every batch (expert) b owns token slots [b*max_tokens, b*max_tokens + n_b); its
// run in sorted_ids starts at the padded prefix of the batches before it.
__global__ void __launch_bounds__(1024) batched_align_kernel(
    int num_batches, int max_tokens, int block_size, const int32_t* __restrict__ batch_num_tokens,
    int32_t* __restrict__ sorted_ids, int32_t* __restrict__ block_ids,
    int32_t* __restrict__ num_tokens_post_pad) {
  __shared__ int start[1024];
  __shared__ int warp_tot[32];
  const int t = threadIdx.x;
  const int blocks_per_batch = (max_tokens + block_size - 1) / block_size;
  const int sorted_size = blocks_per_batch * num_batches * block_size;
  const int sentinel = num_batches * max_tokens;
  for (int i = t; i < sorted_size; i += 1024) sorted_ids[i] = sentinel;
  for (int i = t; i < sorted_size / block_size; i += 1024) block_ids[i] = -1;
  const int n = t < num_batches ? batch_num_tokens[t] : 0;
  const int padded = (n + block_size - 1) / block_size * block_size;
  int incl = padded;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, off);
    if ((t & 31) >= off) incl += o;
  }
  if ((t & 31) == 31) warp_tot[t >> 5] = incl;
  __syncthreads();
  int base = 0;
  for (int w = 0; w < (t >> 5); ++w) base += warp_tot[w];
  start[t] = base + incl - padded;
  if (t == num_batches - 1) num_tokens_post_pad[0] = base + incl;
  __syncthreads();
  // fill: all threads walk all batches' tokens
  for (int b = 0; b < num_batches; ++b) {
    const int nb = batch_num_tokens[b];
    const int s0 = start[b];
    for (int i = t; i < nb; i += 1024) sorted_ids[s0 + i] = b * max_tokens + i;
    const int blocks = (nb + block_size - 1) / block_size;
    for (int i = t; i < blocks; i += 1024) block_ids[s0 / block_size + i] = b;
  }
}

// Activation scales of an MX-quantised A, [total_rows, scale_k] row-major with experts back
// to back, re-laid per expert as [scale_k, rows padded to 4] (M-major), experts back to back
// in the padded numbering.  One thread per destination byte.
__global__ void reorder_scales_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                      const int32_t* __restrict__ rows_per_expert, int num_experts,
                                      int scale_k, int64_t total_padded_rows) {
  const int64_t total = total_padded_rows * scale_k;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    // find the expert whose padded block holds flat destination byte i
    int64_t dst_off = 0, src_off = 0;
    uint8_t v = 0;
    for (int e = 0; e < num_experts; ++e) {
      const int r = rows_per_expert[e];
      const int pr = (r + 3) & ~3;
      const int64_t block = static_cast<int64_t>(pr) * scale_k;
      if (i < dst_off * scale_k + block) {
        const int64_t local = i - dst_off * scale_k;  // inside a [scale_k, pr] block
        const int kcol = static_cast<int>(local / pr);
        const int row = static_cast<int>(local % pr);
        if (row < r) v = src[(src_off + row) * scale_k + kcol];
        break;
      }
      dst_off += pr;
      src_off += r;
    }
    dst[i] = v;
  }
}

// Self-test of the bounded wait the tensor-core kernels rely on: waits on a barrier nobody
// will ever arrive at, with a short budget, and records the time-out in the status word.
}  // namespace
}  // namespace b200moe

extern "C" int b200moe_batched_moe_align_block_size(int max_tokens_per_batch, int block_size,
                                                    const int32_t* batch_num_tokens,
                                                    int num_batches, int32_t* sorted_ids,
                                                    int32_t* block_ids,
                                                    int32_t* num_tokens_post_pad, void* stream) {
  if (max_tokens_per_batch <= 0 || block_size <= 0 || num_batches <= 0 || num_batches > 1024 ||
      !batch_num_tokens || !sorted_ids || !block_ids || !num_tokens_post_pad)
    return B200MOE_INVALID_ARG;
  batched_align_kernel<<<1, 1024, 0, as_stream(stream)>>>(num_batches, max_tokens_per_batch,
                                                          block_size, batch_num_tokens, sorted_ids,
                                                          block_ids, num_tokens_post_pad);
  return launch_status("batched_align_kernel");
}

extern "C" int b200moe_reorder_mxfp_scales(const uint8_t* scales, const int32_t* rows_per_expert,
                                           int num_experts, int scale_k, int64_t total_padded_rows,
                                           uint8_t* out, void* stream) {
  if (num_experts < 0 || scale_k < 0 || total_padded_rows < 0) return B200MOE_INVALID_ARG;
  if (num_experts == 0 || scale_k == 0 || total_padded_rows == 0) return B200MOE_OK;
  if (!rows_per_expert || !out) return B200MOE_INVALID_ARG;
  const int64_t total = total_padded_rows * scale_k;
  int64_t blocks = (total + 255) / 256;
  if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
  reorder_scales_kernel<<<static_cast<int>(blocks), 256, 0, as_stream(stream)>>>(
      scales, out, rows_per_expert, num_experts, scale_k, total_padded_rows);
  return launch_status("reorder_scales_kernel");
}

extern "C" int b200moe_moe_lora_align_block_size(
    const void* topk_ids, int ids_dtype, int64_t num_tokens, int topk,
    const int32_t* token_lora_mapping, int num_experts, int block_size, int max_loras,
    int64_t max_num_tokens_padded, int64_t max_num_m_blocks, int32_t* sorted_token_ids,
    int32_t* expert_ids, int32_t* num_tokens_post_pad, const int32_t* adapter_enabled,
    const int32_t* lora_ids, const int32_t* expert_map, void* stream) {
  if (num_tokens < 0 || topk <= 0 || num_experts <= 0 || block_size <= 0 || max_loras <= 0 ||
      max_num_tokens_padded < 0 || max_num_m_blocks < 0 || !is_index_dtype(ids_dtype) ||
      !token_lora_mapping || !sorted_token_ids || !expert_ids || !num_tokens_post_pad ||
      !adapter_enabled || !lora_ids || (num_tokens > 0 && !topk_ids))
    return B200MOE_INVALID_ARG;
  if (num_experts > kMaxExperts || num_tokens * topk >= (1ll << 31)) return B200MOE_UNSUPPORTED;
  GroupParams p{topk_ids, ids_dtype, num_tokens * topk, num_experts, num_experts, expert_map, 0,
                block_size, token_lora_mapping, 0, topk};
  // lora_ids has max_loras + 1 entries: the real slots and a possible -1 for base-model tokens
  lora_align_kernel<<<max_loras + 1, kThreads, num_experts * kWarps * sizeof(int),
                      as_stream(stream)>>>(p, lora_ids, adapter_enabled, max_loras,
                                           sorted_token_ids, max_num_tokens_padded, expert_ids,
                                           max_num_m_blocks, num_tokens_post_pad);
  return launch_status("lora_align_kernel");
}
