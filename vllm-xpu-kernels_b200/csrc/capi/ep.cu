// Expert-parallel exchange over peer-mapped memory (NVLink / NVSwitch).
//
// Each rank owns a slice of the experts and a slice of the tokens.  All buffers
// that another rank touches live in a symmetric allocation whose per-rank base
// addresses every rank knows, so the exchange is stores to and loads from peer
// addresses issued by this library's own kernels — no collective library call,
// no host round trip for sizes:
//
//   put_counts   my rows per GLOBAL expert -> row `me` of every rank's [G, E]
//                count matrix                             (then a device barrier)
//   offsets      from the full matrix: for every expert, where my rows for it
//                start inside its owner's receive buffer (which is grouped by
//                expert, sources in rank order inside an expert); the rows each
//                of my own experts receives
//   dispatch     every (token, slot) row + activation scales -> its final place
//                in the owner's receive buffer, plus (my rank, my row) per row,
//                as bulk asynchronous copies; `push` is the older form that
//                takes rows already grouped by expert and plain stores
//                                                         (then a device barrier)
//   source_table for every row I sent, the address its result will have in the
//                owner's output buffer, and
//   gather       out[t] = sum_j w[t,j] * row at source_table[row_map[t,j]]: the
//                token's owner reads the k result rows from the peers and does
//                the weighted sum in the same pass ("pull" combine; the second
//                grouped GEMM stores locally at full speed), or
//   return_table (rank, row) of every received row -> the address of that row
//                in the sender's return buffer; the second grouped GEMM takes
//                this table and its epilogue stores straight to the peers
//                ("push" combine).
//
// The receive buffer is already in the order the grouped GEMM wants, so the
// receiving side runs no permutation at all.
//
// The barriers between the steps are kernels of this file too (ep_barrier): every
// rank stores a rising epoch number into a flag word it owns in each peer's
// allocation and then polls its own copy of the words until every peer's epoch
// has arrived.  The poll reads local memory only and is bounded by a wall-clock
// budget; on expiry the kernel leaves B200MOE_TIMEOUT in the device status word
// and returns, so a rank that never shows up costs the others one budget and a
// wrong result, not a hung GPU.  The bulk-copy kernels wait only on the mbarrier
// of their own copies, with a cycle budget.
#include "common.cuh"
#include "tcgen05.cuh"

namespace b200moe {
namespace {

constexpr int kMaxRanks = 16;

struct PeerPtrs {
  uint8_t* base[kMaxRanks];  // base of each rank's symmetric allocation
};

__global__ void ep_put_counts_kernel(const int32_t* __restrict__ send_counts, PeerPtrs peers,
                                     int64_t counts_off, int me, int n) {
  const int p = blockIdx.y;  // rank whose copy of the matrix is written
  int32_t* row = reinterpret_cast<int32_t*>(peers.base[p] + counts_off) + static_cast<int64_t>(me) * n;
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < n; e += gridDim.x * blockDim.x)
    row[e] = send_counts[e];
}

// counts[s*E + e] = rows rank s routes to global expert e (E = G * E_loc experts, expert e
// lives on rank e / E_loc).  One CTA.
__global__ void __launch_bounds__(1024) ep_offsets_kernel(
    const int32_t* __restrict__ counts, int me, int G, int E_loc,
    int32_t* __restrict__ my_prefix,         // [E+1] exclusive prefix of my own counts (send order)
    int32_t* __restrict__ dst_start,         // [E]   first row, in the owner's buffer, of my rows for e
    int32_t* __restrict__ rows_per_expert,   // [E_loc] rows each of MY experts receives
    int32_t* __restrict__ recv_total) {
  __shared__ int total[1024];
  __shared__ int before[1024];
  __shared__ int mine[1024];
  const int E = G * E_loc;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < G; ++s) {
      const int c = counts[s * E + e];
      if (s < me) b += c;
      t += c;
    }
    total[e] = t;
    before[e] = b;
    mine[e] = counts[me * E + e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int first = (e / E_loc) * E_loc;   // first expert of the owning rank
    int base = 0;
    for (int x = first; x < e; ++x) base += total[x];
    dst_start[e] = base + before[e];
    int pre = 0;
    for (int x = 0; x < e; ++x) pre += mine[x];
    my_prefix[e] = pre;
    if (e == E - 1) my_prefix[E] = pre + mine[e];
    if (e / E_loc == me) rows_per_expert[e - first] = total[e];
  }
  if (threadIdx.x == 0) {
    int t = 0;
    for (int x = me * E_loc; x < (me + 1) * E_loc; ++x) t += total[x];
    recv_total[0] = t;
  }
}

// One CTA per send row.  Send rows are grouped by global expert (stable), so a row's place
// in the owner's expert-grouped receive buffer follows from the count matrix alone; the
// receiver's first GEMM reads that buffer as it is.  Each row also carries where its result
// must return to: (sending rank, row of the sender's buffer).
__global__ void __launch_bounds__(128) ep_push_kernel(
    const uint4* __restrict__ send_rows, const uint8_t* __restrict__ send_scales,
    int64_t row_vecs, int64_t scale_bytes, int E, int E_loc, int me,
    const int32_t* __restrict__ my_prefix, const int32_t* __restrict__ dst_start, PeerPtrs peers,
    int64_t rows_off, int64_t scales_off, int64_t meta_off, int64_t capacity) {
  const int64_t i = blockIdx.x;
  if (i >= my_prefix[E]) return;
  int lo = 0, hi = E;  // largest e with my_prefix[e] <= i and a non-empty run
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (my_prefix[mid] <= i) lo = mid; else hi = mid;
  }
  const int e = lo;
  const int64_t j = dst_start[e] + (i - my_prefix[e]);
  if (j >= capacity) return;  // cannot happen with a worst-case capacity; never write out of bounds
  uint8_t* peer = peers.base[e / E_loc];
  uint4* dst = reinterpret_cast<uint4*>(peer + rows_off) + j * row_vecs;
  const uint4* src = send_rows + i * row_vecs;
  for (int64_t v = threadIdx.x; v < row_vecs; v += blockDim.x) dst[v] = src[v];
  if (send_scales) {
    const uint32_t* ss = reinterpret_cast<const uint32_t*>(send_scales + i * scale_bytes);
    uint32_t* ds = reinterpret_cast<uint32_t*>(peer + scales_off + j * scale_bytes);
    for (int64_t v = threadIdx.x; v < scale_bytes / 4; v += blockDim.x) ds[v] = ss[v];
  }
  if (threadIdx.x == 0)
    reinterpret_cast<int64_t*>(peer + meta_off)[j] = (static_cast<int64_t>(me) << 32) | i;
}

// meta[j] = (source rank << 32 | row in the source's send order) -> address of that row in
// the source rank's return buffer, as mapped into this process.
__global__ void ep_return_table_kernel(const int64_t* __restrict__ meta,
                                       const int32_t* __restrict__ recv_total, PeerPtrs peers,
                                       int64_t ret_off, int64_t row_bytes,
                                       int64_t* __restrict__ dst_addr) {
  const int64_t total = recv_total[0];
  for (int64_t j = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; j < total;
       j += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = meta[j];
    dst_addr[j] = reinterpret_cast<int64_t>(peers.base[m >> 32] + ret_off + (m & 0xffffffffll) * row_bytes);
  }
}

// Where the result of each of my send rows will sit: row i goes to expert e's owner at
// row j of its receive buffer (the same arithmetic as the push), and the owner's second
// GEMM leaves the result at row j of its output buffer.
__global__ void ep_source_table_kernel(const int32_t* __restrict__ my_prefix,
                                       const int32_t* __restrict__ dst_start, int E, int E_loc,
                                       PeerPtrs peers, int64_t out_off, int64_t row_bytes,
                                       int64_t capacity, int64_t* __restrict__ src_addr) {
  const int64_t total = my_prefix[E];
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int lo = 0, hi = E;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (my_prefix[mid] <= i) lo = mid; else hi = mid;
    }
    const int64_t j = dst_start[lo] + (i - my_prefix[lo]);
    src_addr[i] = j < capacity ? reinterpret_cast<int64_t>(peers.base[lo / E_loc] + out_off + j * row_bytes)
                               : 0;
  }
}

// One CTA per token.  The k source rows live in other GPUs' memory: each thread first issues
// the 16-byte loads of up to 8 rows, then accumulates them in slot order (fp32), so that
// several NVLink round trips are in flight per thread.  Sum order and rounding are those of
// moe_gather.
template <typename T>
__global__ void __launch_bounds__(256) ep_gather_kernel(T* __restrict__ out,
                                                        const float* __restrict__ weights,
                                                        const int32_t* __restrict__ row_map,
                                                        const int64_t* __restrict__ src_addr, int k,
                                                        int H) {
  constexpr int V = 16 / sizeof(T);
  constexpr int kBatch = 8;
  constexpr int kMaxTopK = 64;
  const int64_t t = blockIdx.x;
  __shared__ const T* rows[kMaxTopK];
  __shared__ float w[kMaxTopK];
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const int r = row_map[t * k + j];
    rows[j] = r < 0 ? nullptr : reinterpret_cast<const T*>(src_addr[r]);
    w[j] = weights[t * k + j];
  }
  __syncthreads();
  for (int c = threadIdx.x * V; c < H; c += blockDim.x * V) {
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    for (int j0 = 0; j0 < k; j0 += kBatch) {
      Vec<T, V> raw[kBatch];
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const T* p = j0 + b < k ? rows[j0 + b] : nullptr;
        if (p) raw[b] = *reinterpret_cast<const Vec<T, V>*>(p + c);
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        if (j0 + b < k && rows[j0 + b]) {
          const float wj = w[j0 + b];
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] += wj * Elem<T>::to_f32(raw[b].v[i]);
        }
      }
    }
    store_f32<T, V>(out + t * H + c, acc);
  }
}

// The same sum with the rows brought over by bulk async copies (TMA, no tensor map, no
// multicast): thread 0 issues one copy per source row -- a few KB each, which crosses
// NVLink as full-size requests -- into a two-stage shared-memory ring; all threads then add
// the k staged rows.  A work item is (token, column chunk); CTAs are persistent.  Every wait
// is bounded: on a timeout the CTA raises the status word and leaves after giving copies in
// flight time to land.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          sm100::smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(sm100::smem_u32(bar))
      : "memory");
}

template <typename T>
__global__ void __launch_bounds__(256) ep_gather_bulk_kernel(
    T* __restrict__ out, const float* __restrict__ weights, const int32_t* __restrict__ row_map,
    const int64_t* __restrict__ src_addr, int num_tokens, int k, int H, int chunk_elems,
    int n_chunks, int* __restrict__ status) {
  constexpr int V = 16 / sizeof(T);
  extern __shared__ __align__(128) uint8_t stage_smem[];
  __shared__ uint64_t full[2];
  __shared__ float w_s[2][64];
  __shared__ int ok_s[2][64];
  __shared__ int abort_flag;
  const int chunk_bytes = chunk_elems * static_cast<int>(sizeof(T));
  const int64_t items = static_cast<int64_t>(num_tokens) * n_chunks;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&full[0], 1);
    sm100::mbar_init(&full[1], 1);
    sm100::mbar_fence_init();
    abort_flag = 0;
  }
  __syncthreads();

  auto issue = [&](int64_t item, int s) {  // thread 0 only
    const int64_t t = item / n_chunks;
    const int col0 = static_cast<int>(item % n_chunks) * chunk_elems;
    const int cols = H - col0 < chunk_elems ? H - col0 : chunk_elems;
    const uint32_t bytes = static_cast<uint32_t>(cols) * sizeof(T);
    int valid = 0;
    for (int j = 0; j < k; ++j) {
      const int r = row_map[t * k + j];
      const int64_t a = r < 0 ? 0 : src_addr[r];
      ok_s[s][j] = a != 0;
      w_s[s][j] = weights[t * k + j];
      valid += a != 0;
    }
    sm100::mbar_arrive_expect_tx(&full[s], valid * bytes);
    for (int j = 0; j < k; ++j) {
      if (!ok_s[s][j]) continue;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(src_addr[row_map[t * k + j]]) +
                           static_cast<int64_t>(col0) * sizeof(T);
      bulk_load(stage_smem + (static_cast<size_t>(s) * k + j) * chunk_bytes, src, bytes, &full[s]);
    }
  };

  int64_t item = blockIdx.x;
  if (threadIdx.x == 0 && item < items) issue(item, 0);
  __syncthreads();
  for (int i = 0; item < items; ++i, item += gridDim.x) {
    const int s = i & 1;
    if (threadIdx.x == 0 && item + gridDim.x < items) issue(item + gridDim.x, s ^ 1);
    const bool got = sm100::mbar_wait(&full[s], (i >> 1) & 1, &abort_flag);
    if (__syncthreads_or(!got)) {
      if (threadIdx.x == 0) atomicExch(status, B200MOE_TIMEOUT);
      for (int n = 0; n < 64; ++n) __nanosleep(10000);  // let copies in flight land
      break;
    }
    const int64_t t = item / n_chunks;
    const int col0 = static_cast<int>(item % n_chunks) * chunk_elems;
    const int cols = H - col0 < chunk_elems ? H - col0 : chunk_elems;
    const uint8_t* base = stage_smem + static_cast<size_t>(s) * k * chunk_bytes;
    for (int c = threadIdx.x * V; c < cols; c += blockDim.x * V) {
      float acc[V];
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] = 0.f;
      for (int j = 0; j < k; ++j) {
        if (!ok_s[s][j]) continue;
        const Vec<T, V> raw = *reinterpret_cast<const Vec<T, V>*>(
            base + static_cast<size_t>(j) * chunk_bytes + static_cast<size_t>(c) * sizeof(T));
        const float wj = w_s[s][j];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] += wj * Elem<T>::to_f32(raw.v[e]);
      }
      store_f32<T, V>(out + t * H + col0 + c, acc);
    }
    __syncthreads();  // stage s may be refilled from the next iteration on
  }
}

__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(sm100::smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

// Dispatch without a local staging copy: one warp per (token, slot) pair.  Lane 0 brings the
// token's row (and its scales) into shared memory with one bulk async copy from local HBM --
// the k copies of a token hit L2 -- and sends it to its place in the owner's expert-grouped
// receive buffer with one bulk async store, so a row crosses NVLink as a few full-size
// writes.  Up to ~30 such warps are resident per SM, each with one row in flight.
__global__ void __launch_bounds__(32) ep_dispatch_bulk_kernel(
    const uint8_t* __restrict__ hidden, const uint8_t* __restrict__ scales, int64_t row_bytes,
    int64_t scale_bytes, const void* __restrict__ ids, int ids_dtype,
    const int32_t* __restrict__ row_map, int64_t pairs, int k, int E_loc, int me,
    const int32_t* __restrict__ my_prefix, const int32_t* __restrict__ dst_start, PeerPtrs peers,
    int64_t rows_off, int64_t scales_off, int64_t meta_off, int64_t capacity,
    int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t row_smem[];
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  const int lane = threadIdx.x;
  if (lane == 0) {
    sm100::mbar_init(&bar, 1);
    sm100::mbar_fence_init();
    abort_flag = 0;
  }
  __syncwarp();
  const bool bulk_scales = scales && scale_bytes % 16 == 0;
  uint32_t parity = 0;
  for (int64_t p = blockIdx.x; p < pairs; p += gridDim.x) {
    const int i = row_map[p];
    if (i < 0) continue;
    const int e = static_cast<int>(load_index(ids, ids_dtype, p));
    const int64_t j = dst_start[e] + (i - my_prefix[e]);
    if (j >= capacity) continue;  // cannot happen with a worst-case capacity
    const int64_t t = p / k;
    uint8_t* peer = peers.base[e / E_loc];
    if (lane == 0) {
      const uint32_t total = static_cast<uint32_t>(row_bytes + (bulk_scales ? scale_bytes : 0));
      sm100::mbar_arrive_expect_tx(&bar, total);
      bulk_load(row_smem, hidden + t * row_bytes, static_cast<uint32_t>(row_bytes), &bar);
      if (bulk_scales)
        bulk_load(row_smem + row_bytes, scales + t * scale_bytes, static_cast<uint32_t>(scale_bytes), &bar);
      if (!sm100::mbar_wait(&bar, parity, &abort_flag)) {
        atomicExch(status, B200MOE_TIMEOUT);
        for (int n = 0; n < 64; ++n) __nanosleep(10000);  // let the copies in flight land
      } else {
        bulk_store(peer + rows_off + j * row_bytes, row_smem, static_cast<uint32_t>(row_bytes));
        if (bulk_scales)
          bulk_store(peer + scales_off + j * scale_bytes, row_smem + row_bytes,
                     static_cast<uint32_t>(scale_bytes));
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        reinterpret_cast<int64_t*>(peer + meta_off)[j] = (static_cast<int64_t>(me) << 32) | i;
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the buffer is free again
      }
    }
    parity ^= 1u;
    __syncwarp();
    if (abort_flag) return;
    if (scales && !bulk_scales) {  // ragged scale rows: plain 4-byte stores
      const uint32_t* ss = reinterpret_cast<const uint32_t*>(scales + t * scale_bytes);
      uint32_t* ds = reinterpret_cast<uint32_t*>(peer + scales_off + j * scale_bytes);
      for (int64_t v = lane; v < scale_bytes / 4; v += 32) ds[v] = ss[v];
    }
  }
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ---- cross-rank barrier ----------------------------------------------------------
// Flag words: kBarrierChannels x kMaxRanks u32 in every rank's allocation; word [c][s] of
// rank r is written by rank s only.  A channel's epoch counts the barriers this rank has
// run on it and lives in this rank's own memory; ranks call the barriers of a channel in
// the same order, so equal epochs mean the same barrier.  "Arrived" is epoch - want >= 0 in
// wrap-around arithmetic: a fast peer that is already one barrier further still counts.
constexpr int kBarrierChannels = B200MOE_EP_BARRIER_CHANNELS;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// One warp; lane s talks to rank s.  Everything this rank's earlier kernels on the stream
// wrote to peer memory is ordered before the flag by the system-scope fence + release store;
// the acquire load orders the peers' writes before whatever this stream runs next.
__device__ __forceinline__ void ep_barrier_body(const PeerPtrs& peers, int64_t flags_off, int me,
                                                int G, int channel, uint32_t* epoch,
                                                long long budget_ns, int* status) {
  const int s = threadIdx.x;
  const uint32_t want = epoch[channel] + 1u;
  bool late = false;
  if (s < G) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(peers.base[s] + flags_off) + channel * kMaxRanks + me, want);
    const uint32_t* mine =
        reinterpret_cast<const uint32_t*>(peers.base[me] + flags_off) + channel * kMaxRanks + s;
    const unsigned long long t0 = globaltimer_ns();
    while (static_cast<int32_t>(ld_acquire_sys(mine) - want) < 0) {
      if (static_cast<long long>(globaltimer_ns() - t0) > budget_ns) {
        late = true;
        break;
      }
      __nanosleep(200);
    }
  }
  const bool any_late = __any_sync(0xffffffffu, late);
  if (s == 0) {
    epoch[channel] = want;  // the count advances either way: a late peer's next barrier still matches
    if (any_late) atomicExch(status, B200MOE_TIMEOUT);
  }
}

__global__ void __launch_bounds__(32) ep_barrier_kernel(PeerPtrs peers, int64_t flags_off, int me,
                                                        int G, int channel, uint32_t* epoch,
                                                        long long budget_ns, int* status) {
  ep_barrier_body(peers, flags_off, me, G, channel, epoch, budget_ns, status);
}

// All ranks of the barrier as the CTAs of ONE cooperative launch over one device buffer
// (CTA r is rank r; its flag words start at flags + r * channels * kMaxRanks, its epochs at
// epochs + r * channels).  Kernels that wait on one another must not be separate launches
// on one GPU, so this is how the protocol is exercised on a single device; ranks in
// `absent_mask` return at once without arriving, which is how a missing rank is played.
__global__ void __launch_bounds__(32) ep_barrier_emulated_kernel(uint32_t* flags, uint32_t* epochs,
                                                                 int G, int channel,
                                                                 uint32_t absent_mask,
                                                                 long long budget_ns, int* status) {
  const int me = blockIdx.x;
  if ((absent_mask >> me) & 1u) return;
  PeerPtrs peers;
  for (int r = 0; r < kMaxRanks; ++r)
    peers.base[r] = reinterpret_cast<uint8_t*>(flags + static_cast<int64_t>(r < G ? r : 0) * kBarrierChannels * kMaxRanks);
  ep_barrier_body(peers, 0, me, G, channel, epochs + me * kBarrierChannels, budget_ns, status);
}

// ---- token-level exchange: a token crosses to a rank once, however many of its experts
// live there -----------------------------------------------------------------------------
// hits[t, r] = r if any of token t's expert ids lives on rank r, else -1: the "ids" matrix
// that turns the row-grouping and dispatch kernels above into a token-to-rank exchange
// (experts_per_rank = 1, top-k = world).
__global__ void ep_rank_hits_kernel(const void* __restrict__ ids, int ids_dtype, int T, int k,
                                    int E_loc, int G, int32_t* __restrict__ hits) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  uint32_t mask = 0;
  for (int j = 0; j < k; ++j) {
    const int64_t e = load_index(ids, ids_dtype, static_cast<int64_t>(t) * k + j);
    if (e >= 0 && e < static_cast<int64_t>(E_loc) * G) mask |= 1u << static_cast<int>(e / E_loc);
  }
  for (int r = 0; r < G; ++r) hits[static_cast<int64_t>(t) * G + r] = (mask >> r) & 1u ? r : -1;
}

// side[t] = (k expert ids as i32 | k routing weights as f32 | padding to `stride` words):
// what travels with a token.
__global__ void ep_pack_routing_kernel(const void* __restrict__ ids, int ids_dtype,
                                       const float* __restrict__ weights, int64_t n, int k,
                                       int stride, int32_t* __restrict__ side) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const int64_t t = i / k;
  const int j = static_cast<int>(i - t * k);
  side[t * stride + j] = static_cast<int32_t>(load_index(ids, ids_dtype, i));
  side[t * stride + k + j] = __float_as_int(weights[i]);
}

// The receiving side of the same: for the *recv_total tokens that arrived, ids become LOCAL
// expert ids (or -1 where the expert lives elsewhere) and the weights are copied; every
// later row of the worst-case buffer gets -1, so whatever an earlier call left there is
// never routed.
__global__ void ep_unpack_routing_kernel(const int32_t* __restrict__ side,
                                         const int32_t* __restrict__ recv_total, int64_t n, int k,
                                         int stride, int me, int E_loc,
                                         int32_t* __restrict__ ids_local,
                                         float* __restrict__ weights) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const int64_t t = i / k;
  const int j = static_cast<int>(i - t * k);
  int32_t id = -1;
  float w = 0.f;
  if (t < recv_total[0]) {
    const int32_t local = side[t * stride + j] - me * E_loc;
    if (local >= 0 && local < E_loc) {
      id = local;
      w = __int_as_float(side[t * stride + k + j]);
    }
  }
  ids_local[i] = id;
  weights[i] = w;
}

long long barrier_budget_ns(int64_t budget_ns) {
  if (budget_ns > 0) return budget_ns;
  // read per call: a host may shorten it for a drill without restarting
  const char* env = getenv("B200MOE_EP_BARRIER_TIMEOUT_MS");
  const long long ms = env ? atoll(env) : 0;
  return (ms > 0 ? ms : 30000ll) * 1000000ll;
}

bool load_peers(const int64_t* peer_bases_host, int G, PeerPtrs* out) {
  if (!peer_bases_host || G <= 0 || G > kMaxRanks) return false;
  for (int i = 0; i < kMaxRanks; ++i)
    out->base[i] = i < G ? reinterpret_cast<uint8_t*>(peer_bases_host[i]) : nullptr;
  return true;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_ep_barrier(const int64_t* peer_bases_host, int64_t flags_offset, int my_rank,
                                  int world, int channel, uint32_t* epochs, int64_t budget_ns,
                                  void* stream) {
  PeerPtrs peers;
  if (!load_peers(peer_bases_host, world, &peers) || my_rank < 0 || my_rank >= world || channel < 0 ||
      channel >= kBarrierChannels || !epochs || flags_offset < 0 || flags_offset % 4 != 0)
    return B200MOE_INVALID_ARG;
  int* status = device_status_word();
  if (!status) return B200MOE_CUDA_ERROR;
  ep_barrier_kernel<<<1, 32, 0, as_stream(stream)>>>(peers, flags_offset, my_rank, world, channel,
                                                     epochs, barrier_budget_ns(budget_ns), status);
  return launch_status("ep_barrier_kernel");
}

extern "C" int b200moe_ep_barrier_emulated(uint32_t* flags, uint32_t* epochs, int world, int channel,
                                           uint32_t absent_mask, int64_t budget_ns, void* stream) {
  if (!flags || !epochs || world <= 0 || world > kMaxRanks || channel < 0 || channel >= kBarrierChannels)
    return B200MOE_INVALID_ARG;
  int* status = device_status_word();
  if (!status) return B200MOE_CUDA_ERROR;
  long long budget = barrier_budget_ns(budget_ns);
  void* args[] = {&flags, &epochs, &world, &channel, &absent_mask, &budget, &status};
  // cooperative: all `world` CTAs are resident together, or the launch fails
  const cudaError_t err = cudaLaunchCooperativeKernel(
      reinterpret_cast<const void*>(ep_barrier_emulated_kernel), dim3(world), dim3(32), args, 0,
      as_stream(stream));
  if (err != cudaSuccess) {
    set_last_error("cudaLaunchCooperativeKernel(ep_barrier_emulated_kernel)", err);
    return B200MOE_CUDA_ERROR;
  }
  count_launch();
  return B200MOE_OK;
}

extern "C" int b200moe_ep_rank_hits(const void* topk_ids, int ids_dtype, int num_tokens, int topk,
                                    int experts_per_rank, int world, int32_t* hits, void* stream) {
  if (!topk_ids || !hits || !is_index_dtype(ids_dtype) || num_tokens < 0 || topk <= 0 ||
      experts_per_rank <= 0 || world <= 0 || world > kMaxRanks)
    return B200MOE_INVALID_ARG;
  if (num_tokens == 0) return B200MOE_OK;
  ep_rank_hits_kernel<<<(num_tokens + 255) / 256, 256, 0, as_stream(stream)>>>(
      topk_ids, ids_dtype, num_tokens, topk, experts_per_rank, world, hits);
  return launch_status("ep_rank_hits_kernel");
}

extern "C" int b200moe_ep_pack_routing(const void* topk_ids, int ids_dtype, const float* topk_weights,
                                       int num_tokens, int topk, int side_stride, int32_t* side,
                                       void* stream) {
  if (!topk_ids || !topk_weights || !side || !is_index_dtype(ids_dtype) || num_tokens < 0 || topk <= 0 ||
      side_stride < 2 * topk)
    return B200MOE_INVALID_ARG;
  if (num_tokens == 0) return B200MOE_OK;
  const int64_t n = static_cast<int64_t>(num_tokens) * topk;
  ep_pack_routing_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, as_stream(stream)>>>(
      topk_ids, ids_dtype, topk_weights, n, topk, side_stride, side);
  return launch_status("ep_pack_routing_kernel");
}

extern "C" int b200moe_ep_unpack_routing(const int32_t* side, const int32_t* recv_total,
                                         int64_t capacity_tokens, int topk, int side_stride,
                                         int my_rank, int experts_per_rank, int32_t* ids_local,
                                         float* weights, void* stream) {
  if (!side || !recv_total || !ids_local || !weights || capacity_tokens < 0 || topk <= 0 ||
      side_stride < 2 * topk || my_rank < 0 || experts_per_rank <= 0)
    return B200MOE_INVALID_ARG;
  if (capacity_tokens == 0) return B200MOE_OK;
  const int64_t n = capacity_tokens * topk;
  ep_unpack_routing_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, as_stream(stream)>>>(
      side, recv_total, n, topk, side_stride, my_rank, experts_per_rank, ids_local, weights);
  return launch_status("ep_unpack_routing_kernel");
}

extern "C" int b200moe_ep_put_counts(const int32_t* send_counts, int num_counts,
                                     const int64_t* peer_bases_host, int64_t counts_offset,
                                     int my_rank, int world, void* stream) {
  PeerPtrs peers;
  if (!send_counts || num_counts <= 0 || !load_peers(peer_bases_host, world, &peers) || my_rank < 0 ||
      my_rank >= world)
    return B200MOE_INVALID_ARG;
  ep_put_counts_kernel<<<dim3((num_counts + 255) / 256, world), 256, 0, as_stream(stream)>>>(
      send_counts, peers, counts_offset, my_rank, num_counts);
  return launch_status("ep_put_counts_kernel");
}

extern "C" int b200moe_ep_offsets(const int32_t* counts, int my_rank, int world,
                                  int experts_per_rank, int32_t* my_prefix, int32_t* dst_start,
                                  int32_t* rows_per_expert, int32_t* recv_total, void* stream) {
  if (!counts || !my_prefix || !dst_start || !rows_per_expert || !recv_total || world <= 0 ||
      world > kMaxRanks || my_rank < 0 || my_rank >= world || experts_per_rank <= 0 ||
      world * experts_per_rank > 1024)
    return B200MOE_INVALID_ARG;
  ep_offsets_kernel<<<1, 1024, 0, as_stream(stream)>>>(counts, my_rank, world, experts_per_rank,
                                                       my_prefix, dst_start, rows_per_expert, recv_total);
  return launch_status("ep_offsets_kernel");
}

extern "C" int b200moe_ep_push(const void* send_rows, const void* send_scales, int64_t num_rows,
                               int64_t row_bytes, int64_t scale_row_bytes, int my_rank, int world,
                               int experts_per_rank, const int32_t* my_prefix,
                               const int32_t* dst_start, const int64_t* peer_bases_host,
                               int64_t rows_offset, int64_t scales_offset, int64_t meta_offset,
                               int64_t capacity, void* stream) {
  PeerPtrs peers;
  if (!send_rows || !my_prefix || !dst_start || !load_peers(peer_bases_host, world, &peers) ||
      row_bytes % 16 != 0 || scale_row_bytes % 4 != 0 || num_rows < 0 || experts_per_rank <= 0)
    return B200MOE_INVALID_ARG;
  if (num_rows == 0) return B200MOE_OK;
  ep_push_kernel<<<static_cast<unsigned>(num_rows), 128, 0, as_stream(stream)>>>(
      reinterpret_cast<const uint4*>(send_rows), reinterpret_cast<const uint8_t*>(send_scales),
      row_bytes / 16, scale_row_bytes, world * experts_per_rank, experts_per_rank, my_rank, my_prefix,
      dst_start, peers, rows_offset, scales_offset, meta_offset, capacity);
  return launch_status("ep_push_kernel");
}

extern "C" int b200moe_ep_return_table(const int64_t* meta, const int32_t* recv_total, int world,
                                       const int64_t* peer_bases_host, int64_t return_offset,
                                       int64_t row_bytes, int64_t* dst_addr, void* stream) {
  PeerPtrs peers;
  if (!meta || !recv_total || !dst_addr || !load_peers(peer_bases_host, world, &peers))
    return B200MOE_INVALID_ARG;
  ep_return_table_kernel<<<kNumSMs, 256, 0, as_stream(stream)>>>(meta, recv_total, peers,
                                                                 return_offset, row_bytes, dst_addr);
  return launch_status("ep_return_table_kernel");
}

extern "C" int b200moe_ep_source_table(const int32_t* my_prefix, const int32_t* dst_start,
                                       int64_t num_rows, int world, int experts_per_rank,
                                       const int64_t* peer_bases_host, int64_t out_offset,
                                       int64_t row_bytes, int64_t capacity, int64_t* src_addr,
                                       void* stream) {
  PeerPtrs peers;
  if (!my_prefix || !dst_start || !src_addr || !load_peers(peer_bases_host, world, &peers) ||
      experts_per_rank <= 0 || num_rows < 0 || row_bytes <= 0)
    return B200MOE_INVALID_ARG;
  if (num_rows == 0) return B200MOE_OK;
  const int64_t blocks = (num_rows + 255) / 256;
  ep_source_table_kernel<<<static_cast<unsigned>(blocks < kNumSMs * 4 ? blocks : kNumSMs * 4), 256, 0,
                           as_stream(stream)>>>(my_prefix, dst_start, world * experts_per_rank,
                                                experts_per_rank, peers, out_offset, row_bytes,
                                                capacity, src_addr);
  return launch_status("ep_source_table_kernel");
}

extern "C" int b200moe_ep_gather(void* out, int dtype, const float* weights, const int32_t* row_map,
                                 const int64_t* src_addr, int T, int k, int H, void* stream) {
  if (T < 0 || k <= 0 || k > 64 || H <= 0) return B200MOE_INVALID_ARG;
  if (T == 0) return B200MOE_OK;
  if (!out || !weights || !row_map || !src_addr) return B200MOE_INVALID_ARG;
  if ((H * dtype_size(dtype)) % 16 != 0) return B200MOE_INVALID_ARG;
  // B200MOE_EP_GATHER=loads selects the plain-load kernel (kept for comparison).
  const char* mode = getenv("B200MOE_EP_GATHER");
  const bool bulk = !(mode && strcmp(mode, "loads") == 0);
  return B200MOE_DISPATCH_FLOAT(dtype, [&] {
    constexpr int V = 16 / sizeof(scalar_t);
    cudaStream_t st = as_stream(stream);
    if (!bulk) {
      int threads = (H / V + 31) / 32 * 32;
      threads = threads > 256 ? 256 : threads;
      ep_gather_kernel<scalar_t><<<T, threads, 0, st>>>(reinterpret_cast<scalar_t*>(out), weights,
                                                        row_map, src_addr, k, H);
      return launch_status("ep_gather_kernel");
    }
    // column chunk: k staged rows per stage within 48 KB, two stages, two CTAs per SM
    const int row_bytes = H * static_cast<int>(sizeof(scalar_t));
    int cmax = (48 * 1024 / k) / 16 * 16;
    if (cmax > row_bytes) cmax = row_bytes;
    const int n_chunks = (row_bytes + cmax - 1) / cmax;
    const int chunk_bytes = ((row_bytes + n_chunks - 1) / n_chunks + 15) / 16 * 16;
    const size_t smem = 2 * static_cast<size_t>(k) * chunk_bytes;
    struct Tag {};
    const int arc = ensure_dynamic_smem<Tag>(ep_gather_bulk_kernel<scalar_t>, 100 * 1024,
                                             "cudaFuncSetAttribute(ep_gather_bulk_kernel)");
    if (arc != B200MOE_OK) return arc;
    int* status = device_status_word();
    if (!status) return static_cast<int>(B200MOE_CUDA_ERROR);
    const int64_t items = static_cast<int64_t>(T) * n_chunks;
    const int grid = static_cast<int>(items < 2 * kNumSMs ? items : 2 * kNumSMs);
    ep_gather_bulk_kernel<scalar_t><<<grid, 256, smem, st>>>(
        reinterpret_cast<scalar_t*>(out), weights, row_map, src_addr, T, k, H,
        chunk_bytes / static_cast<int>(sizeof(scalar_t)), n_chunks, status);
    return launch_status("ep_gather_bulk_kernel");
  });
}

extern "C" int b200moe_ep_dispatch(const void* hidden, const void* scales, int64_t row_bytes,
                                   int64_t scale_row_bytes, const void* topk_ids, int ids_dtype,
                                   const int32_t* row_map, int num_tokens, int topk, int my_rank,
                                   int world, int experts_per_rank, const int32_t* my_prefix,
                                   const int32_t* dst_start, const int64_t* peer_bases_host,
                                   int64_t rows_offset, int64_t scales_offset, int64_t meta_offset,
                                   int64_t capacity, void* stream) {
  PeerPtrs peers;
  if (!hidden || !topk_ids || !row_map || !my_prefix || !dst_start || !is_index_dtype(ids_dtype) ||
      !load_peers(peer_bases_host, world, &peers) || row_bytes <= 0 || row_bytes % 16 != 0 ||
      scale_row_bytes % 4 != 0 || num_tokens < 0 || topk <= 0 || experts_per_rank <= 0)
    return B200MOE_INVALID_ARG;
  if (num_tokens == 0) return B200MOE_OK;
  const size_t smem = static_cast<size_t>(row_bytes) + (scale_row_bytes % 16 == 0 ? scale_row_bytes : 0);
  if (smem > 200 * 1024) return B200MOE_UNSUPPORTED;
  int* status = device_status_word();
  if (!status) return B200MOE_CUDA_ERROR;
  struct DispatchTag {};
  const int arc = ensure_dynamic_smem<DispatchTag>(ep_dispatch_bulk_kernel, 200 * 1024,
                                                   "cudaFuncSetAttribute(ep_dispatch_bulk_kernel)");
  if (arc != B200MOE_OK) return arc;
  int per_sm = static_cast<int>((216 * 1024) / (smem + 1024));
  per_sm = per_sm > 32 ? 32 : (per_sm < 1 ? 1 : per_sm);
  const int64_t pairs = static_cast<int64_t>(num_tokens) * topk;
  const int64_t want = static_cast<int64_t>(kNumSMs) * per_sm;
  ep_dispatch_bulk_kernel<<<static_cast<unsigned>(pairs < want ? pairs : want), 32, smem,
                            as_stream(stream)>>>(
      reinterpret_cast<const uint8_t*>(hidden), reinterpret_cast<const uint8_t*>(scales), row_bytes,
      scale_row_bytes, topk_ids, ids_dtype, row_map, pairs, topk, experts_per_rank, my_rank,
      my_prefix, dst_start, peers, rows_offset, scales_offset, meta_offset, capacity, status);
  return launch_status("ep_dispatch_bulk_kernel");
}
