// Expert-parallel exchange over peer-mapped memory (NVLink / NVSwitch).
//
// Each rank owns a slice of the experts and a slice of the tokens.  All buffers
// that another rank writes live in a symmetric allocation whose per-rank base
// addresses every rank knows, so the exchange is plain stores to peer
// addresses from ordinary kernels — no collective library call, no host round
// trip for sizes:
//
//   put_counts   my rows per GLOBAL expert -> row `me` of every rank's [G, E]
//                count matrix                             (then a device barrier)
//   offsets      from the full matrix: for every expert, where my rows for it
//                start inside its owner's receive buffer (which is grouped by
//                expert, sources in rank order inside an expert); the rows each
//                of my own experts receives
//   push         my send rows (grouped by global expert, as remap_hidden_states
//                leaves them) + activation scales -> their final place in the
//                owners' receive buffers, plus (my rank, my row) per row
//                                                         (then a device barrier)
//   return_table (rank, row) of every received row -> the address of that row
//                in the sender's return buffer; the second grouped GEMM takes
//                this table and its epilogue stores straight to the peers.
//
// The receive buffer is already in the order the grouped GEMM wants, so the
// receiving side runs no permutation at all.
//
// The barriers between the steps are issued by the caller on the same stream.
// Every kernel here only writes; nothing spins on remote data.
#include "common.cuh"

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

bool load_peers(const int64_t* peer_bases_host, int G, PeerPtrs* out) {
  if (!peer_bases_host || G <= 0 || G > kMaxRanks) return false;
  for (int i = 0; i < kMaxRanks; ++i)
    out->base[i] = i < G ? reinterpret_cast<uint8_t*>(peer_bases_host[i]) : nullptr;
  return true;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

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
