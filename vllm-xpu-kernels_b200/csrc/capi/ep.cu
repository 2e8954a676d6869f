// Expert-parallel exchange over peer-mapped memory (NVLink / NVSwitch).
//
// Each rank owns a slice of the experts and a slice of the tokens.  All buffers
// that another rank writes live in a symmetric allocation whose per-rank base
// addresses every rank knows, so the exchange is plain stores to peer
// addresses from ordinary kernels — no collective library call, no host round
// trip for sizes:
//
//   put_counts   my per-destination row counts -> row `me` of every rank's
//                [G, G] count matrix                     (then a device barrier)
//   offsets      from the full matrix: where my rows go inside each
//                destination's receive buffer, where each source's rows start
//                in mine, how many rows I receive; marks the unused tail of my
//                receive buffer as "no expert"
//   push         my packed send rows (+ activation scales + local expert ids)
//                -> the destinations' receive buffers     (then a device barrier)
//   return_table for every row of the local, expert-permuted GEMM output: the
//                peer address it must end up at (the slot of the source rank's
//                return buffer the token came from); the second grouped GEMM
//                takes this table and its epilogue stores straight to the peers.
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
                                     int64_t counts_off, int me, int G) {
  const int d = threadIdx.x;   // entry of my row
  const int p = blockIdx.x;    // rank whose copy of the matrix is written
  if (d < G && p < G)
    reinterpret_cast<int32_t*>(peers.base[p] + counts_off)[me * G + d] = send_counts[d];
}

// counts[s*G + d] = rows rank s sends to rank d.
__global__ void ep_offsets_kernel(const int32_t* __restrict__ counts, int me, int G,
                                  int32_t* __restrict__ send_base,   // [G+1] prefix of my row
                                  int32_t* __restrict__ dst_base,    // [G] my first row inside dest d's buffer
                                  int32_t* __restrict__ recv_base,   // [G+1] first row of source s in my buffer
                                  int32_t* __restrict__ recv_expert, int64_t capacity) {
  __shared__ int total;
  if (threadIdx.x == 0) {
    int run = 0;
    for (int d = 0; d < G; ++d) { send_base[d] = run; run += counts[me * G + d]; }
    send_base[G] = run;
    run = 0;
    for (int s = 0; s < G; ++s) { recv_base[s] = run; run += counts[s * G + me]; }
    recv_base[G] = run;
    total = run;
    for (int d = 0; d < G; ++d) {
      int before = 0;
      for (int s = 0; s < me; ++s) before += counts[s * G + d];
      dst_base[d] = before;
    }
  }
  __syncthreads();
  // rows of my receive buffer that nobody writes this step route to no expert
  for (int64_t i = total + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < capacity;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    recv_expert[i] = -1;
}

// One CTA per send row.
__global__ void __launch_bounds__(128) ep_push_kernel(
    const uint4* __restrict__ send_rows, const uint8_t* __restrict__ send_scales,
    const int32_t* __restrict__ send_expert, int64_t row_vecs, int64_t scale_bytes, int G,
    const int32_t* __restrict__ send_base, const int32_t* __restrict__ dst_base, PeerPtrs peers,
    int64_t rows_off, int64_t scales_off, int64_t expert_off, int64_t capacity) {
  const int64_t i = blockIdx.x;
  if (i >= send_base[G]) return;
  int d = 0;
  while (d + 1 < G && send_base[d + 1] <= i) ++d;
  const int64_t j = dst_base[d] + (i - send_base[d]);
  if (j >= capacity) return;  // cannot happen with a worst-case capacity; never write out of bounds
  uint8_t* peer = peers.base[d];
  uint4* dst = reinterpret_cast<uint4*>(peer + rows_off) + j * row_vecs;
  const uint4* src = send_rows + i * row_vecs;
  for (int64_t v = threadIdx.x; v < row_vecs; v += blockDim.x) dst[v] = src[v];
  if (send_scales) {
    const uint32_t* ss = reinterpret_cast<const uint32_t*>(send_scales + i * scale_bytes);
    uint32_t* ds = reinterpret_cast<uint32_t*>(peer + scales_off + j * scale_bytes);
    for (int64_t v = threadIdx.x; v < scale_bytes / 4; v += blockDim.x) ds[v] = ss[v];
  }
  if (threadIdx.x == 0) reinterpret_cast<int32_t*>(peer + expert_off)[j] = send_expert[i];
}

// row_map[j] = row of the local permuted buffers that received row j went to (-1: none).
__global__ void ep_return_table_kernel(const int32_t* __restrict__ row_map,
                                       const int32_t* __restrict__ recv_base,
                                       const int32_t* __restrict__ counts, int me, int G,
                                       PeerPtrs peers, int64_t ret_off, int64_t row_bytes,
                                       int64_t* __restrict__ dst_addr) {
  const int64_t total = recv_base[G];
  for (int64_t j = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; j < total;
       j += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int r = row_map[j];
    if (r < 0) continue;
    int s = 0;
    while (s + 1 < G && recv_base[s + 1] <= j) ++s;
    int64_t slot = j - recv_base[s];
    for (int d = 0; d < me; ++d) slot += counts[s * G + d];  // rows rank s sent to ranks before me
    dst_addr[r] = reinterpret_cast<int64_t>(peers.base[s] + ret_off + slot * row_bytes);
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

extern "C" int b200moe_ep_put_counts(const int32_t* send_counts, const int64_t* peer_bases_host,
                                     int64_t counts_offset, int my_rank, int world, void* stream) {
  PeerPtrs peers;
  if (!send_counts || !load_peers(peer_bases_host, world, &peers) || my_rank < 0 || my_rank >= world)
    return B200MOE_INVALID_ARG;
  ep_put_counts_kernel<<<world, 32, 0, as_stream(stream)>>>(send_counts, peers, counts_offset,
                                                            my_rank, world);
  return launch_status("ep_put_counts_kernel");
}

extern "C" int b200moe_ep_offsets(const int32_t* counts, int my_rank, int world, int32_t* send_base,
                                  int32_t* dst_base, int32_t* recv_base, int32_t* recv_expert,
                                  int64_t capacity, void* stream) {
  if (!counts || !send_base || !dst_base || !recv_base || !recv_expert || world <= 0 ||
      world > kMaxRanks || my_rank < 0 || my_rank >= world || capacity < 0)
    return B200MOE_INVALID_ARG;
  ep_offsets_kernel<<<kNumSMs, 256, 0, as_stream(stream)>>>(counts, my_rank, world, send_base,
                                                            dst_base, recv_base, recv_expert, capacity);
  return launch_status("ep_offsets_kernel");
}

extern "C" int b200moe_ep_push(const void* send_rows, const void* send_scales,
                               const int32_t* send_expert, int64_t num_rows, int64_t row_bytes,
                               int64_t scale_row_bytes, int world, const int32_t* send_base,
                               const int32_t* dst_base, const int64_t* peer_bases_host,
                               int64_t rows_offset, int64_t scales_offset, int64_t expert_offset,
                               int64_t capacity, void* stream) {
  PeerPtrs peers;
  if (!send_rows || !send_expert || !send_base || !dst_base || !load_peers(peer_bases_host, world, &peers) ||
      row_bytes % 16 != 0 || scale_row_bytes % 4 != 0 || num_rows < 0)
    return B200MOE_INVALID_ARG;
  if (num_rows == 0) return B200MOE_OK;
  ep_push_kernel<<<static_cast<unsigned>(num_rows), 128, 0, as_stream(stream)>>>(
      reinterpret_cast<const uint4*>(send_rows), reinterpret_cast<const uint8_t*>(send_scales),
      send_expert, row_bytes / 16, scale_row_bytes, world, send_base, dst_base, peers, rows_offset,
      scales_offset, expert_offset, capacity);
  return launch_status("ep_push_kernel");
}

extern "C" int b200moe_ep_return_table(const int32_t* row_map, const int32_t* recv_base,
                                       const int32_t* counts, int my_rank, int world,
                                       const int64_t* peer_bases_host, int64_t return_offset,
                                       int64_t row_bytes, int64_t capacity, int64_t* dst_addr,
                                       void* stream) {
  PeerPtrs peers;
  if (!row_map || !recv_base || !counts || !dst_addr || !load_peers(peer_bases_host, world, &peers) ||
      my_rank < 0 || my_rank >= world)
    return B200MOE_INVALID_ARG;
  if (capacity == 0) return B200MOE_OK;
  ep_return_table_kernel<<<kNumSMs * 2, 256, 0, as_stream(stream)>>>(
      row_map, recv_base, counts, my_rank, world, peers, return_offset, row_bytes, dst_addr);
  return launch_status("ep_return_table_kernel");
}
