// Grouped GEMM of the fused-MoE layer on the Blackwell tensor cores.
//
//   D[rows of expert e, :] = A[rows of expert e, :] * B_e (+ bias_e)
//
// One persistent, warp-specialised CTA per SM:
//   warp 0      TMA producer: 128-byte-swizzled tiles of A and B into a ring of
//               shared-memory stages, one mbarrier pair per stage;
//   warp 1      owns tensor memory and issues tcgen05.mma (one elected lane);
//   warps 2..   read accumulators out of tensor memory (tcgen05.ld), apply
//               scales / bias / the gated activation and store rows.
// Every role walks the same static tile sequence (tile = blockIdx.x + i*grid),
// so no tile index is passed between warps.  Expert row ranges come from
// rows_per_expert on the device: each CTA prefix-sums it into shared memory and
// finds a tile's expert by binary search, so there is no host sync, no helper
// launch and no per-call workspace.  M tiles start at the expert's first row;
// rows past the expert's end are loaded (they belong to the next expert or are
// zero-filled by TMA) but never stored.
//
// FP8 with 128x128 fp32 weight scales and per-row-per-128 activation scales
// cannot be folded into the MMA, so for that recipe the MMA warp writes one
// partial accumulator per 128 of K into a ring of tensor-memory buffers and the
// reader warps add scale * partial into fp32 registers while the next partial
// is being computed.
//
// All waits are bounded: a wait that runs out of budget raises a CTA-wide abort
// flag, records B200MOE_TIMEOUT in a device status word and the CTA tears down
// (frees tensor memory) instead of hanging.
#include <cuda.h>

#include <stdlib.h>

#include <mutex>

#include "common.cuh"
#include "tcgen05.cuh"

namespace b200moe {

__device__ int g_device_status = 0;

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int kStageRowBytes = 128;  // one swizzle row: 64 bf16 or 128 fp8 along the box's inner dim
constexpr int kMaxExpertsSmem = 1024;
constexpr int kSwizzleGroupM = 8;
constexpr int kMaxKBlocks = 160;  // K <= 20480 for the FP8 block-scaled recipe

// KIND_F8S: e4m3 x e4m3 with POWER-OF-TWO block scales (per row per 128 of K for A, per
// 128x128 block for B), applied by the tensor core itself (kind::mxf8f6f4.block_scale, UE8M0
// factors in tensor memory): one accumulation phase per tile, no promotion in registers.
enum : int { KIND_F16 = 0, KIND_F8 = 1, KIND_F8S = 2 };
constexpr int kSfaBytes = 512;    // per group of four K blocks: one scale word (4 x e8m0) per row of the A tile
constexpr int kSfbBytes = 1024;   // ... and per weight column of the tile (256)
constexpr int kSfGroupBytes = kSfaBytes + kSfbBytes;
constexpr int kSfaCol = 256;      // tensor-memory columns of the scale words (KIND_F8S: one
constexpr int kSfbCol = 260;      //   256-column accumulator at column 0)

// Internal epilogue code next to the three public ones: the split gated tile with any of the
// gated activations and the layer's clamp, selected at run time.  It is an instantiation of
// its own so that the SiLU epilogue of the default path keeps its registers to itself.
constexpr int kEpiGatedAny = 3;

struct GemmParams {
  const float* a_scale;
  const float* b_scale;
  const void* bias;
  int bias_dtype;
  void* D;
  float* d_scale;
  int d_dtype;
  const int32_t* rows_per_expert;
  int64_t R;
  int N, K, E;
  int ldd;     // row stride of D in elements
  int ab_fmt;  // operand format code of the instruction descriptor
  const int64_t* d_row_ptr;  // optional per-row destination addresses (store epilogue)
  float alpha, limit;
  int act;               // B200MOE_ACT_* of the split gated epilogue
  float act_p0, act_p1;  // its parameters (swiglustep limit; situ betas)
  float clamp;           // > 0: gate <= clamp and |up| <= clamp before the activation
  int pow2_scales;       // the quantising epilogue rounds its scales up to powers of two
};

struct TileCoord {
  int expert;
  int row_start;   // first row of A / D
  int rows_valid;  // rows of this tile that belong to the expert
  int n_tile;
};

struct Schedule {
  int tile_prefix[kMaxExpertsSmem + 1];
  int row_prefix[kMaxExpertsSmem + 1];
  int num_experts;
  int n_tiles;
  int tile_m;  // rows per scheduled M tile: 128, or 256 for a CTA pair
};

// Prefix sums of rows and of M tiles per expert, by warp 0 of the CTA.
__device__ __forceinline__ void build_schedule(Schedule& s, const int32_t* rows_per_expert, int E,
                                               int64_t R, int n_tiles, int tile_m) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int tile_run = 0;
    long long row_run = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + lane;
      long long rows = e < E ? rows_per_expert[e] : 0;
      if (rows < 0) rows = 0;
      long long incl_rows = rows;
      int tiles = static_cast<int>((rows + tile_m - 1) / tile_m);
      int incl_tiles = tiles;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const long long r = __shfl_up_sync(0xffffffffu, incl_rows, off);
        const int t = __shfl_up_sync(0xffffffffu, incl_tiles, off);
        if (lane >= off) {
          incl_rows += r;
          incl_tiles += t;
        }
      }
      if (e < E) {
        long long rs = row_run + incl_rows - rows;
        s.row_prefix[e] = static_cast<int>(rs < R ? rs : R);
        s.tile_prefix[e] = tile_run + incl_tiles - tiles;
      }
      row_run += __shfl_sync(0xffffffffu, incl_rows, 31);
      tile_run += __shfl_sync(0xffffffffu, incl_tiles, 31);
    }
    if (lane == 0) {
      s.row_prefix[E] = static_cast<int>(row_run < R ? row_run : R);
      s.tile_prefix[E] = tile_run;
      s.num_experts = E;
      s.n_tiles = n_tiles;
      s.tile_m = tile_m;
    }
  }
}

__device__ __forceinline__ int total_tiles(const Schedule& s) {
  return s.tile_prefix[s.num_experts] * s.n_tiles;
}

// Tile t -> coordinates.  M tiles are visited in groups of kSwizzleGroupM with
// the M index fastest, so a weight tile is reused by neighbouring CTAs while it
// is still in L2.
__device__ __forceinline__ TileCoord decode_tile(const Schedule& s, int t) {
  const int mt = s.tile_prefix[s.num_experts];
  const int per_group = kSwizzleGroupM * s.n_tiles;
  const int g = t / per_group;
  const int first_m = g * kSwizzleGroupM;
  const int gsize = (mt - first_m) < kSwizzleGroupM ? (mt - first_m) : kSwizzleGroupM;
  const int within = t - g * per_group;
  const int m = first_m + within % gsize;
  TileCoord c;
  c.n_tile = within / gsize;
  int lo = 0, hi = s.num_experts;  // largest e with tile_prefix[e] <= m
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s.tile_prefix[mid] <= m) lo = mid; else hi = mid;
  }
  c.expert = lo;
  const int local = m - s.tile_prefix[lo];
  const int rows_e = s.row_prefix[lo + 1] - s.row_prefix[lo];
  c.row_start = s.row_prefix[lo] + local * s.tile_m;
  const int left = rows_e - local * s.tile_m;
  c.rows_valid = left < s.tile_m ? (left < 0 ? 0 : left) : s.tile_m;
  return c;
}

// Epilogue math uses the special-function unit directly (ex2.approx, rcp.approx: two
// MUFU operations per sigmoid, relative error ~1e-6).  The correctly rounded
// reciprocal and expf are instruction sequences an order of magnitude longer, and
// the reader warps run the epilogue while the MMA warp waits for them; the results
// are rounded to bf16 or e4m3 right after.
__device__ __forceinline__ float fast_sigmoid(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return r;
}

__device__ __forceinline__ float silu_f32(float g) { return g * fast_sigmoid(g); }

__device__ __forceinline__ float swiglu_oai_f32(float g, float u, float alpha, float limit) {
  g = fminf(g, limit);
  u = fmaxf(fminf(u, limit), -limit);
  return (u + 1.0f) * (g * fast_sigmoid(g * alpha));
}

// act(gate) * up for the activations other than SiLU, in fp32 (one rounding, at the store).
__device__ __forceinline__ float gated_act_f32(int act, float g, float u, float p0, float p1) {
  switch (act) {
    case B200MOE_ACT_GELU:
      return g * 0.5f * (1.0f + erff(g * 0.70710678118654752440f)) * u;
    case B200MOE_ACT_GELU_TANH: {
      const float inner = 0.79788456080286535588f * (g + 0.044715f * (g * g * g));
      return 0.5f * g * (1.0f + tanhf(inner)) * u;
    }
    case B200MOE_ACT_SWIGLUSTEP:
      return fminf(silu_f32(g), p0) * fmaxf(fminf(u, p0), -p0);
    case B200MOE_ACT_SITU: {
      const float ag = p0 * tanhf(g / p0) * fast_sigmoid(g);
      const float au = p1 > 0.0f ? p1 * tanhf(u / p1) : u;
      return ag * au;
    }
    default:
      return silu_f32(g) * u;
  }
}

__device__ __forceinline__ float load_bias(const void* bias, int dtype, int64_t i) {
  if (dtype == B200MOE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[i]);
  if (dtype == B200MOE_F16) return __half2float(reinterpret_cast<const __half*>(bias)[i]);
  return reinterpret_cast<const float*>(bias)[i];
}

// Stores `n` (multiple of 8) fp32 values as 16-bit elements with 16-byte stores.
template <int NV>
__device__ __forceinline__ void store_row16(void* D, int d_dtype, int64_t elem_off,
                                            const float (&v)[NV], int n_valid) {
  if (d_dtype == B200MOE_BF16) {
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(D) + elem_off;
#pragma unroll
    for (int i = 0; i < NV; i += 8) {
      if (i + 8 <= n_valid) {
        Vec<__nv_bfloat16, 8> o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16_rn(v[i + j]);
        *reinterpret_cast<Vec<__nv_bfloat16, 8>*>(p + i) = o;
      } else {
        for (int j = 0; j < 8; ++j)
          if (i + j < n_valid) p[i + j] = __float2bfloat16_rn(v[i + j]);
      }
    }
  } else {
    __half* p = reinterpret_cast<__half*>(D) + elem_off;
#pragma unroll
    for (int i = 0; i < NV; i += 8) {
      if (i + 8 <= n_valid) {
        Vec<__half, 8> o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = __float2half_rn(v[i + j]);
        *reinterpret_cast<Vec<__half, 8>*>(p + i) = o;
      } else {
        for (int j = 0; j < 8; ++j)
          if (i + j < n_valid) p[i + j] = __float2half_rn(v[i + j]);
      }
    }
  }
}

template <int KIND_, bool B_MN_MAJOR_, bool PROMOTE_, int BN_, int EPI_, int STAGES_,
          bool PAIR_ = false, bool OFFLOAD_ = false>
struct Config {
  static constexpr int KIND = KIND_;
  // PAIR: two CTAs of a cluster share each MMA (cta_group::2).  The scheduled tile is
  // 256 x BN; each CTA loads its own 128 rows of A and half of the B columns, so the
  // bytes a CTA pulls from L2 per flop drop by a third against two independent CTAs.
  static constexpr bool PAIR = PAIR_;
  static constexpr int TILE_M = PAIR_ ? 256 : 128;
  static constexpr int B_COLS = PAIR_ ? BN_ / 2 : BN_;  // B columns this CTA loads
  static constexpr bool B_MN_MAJOR = B_MN_MAJOR_;
  static constexpr bool PROMOTE = PROMOTE_;
  static constexpr int BN = BN_;
  static constexpr int EPI = EPI_;
  static constexpr int STAGES = STAGES_;
  static constexpr bool SCALED = KIND_ == KIND_F8S;
  static constexpr int ELT = KIND == KIND_F16 ? 2 : 1;
  static constexpr int BK = kStageRowBytes / ELT;       // elements of K per stage
  static constexpr int UMMA_K = 32 / ELT;                // K per MMA instruction
  static constexpr int A_BYTES = BM * kStageRowBytes;
  static constexpr int B_BYTES = B_COLS * kStageRowBytes;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int CHUNK_COLS = kStageRowBytes / ELT;  // N columns per MN-major TMA box
  static constexpr int N_CHUNKS = B_COLS / CHUNK_COLS;      // boxes this CTA loads per stage
  // tensor-memory accumulator ring: all 512 columns, or one 256-column buffer next to the
  // scale columns (the accumulator then leaves tensor memory once per tile, at its end)
  static constexpr int ACC_BUFS = SCALED ? 1 : 512 / BN;
  static constexpr int SF_BYTES = SCALED ? 2 * kSfGroupBytes : 0;   // two scale groups after the operand ring
  static constexpr int TMEM_COLS = 512;
  static constexpr int EPI_WARPS = 8;                    // two reader warps per TMEM lane quadrant
  static constexpr int THREADS = 128 + EPI_WARPS * 32;   // warps 0..3: producer, MMA, 2 spare
  static constexpr int CPT = BN / 2;                     // accumulator columns per reader thread
  static constexpr int NCH = CPT / 32;                   // 32-column tcgen05.ld chunks per thread
  static constexpr bool GATED_SPLIT =
      EPI == B200MOE_EPI_SILU_MUL || EPI == kEpiGatedAny;  // tile = [gate half | up half]
  // The fp8 128x256 tile keeps 128 fp32 accumulators per reader thread: the reader
  // warpgroups take registers from the producer/MMA warpgroup (setmaxnreg).
  static constexpr bool REBALANCE_REGS = BN == 256;
  static constexpr int XCHG = (EPI_ == B200MOE_EPI_SILU_MUL || EPI_ == kEpiGatedAny) ? 256 : 1;
  // OFFLOAD: the reader warps leave the finished tile as 16-bit rows in shared memory and go
  // straight back to the accumulators; the two spare warps of the producer warpgroup write
  // it to global memory while the next tile is being computed.
  static constexpr bool OFFLOAD = OFFLOAD_;
  static constexpr int OUT_ROW_BYTES = BN_ * 2;
  static constexpr int OUT_BYTES = OFFLOAD_ ? BM * OUT_ROW_BYTES : 0;
  static constexpr size_t SMEM_BYTES =
      1024 + static_cast<size_t>(STAGES) * STAGE_BYTES + SF_BYTES + OUT_BYTES;
  static constexpr int SB_SMEM = PROMOTE_ ? 2 * kMaxKBlocks : 1;
  static_assert(!SCALED || (BN_ == 256 && !PROMOTE_ && !PAIR_ && B_MN_MAJOR_),
                "the tensor-core-scaled FP8 kernel is laid out for single CTAs and 256-column tiles");
  static_assert(!(GATED_SPLIT && B_MN_MAJOR_ && !PAIR_ && N_CHUNKS < 2),
                "a split gated tile needs two weight boxes");
  static_assert(!PAIR_ || BN_ == 256, "CTA pairs are laid out for 256-column tiles");
  static_assert(!OFFLOAD_ || (PROMOTE_ && EPI_ == B200MOE_EPI_STORE && BN_ == 256 && KIND_ != KIND_F8S),
                "the offloaded store is laid out for the promoting FP8 kernel's 128 x 256 store tiles");
  static_assert(SMEM_BYTES > 116 * 1024, "one CTA per SM is assumed by the tensor-memory allocation");
  static_assert(NCH == 2 || NCH == 4, "reader pipeline alternates two 32-column buffers");
};

struct alignas(8) Barriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tfull[4];
  uint64_t tempty[4];
  uint64_t sready;  // this tile's staged scales are in shared memory (one arrival per reader warp)
  uint64_t sffull[2];   // KIND_F8S: a group of scale words is in shared memory / has been copied
  uint64_t sfempty[2];  //           to tensor memory
  uint64_t ofull;       // OFFLOAD: the staged output tile is complete (one arrival per reader warp)
  uint64_t oempty;      //          ... has been written out (one arrival per store warp)
};

// Tensor-memory column (inside one accumulator buffer) of chunk c of a reader
// thread in column group g.  In a split gated tile the thread reads CPT/2 gate
// columns and the CPT/2 up columns that go with them.
template <typename C>
__device__ __forceinline__ int chunk_tmem_col(int g, int c) {
  if (C::GATED_SPLIT)
    return c < C::NCH / 2 ? g * (C::CPT / 2) + c * 32
                          : C::BN / 2 + g * (C::CPT / 2) + (c - C::NCH / 2) * 32;
  return g * C::CPT + c * 32;
}

// Column of the full-N problem that tensor-memory column `tcol` of tile `n_tile` holds.
template <typename C>
__device__ __forceinline__ int problem_col(int n_tile, int tcol, int N) {
  if (C::GATED_SPLIT)
    return (tcol < C::BN / 2 ? 0 : N / 2 - C::BN / 2) + n_tile * (C::BN / 2) + tcol;
  return n_tile * C::BN + tcol;
}

// acc[0..32) += s * t[0..32) with the packed two-wide fp32 FMA of sm_100 (or a
// plain copy when the tile has a single accumulation phase).
template <bool PROMOTE>
__device__ __forceinline__ void accumulate32(float* acc, const float (&t)[32], float s) {
  if constexpr (PROMOTE) {
    const float2 s2 = make_float2(s, s);
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const float2 r = __ffma2_rn(s2, make_float2(t[j], t[j + 1]), make_float2(acc[j], acc[j + 1]));
      acc[j] = r.x;
      acc[j + 1] = r.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) acc[j] = t[j];
  }
}

// The same store for a whole warp, coalesced.  Each lane holds NV consecutive columns of
// its own row (lane = row), so a direct store instruction would touch 32 different rows
// with 16 bytes each -- 32 separate lines per instruction, which costs the readers about
// 2 us per 128x256 tile.  Here every 32-column chunk goes through a 2 KB per-warp buffer
// in shared memory (16-byte pieces XOR-swizzled so that neither side has bank conflicts)
// and comes back with four lanes per row: a store instruction then writes 8 rows x 64
// contiguous bytes.  `row_base(rr)` returns the address of element 0 of row rr of this
// warp's 32 rows (or nullptr to skip the row); all 32 lanes must call this together.
template <int NV, typename RowBase>
__device__ __forceinline__ void store_rows_coalesced(uint4* wbuf, int lane, int d_dtype, int col0,
                                                     const float (&v)[NV], int n_valid,
                                                     RowBase row_base) {
  static_assert(NV % 32 == 0, "whole 32-column chunks");
  uint8_t* rows[4];
#pragma unroll
  for (int it = 0; it < 4; ++it) rows[it] = reinterpret_cast<uint8_t*>(row_base(it * 8 + (lane >> 2)));
  const int qq = lane & 3;
#pragma unroll
  for (int c = 0; c < NV / 32; ++c) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = v[c * 32 + q * 8 + 2 * i], b = v[c * 32 + q * 8 + 2 * i + 1];
        if (d_dtype == B200MOE_BF16) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
          w[i] = *reinterpret_cast<const uint32_t*>(&h);
        } else {
          const __half2 h = __floats2half2_rn(a, b);
          w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
      }
      wbuf[lane * 4 + (q ^ ((lane >> 1) & 3))] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int rr = it * 8 + (lane >> 2);
      const uint4 piece = wbuf[rr * 4 + (qq ^ ((rr >> 1) & 3))];
      const int col = c * 32 + qq * 8;  // first of the 8 columns this lane stores
      if (rows[it]) {
        uint8_t* dst = rows[it] + static_cast<int64_t>(col0 + col) * 2;
        if (col + 8 <= n_valid) {
          *reinterpret_cast<uint4*>(dst) = piece;
        } else {  // ragged right edge: element by element
          const uint16_t* e = reinterpret_cast<const uint16_t*>(&piece);
          for (int j = 0; j < 8; ++j)
            if (col + j < n_valid) reinterpret_cast<uint16_t*>(dst)[j] = e[j];
        }
      }
    }
    __syncwarp();
  }
}

// acc[] += the expert's bias for the columns this reader thread holds.
template <typename C>
__device__ __forceinline__ void add_bias(const GemmParams& p, const TileCoord& tc, int g,
                                         float (&acc)[C::CPT]) {
  if (!p.bias) return;
#pragma unroll
  for (int c = 0; c < C::NCH; ++c) {
    const int col0 = problem_col<C>(tc.n_tile, chunk_tmem_col<C>(g, c), p.N);
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N)
        acc[c * 32 + j] += load_bias(p.bias, p.bias_dtype,
                                     static_cast<int64_t>(tc.expert) * p.N + col0 + j);
  }
}

// Offloaded store, reader side: row `row` of the tile (this thread's) as 16-bit values into
// the staging tile.  A row is BN * 2 bytes = 32 pieces of 16 bytes; piece c of row r sits at
// piece (c ^ (r & 31)) of that row, so that the 32 lanes of a reader warp (32 rows, same
// piece) and the 32 lanes of a store warp (one row, 32 pieces) both spread over all banks.
template <typename C>
__device__ __forceinline__ void stage_row(uint8_t* out_stage, int row, int g, int d_dtype,
                                          const float (&acc)[C::CPT]) {
  uint8_t* rbase = out_stage + row * C::OUT_ROW_BYTES;
  const int sw = row & 31;
#pragma unroll
  for (int i = 0; i < C::CPT / 8; ++i) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float a = acc[i * 8 + 2 * k], b = acc[i * 8 + 2 * k + 1];
      if (d_dtype == B200MOE_BF16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        w[k] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __half2 h = __floats2half2_rn(a, b);
        w[k] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    const int piece = g * (C::CPT / 8) + i;
    *reinterpret_cast<uint4*>(rbase + ((piece ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Offloaded store, store-warp side: rows [row_lo, row_hi) of the staged tile to D, one
// 512-byte row per warp instruction.
template <typename C>
__device__ __forceinline__ void write_staged_rows(const GemmParams& p, const TileCoord& tc,
                                                  int rank, const uint8_t* out_stage, int row_lo,
                                                  int row_hi, int lane) {
  const int col = tc.n_tile * C::BN + lane * 8;   // first of this lane's 8 columns
  int valid = tc.rows_valid - rank * BM;           // rows of this CTA's 128 that exist
  if (row_hi > valid) row_hi = valid;
  if (col >= p.N) return;
  uint8_t* d0 = reinterpret_cast<uint8_t*>(p.D) +
                (static_cast<int64_t>(tc.row_start) + rank * BM) * p.ldd * 2 + static_cast<int64_t>(col) * 2;
  const bool whole = col + 8 <= p.N;
  // 40 registers per thread in this warpgroup: two rows in flight, one running pointer
  const int64_t row_pitch = static_cast<int64_t>(p.ldd) * 2;
  uint8_t* dst = d0 + row_lo * row_pitch;
  int r = row_lo;
  if (whole) {
    for (; r + 2 <= row_hi; r += 2, dst += 2 * row_pitch) {
      const uint4 v0 = *reinterpret_cast<const uint4*>(out_stage + r * C::OUT_ROW_BYTES + ((lane ^ (r & 31)) << 4));
      const uint4 v1 = *reinterpret_cast<const uint4*>(out_stage + (r + 1) * C::OUT_ROW_BYTES +
                                                       ((lane ^ ((r + 1) & 31)) << 4));
      *reinterpret_cast<uint4*>(dst) = v0;
      *reinterpret_cast<uint4*>(dst + row_pitch) = v1;
    }
  }
  for (; r < row_hi; ++r, dst += row_pitch) {
    const uint4 v = *reinterpret_cast<const uint4*>(out_stage + r * C::OUT_ROW_BYTES + ((lane ^ (r & 31)) << 4));
    if (whole) {
      *reinterpret_cast<uint4*>(dst) = v;
    } else {  // ragged right edge: element by element
      const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
      for (int j = 0; j < 8; ++j)
        if (col + j < p.N) reinterpret_cast<uint16_t*>(dst)[j] = e[j];
    }
  }
}

// acc[] -> global memory for one row of one tile.
template <typename C>
__device__ __forceinline__ void tile_epilogue(const GemmParams& p, const TileCoord& tc, int g,
                                              bool row_ok, int64_t grow, float (&acc)[C::CPT],
                                              float* xchg, uint4* wbuf) {
  constexpr int CPT = C::CPT;
  const int lane = threadIdx.x & 31;
  // rows of this warp: grow - lane .. grow - lane + 31, valid below `warp_rows_valid`
  const int64_t warp_row0 = grow - lane;
  const int warp_rows_valid = tc.rows_valid - static_cast<int>(warp_row0 - tc.row_start);
  auto local_row = [&](int rr) -> void* {  // element 0 of row rr in D
    if (rr >= warp_rows_valid) return nullptr;
    return reinterpret_cast<uint8_t*>(p.D) + (warp_row0 + rr) * p.ldd * 2;
  };
  add_bias<C>(p, tc, g, acc);
  if constexpr (C::EPI == B200MOE_EPI_STORE) {
    const int col0 = tc.n_tile * C::BN + g * CPT;
    if (col0 < p.N) {
      auto remote_row = [&](int rr) -> void* {  // the row's home may be another GPU's memory
        return rr < warp_rows_valid ? reinterpret_cast<void*>(p.d_row_ptr[warp_row0 + rr]) : nullptr;
      };
      if (p.d_row_ptr) store_rows_coalesced<CPT>(wbuf, lane, p.d_dtype, col0, acc, p.N - col0, remote_row);
      else store_rows_coalesced<CPT>(wbuf, lane, p.d_dtype, col0, acc, p.N - col0, local_row);
    }
  } else if constexpr (C::GATED_SPLIT) {
    constexpr int HALF = CPT / 2;
    const int half_n = p.N / 2;
    const int col0 = tc.n_tile * (C::BN / 2) + g * HALF;
    float o[HALF];
    if constexpr (C::EPI == B200MOE_EPI_SILU_MUL) {
#pragma unroll
      for (int j = 0; j < HALF; ++j) o[j] = silu_f32(acc[j]) * acc[HALF + j];
    } else {  // the layer's clamp and the other gated activations, same place, same pass
#pragma unroll  // fully: the accumulators stay in registers only with static indices
      for (int j = 0; j < HALF; ++j) {
        float gte = acc[j], up = acc[HALF + j];
        if (p.clamp > 0.0f) {
          gte = fminf(gte, p.clamp);
          up = fmaxf(fminf(up, p.clamp), -p.clamp);
        }
        o[j] = gated_act_f32(p.act, gte, up, p.act_p0, p.act_p1);
      }
    }
    if (p.d_dtype == B200MOE_E4M3) {
      // per-token-group-128 quantisation of the activation: the 128 output columns of
      // this tile are one group, held by two threads (column groups 0 and 1)
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < HALF; ++j) amax = fmaxf(amax, fabsf(o[j]));
      const int row = threadIdx.x & 127;  // quad*32 + lane for reader warps 4..11
      xchg[g * 128 + row] = amax;
      // the two warps that hold the same 32 rows (column groups 0 and 1) meet on their own barrier
      asm volatile("bar.sync %0, 64;" ::"r"(1 + ((threadIdx.x >> 5) & 3)) : "memory");
      amax = fmaxf(amax, xchg[(g ^ 1) * 128 + row]);
      float s = fmaxf(amax * (1.0f / 448.0f), 1.0f / (448.0f * 512.0f));
      if (p.pow2_scales) {  // next power of two: the consumer applies it inside the MMA
        const uint32_t bits = __float_as_uint(s);
        s = __uint_as_float(((bits & 0x007FFFFFu) ? bits + 0x00800000u : bits) & 0xFF800000u);
      }
      const float inv_s = 1.0f / s;
      if (row_ok && col0 < half_n) {
        if (g == 0) p.d_scale[grow * (half_n / 128) + tc.n_tile] = s;
        uint8_t* dst = reinterpret_cast<uint8_t*>(p.D) + grow * p.ldd + col0;
#pragma unroll
        for (int j = 0; j < HALF; j += 16) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float v0 = fmaxf(-448.0f, fminf(o[j + 4 * i + 0] * inv_s, 448.0f));
            const float v1 = fmaxf(-448.0f, fminf(o[j + 4 * i + 1] * inv_s, 448.0f));
            const float v2 = fmaxf(-448.0f, fminf(o[j + 4 * i + 2] * inv_s, 448.0f));
            const float v3 = fmaxf(-448.0f, fminf(o[j + 4 * i + 3] * inv_s, 448.0f));
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v0, v1), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v2, v3), __NV_SATFINITE, __NV_E4M3);
            w[i] = lo | (hi << 16);
          }
          *reinterpret_cast<uint4*>(dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    } else if (col0 < half_n) {
      store_rows_coalesced<HALF>(wbuf, lane, p.d_dtype, col0, o, half_n - col0, local_row);
    }
  } else {  // SWIGLU_OAI: (gate, up) pairs are adjacent columns
    const int col0 = tc.n_tile * C::BN + g * CPT;
    float o[CPT / 2];
#pragma unroll
    for (int j = 0; j < CPT / 2; ++j) {
      float gte = acc[2 * j], up = acc[2 * j + 1];
      if (p.clamp > 0.0f) {  // the layer's clamp on the interleaved halves
        gte = fminf(gte, p.clamp);
        up = fmaxf(fminf(up, p.clamp), -p.clamp);
      }
      o[j] = swiglu_oai_f32(gte, up, p.alpha, p.limit);
    }
    if (col0 < p.N)
      store_rows_coalesced<CPT / 2>(wbuf, lane, p.d_dtype, col0 / 2, o, (p.N - col0) / 2, local_row);
  }
}

// One pipeline stage of operands for K block `kb` of tile `tc`: this CTA's A box
// (its 128 rows) and its B box(es).  In a CTA pair, rank 1 takes the second 128 rows
// and the second half of the tile's columns, and every load reports to the leader's
// barrier.
template <typename C>
__device__ __forceinline__ void issue_stage(const CUtensorMap& map_a, const CUtensorMap& map_b,
                                            const GemmParams& p, const TileCoord& tc, int kb,
                                            int rank, uint8_t* stage_smem, uint64_t* bar) {
  uint8_t* a_dst = stage_smem;
  uint8_t* b_dst = stage_smem + C::A_BYTES;
  auto b_box = [&](int off, int x, int y, int z) {
    if constexpr (C::PAIR) tma_load_3d_pair(b_dst + off, &map_b, bar, x, y, z);
    else tma_load_3d(b_dst + off, &map_b, bar, x, y, z);
  };
  if constexpr (C::PAIR) tma_load_2d_pair(a_dst, &map_a, bar, kb * C::BK, tc.row_start + rank * BM);
  else tma_load_2d(a_dst, &map_a, bar, kb * C::BK, tc.row_start);
  const int tcol0 = rank * C::B_COLS;  // first tile column this CTA loads
  if constexpr (C::B_MN_MAJOR) {
#pragma unroll
    for (int c = 0; c < C::N_CHUNKS; ++c)
      b_box(c * (C::BK * kStageRowBytes),
            problem_col<C>(tc.n_tile, tcol0 + c * C::CHUNK_COLS, p.N), kb * C::BK, tc.expert);
  } else if constexpr (C::GATED_SPLIT && !C::PAIR) {
    b_box(0, kb * C::BK, tc.n_tile * (C::BN / 2), tc.expert);
    b_box((C::BN / 2) * kStageRowBytes, kb * C::BK, p.N / 2 + tc.n_tile * (C::BN / 2), tc.expert);
  } else {
    b_box(0, kb * C::BK, problem_col<C>(tc.n_tile, tcol0, p.N), tc.expert);
  }
}

template <typename C>
__global__ void __launch_bounds__(C::THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Schedule sched;
  __shared__ Barriers bars;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float xchg[2][C::XCHG];  // group-amax exchange of the quantising epilogue, by tile parity
  __shared__ float sb_smem[2][C::SB_SMEM];  // weight scales of the tile's two column blocks
  __shared__ uint4 epi_buf[C::OFFLOAD ? 1 : C::EPI_WARPS][128];   // per reader warp: 32 rows x 64 B for coalesced stores

  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = C::GATED_SPLIT ? (p.N / 2 + C::BN / 2 - 1) / (C::BN / 2)
                                     : (p.N + C::BN - 1) / C::BN;
  const int num_kb = (p.K + C::BK - 1) / C::BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&bars.full[s], 1);
      mbar_init(&bars.empty[s], 1);
    }
    for (int b = 0; b < C::ACC_BUFS; ++b) {
      mbar_init(&bars.tfull[b], 1);
      mbar_init(&bars.tempty[b], C::EPI_WARPS * (C::PAIR ? 2 : 1));  // both CTAs' readers
    }
    mbar_init(&bars.sready, C::EPI_WARPS);
    mbar_init(&bars.ofull, C::EPI_WARPS);
    mbar_init(&bars.oempty, 2);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars.sffull[b], 1);
      mbar_init(&bars.sfempty[b], 1);
    }
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  build_schedule(sched, p.rows_per_expert, p.E, p.R, n_tiles, C::TILE_M);
  if (warp == 1) {
    if constexpr (C::PAIR) {
      tmem_alloc_pair(&tmem_base_slot, C::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&tmem_base_slot, C::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (C::PAIR) cluster_sync();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const int rank = C::PAIR ? static_cast<int>(cluster_ctarank()) : 0;
  const int sched_id = C::PAIR ? blockIdx.x / 2 : blockIdx.x;      // position in the tile sequence
  const int sched_stride = C::PAIR ? gridDim.x / 2 : gridDim.x;
  const uint32_t tmem_base = tmem_base_slot;
  const int num_tiles = total_tiles(sched);
  volatile int* abort_p = &abort_flag;

  if (warp < 4) {
    if constexpr (C::REBALANCE_REGS) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0 && lane == 0) {
      // ---------------- TMA producer ----------------
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = sched_id; t < num_tiles && ok; t += sched_stride) {
        const TileCoord tc = decode_tile(sched, t);
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          ok = mbar_wait(&bars.empty[stage], phase ^ 1u, abort_p);
          if (!ok) break;
          // the leader's barrier counts the bytes of both CTAs of a pair
          if (rank == 0)
            mbar_arrive_expect_tx(&bars.full[stage], C::STAGE_BYTES * (C::PAIR ? 2 : 1));
          issue_stage<C>(map_a, map_b, p, tc, kb, rank, tiles + stage * C::STAGE_BYTES,
                         &bars.full[stage]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    } else if (C::SCALED && warp == 1 && lane == 0) {
      // ---------------- MMA issuer, scales applied by the tensor core ----------------
      // A scale word in tensor memory holds four e8m0 bytes per row, and an MMA picks one of
      // them by an index in its instruction descriptor.  A 128-block scale is the same for the
      // four 32-deep MMAs of a stage, so the four bytes of a word carry FOUR K BLOCKS: the
      // three 512-byte pieces (rows of A, the two 128-column halves of the weight tile) are
      // copied from shared to tensor memory once per group of four stages, and the MMAs of
      // stage j of the group all use byte j.  One accumulation phase per tile.
      // The tensor pipe's queue is shallow and this one thread feeds it, with the 40 registers
      // the producer warpgroup keeps: descriptor low words are base + stage * constant, high
      // words constants, and the loop is not unrolled (an unrolled version spills and measured
      // half the speed).
      uint8_t* sf_smem = tiles + C::STAGES * C::STAGE_BYTES;
      const uint32_t a0 = smem_u32(tiles);
      const uint32_t sw_hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version, 128-byte swizzle
      const uint32_t sf_hi = (128u >> 4) | (1u << 14);                // SBO 128, version, no swizzle
      const uint32_t a_lo0 = ((a0 & 0x3FFFFu) >> 4) | ((16u >> 4) << 16);
      const uint32_t b_lo0 = (((a0 + C::A_BYTES) & 0x3FFFFu) >> 4) | (((C::BK * kStageRowBytes) >> 4) << 16);
      const uint32_t sf_lo0 = (smem_u32(sf_smem) & 0x3FFFFu) >> 4;
      auto desc = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };
      const uint32_t sfa_t = tmem_base + kSfaCol, sfb_t = tmem_base + kSfbCol;
      constexpr uint32_t kBStep = (C::UMMA_K * kStageRowBytes) >> 4;  // one 32-deep K slice of B
      const uint32_t idesc0 = make_idesc_mx(0u, 0u, 1u, BM, C::BN, 0, 0);
      uint32_t stage = 0, phase = 0, buf_phase = 0, group = 0;
      bool ok = true;
      for (int t = sched_id; t < num_tiles && ok; t += sched_stride) {
        ok = mbar_wait(&bars.tempty[0], buf_phase ^ 1u, abort_p);  // the accumulator has been read out
        if (!ok) break;
        uint32_t accum = 0;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          const uint32_t j = static_cast<uint32_t>(kb) & 3u;
          if (j == 0) {  // next group of scale words: shared -> tensor memory
            const uint32_t g = group & 1u;
            ok = mbar_wait(&bars.sffull[g], (group >> 1) & 1u, abort_p);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sf_lo = sf_lo0 + g * (kSfGroupBytes >> 4);
            tmem_cp_32x128b_x4(sfa_t, desc(sf_lo, sf_hi));
            tmem_cp_32x128b_x4(sfb_t, desc(sf_lo + (kSfaBytes >> 4), sf_hi));
            tmem_cp_32x128b_x4(sfb_t + 4, desc(sf_lo + ((kSfaBytes + 512) >> 4), sf_hi));
            mma_commit(&bars.sfempty[g]);  // the loader may refill once the copies are done
            ++group;
          }
          ok = mbar_wait(&bars.full[stage], phase, abort_p);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (C::STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + stage * (C::STAGE_BYTES >> 4);
          const uint32_t idesc = idesc0 | (j << 4) | (j << 29);  // scale byte j for A and for B
          mma_mxf8f6f4(tmem_base, desc(a_lo, sw_hi), desc(b_lo, sw_hi), idesc, sfa_t, sfb_t, accum);
          mma_mxf8f6f4(tmem_base, desc(a_lo + 2, sw_hi), desc(b_lo + kBStep, sw_hi), idesc, sfa_t, sfb_t, 1u);
          mma_mxf8f6f4(tmem_base, desc(a_lo + 4, sw_hi), desc(b_lo + 2 * kBStep, sw_hi), idesc, sfa_t, sfb_t, 1u);
          mma_mxf8f6f4(tmem_base, desc(a_lo + 6, sw_hi), desc(b_lo + 3 * kBStep, sw_hi), idesc, sfa_t, sfb_t, 1u);
          accum = 1;
          mma_commit(&bars.empty[stage]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) mma_commit(&bars.tfull[0]);
        buf_phase ^= 1u;
      }
    } else if (C::SCALED && warp == 2) {
      // ---------------- scale loader (KIND_F8S) ----------------
      // Per group of four K blocks: the activation scales of the tile's 128 rows (lane l owns
      // rows l, 32+l, 64+l, 96+l: exactly the 16-byte piece the tensor-memory copy wants from
      // it; four K blocks of a row are one 16-byte load) and the weight-block scales of the
      // tile's two column halves, each turned into its exponent byte, byte j of a word = K
      // block j of the group.  A scale that is not a power of two would be applied wrongly:
      // it raises the device status word instead of passing silently.
      uint8_t* sf_smem = tiles + C::STAGES * C::STAGE_BYTES;
      const int nb_count = p.N / 128;
      const int groups = (num_kb + 3) / 4;
      const bool vec = (num_kb & 3) == 0;
      uint32_t group = 0;
      bool ok = true, bad = false;
      auto e8 = [&](float v) -> uint32_t {
        const uint32_t bits = __float_as_uint(v);
        if ((bits & 0x807FFFFFu) != 0u) bad = true;   // negative or mantissa bits set
        return (bits >> 23) & 0xFFu;
      };
      auto word = [&](const float4& v) { return e8(v.x) | (e8(v.y) << 8) | (e8(v.z) << 16) | (e8(v.w) << 24); };
      for (int t = sched_id; t < num_tiles && ok; t += sched_stride) {
        const TileCoord tc = decode_tile(sched, t);
        int nb0 = problem_col<C>(tc.n_tile, 0, p.N) / 128;
        int nb1 = problem_col<C>(tc.n_tile, 128, p.N) / 128;
        nb0 = nb0 < nb_count ? nb0 : nb_count - 1;
        nb1 = nb1 < nb_count ? nb1 : nb_count - 1;
        const float* sb = p.b_scale + static_cast<int64_t>(tc.expert) * num_kb * nb_count;
        // one base pointer and four small offsets (this warp runs on 40 registers)
        const int64_t row0 = static_cast<int64_t>(tc.row_start) + lane;
        const int64_t base_row = row0 < p.R ? row0 : p.R - 1;
        const float* sa0 = p.a_scale + base_row * num_kb;
        int off[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          int64_t row = row0 + c * 32;
          if (row >= p.R) row = p.R - 1;  // rows past the end are never stored
          off[c] = static_cast<int>((row - base_row) * num_kb);
        }
        for (int grp = 0; grp < groups && ok; ++grp) {
          const int kb0 = grp * 4;
          uint4 wa;
          uint32_t* wp = reinterpret_cast<uint32_t*>(&wa);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float4 v = make_float4(1.f, 1.f, 1.f, 1.f);
            const float* src = sa0 + off[c] + kb0;
            if (vec) {
              v = *reinterpret_cast<const float4*>(src);
            } else {
              v.x = src[0];
              if (kb0 + 1 < num_kb) v.y = src[1];
              if (kb0 + 2 < num_kb) v.z = src[2];
              if (kb0 + 3 < num_kb) v.w = src[3];
            }
            wp[c] = word(v);
          }
          float4 b0 = make_float4(1.f, 1.f, 1.f, 1.f), b1 = b0;
          b0.x = sb[kb0 * nb_count + nb0];
          b1.x = sb[kb0 * nb_count + nb1];
          if (kb0 + 1 < num_kb) { b0.y = sb[(kb0 + 1) * nb_count + nb0]; b1.y = sb[(kb0 + 1) * nb_count + nb1]; }
          if (kb0 + 2 < num_kb) { b0.z = sb[(kb0 + 2) * nb_count + nb0]; b1.z = sb[(kb0 + 2) * nb_count + nb1]; }
          if (kb0 + 3 < num_kb) { b0.w = sb[(kb0 + 3) * nb_count + nb0]; b1.w = sb[(kb0 + 3) * nb_count + nb1]; }
          const uint32_t w0 = word(b0), w1 = word(b1);
          const uint32_t g = group & 1u;
          ok = mbar_wait(&bars.sfempty[g], ((group >> 1) & 1u) ^ 1u, abort_p);
          if (!ok) break;
          uint8_t* dst = sf_smem + g * kSfGroupBytes;
          *reinterpret_cast<uint4*>(dst + lane * 16) = wa;
          *reinterpret_cast<uint4*>(dst + kSfaBytes + lane * 16) = make_uint4(w0, w0, w0, w0);
          *reinterpret_cast<uint4*>(dst + kSfaBytes + 512 + lane * 16) = make_uint4(w1, w1, w1, w1);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.sffull[g]);
          ++group;
        }
      }
      if (__any_sync(0xffffffffu, bad) && lane == 0) atomicExch(&g_device_status, B200MOE_INVALID_ARG);
    } else if (warp == 1 && lane == 0 && rank == 0) {
      // ---------------- MMA issuer (the even CTA of a pair) ----------------
      const uint32_t idesc =
          make_idesc(p.ab_fmt, p.ab_fmt, 0u, C::B_MN_MAJOR ? 1u : 0u, C::TILE_M, C::BN);
      const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version, 128-byte swizzle
      const uint32_t a_lo0 = ((smem_u32(tiles) & 0x3FFFFu) >> 4) | ((16u >> 4) << 16);
      const uint32_t b_lo0 = (((smem_u32(tiles) + C::A_BYTES) & 0x3FFFFu) >> 4) |
                             (((C::B_MN_MAJOR ? C::BK * kStageRowBytes : 16) >> 4) << 16);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      const int phases_per_tile = C::PROMOTE ? num_kb : 1;
      const int kb_per_phase = C::PROMOTE ? 1 : num_kb;
      for (int t = sched_id; t < num_tiles && ok; t += sched_stride) {
        for (int ph = 0; ph < phases_per_tile && ok; ++ph) {
          // With one accumulation phase per K block the free accumulator buffer is what this
          // thread waits for; look at the operand stage first, so that wait is already behind
          // it when the buffer comes back.
          if constexpr (C::PROMOTE) {
            ok = mbar_wait(&bars.full[stage], phase, abort_p);
            if (!ok) break;
          }
          ok = mbar_wait(&bars.tempty[buf], buf_phase ^ 1u, abort_p);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * C::BN;
          for (int kb = 0; kb < kb_per_phase && ok; ++kb) {
            if constexpr (!C::PROMOTE) {
              ok = mbar_wait(&bars.full[stage], phase, abort_p);
              if (!ok) break;
              tc_fence_after();
            }
            // descriptors: constant high words, low words = base + stage * constant (+ an
            // immediate per K slice); this thread's scalar work between two MMAs is time the
            // tensor pipe idles
            const uint32_t a_lo = a_lo0 + stage * (C::STAGE_BYTES >> 4);
            const uint32_t b_lo = b_lo0 + stage * (C::STAGE_BYTES >> 4);
#pragma unroll
            for (int kk = 0; kk < C::BK / C::UMMA_K; ++kk) {
              const uint64_t a_desc = (static_cast<uint64_t>(desc_hi) << 32) | (a_lo + kk * 2);
              const uint64_t b_desc = (static_cast<uint64_t>(desc_hi) << 32) |
                                      (b_lo + kk * (C::B_MN_MAJOR ? ((C::UMMA_K * kStageRowBytes) >> 4) : 2));
              const uint32_t accum = (kb > 0 || kk > 0) ? 1u : 0u;
              if constexpr (C::PAIR) {
                if (C::KIND == KIND_F16) mma_f16_pair(d_tmem, a_desc, b_desc, idesc, accum);
                else mma_f8_pair(d_tmem, a_desc, b_desc, idesc, accum);
              } else {
                if (C::KIND == KIND_F16) mma_f16(d_tmem, a_desc, b_desc, idesc, accum);
                else mma_f8(d_tmem, a_desc, b_desc, idesc, accum);
              }
            }
            if constexpr (C::PAIR) mma_commit_pair(&bars.empty[stage]);
            else mma_commit(&bars.empty[stage]);
            if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok) {
            if constexpr (C::PAIR) mma_commit_pair(&bars.tfull[buf]);
            else mma_commit(&bars.tfull[buf]);
          }
          if (++buf == C::ACC_BUFS) { buf = 0; buf_phase ^= 1u; }
        }
      }
    } else if (C::OFFLOAD && warp >= 2) {
      // ---------------- store warps (OFFLOAD): staged tile -> global memory ----------------
      const uint8_t* out_stage = tiles + C::STAGES * C::STAGE_BYTES + C::SF_BYTES;
      uint32_t out_phase = 0;
      bool ok = true;
      for (int t = sched_id; t < num_tiles && ok; t += sched_stride, out_phase ^= 1u) {
        const TileCoord tc = decode_tile(sched, t);
        ok = mbar_wait_relaxed(&bars.ofull, out_phase, abort_p);
        if (!ok) break;
        write_staged_rows<C>(p, tc, rank, out_stage, (warp - 2) * (BM / 2), (warp - 1) * (BM / 2), lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.oempty);
      }
    }
  } else {
    // ---------------- accumulator readers / epilogue ----------------
    if constexpr (C::REBALANCE_REGS) asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int ew = warp - 4;
    const int quad = warp & 3;   // TMEM lane quadrant this warp may read
    const int g = ew >> 2;       // column group
    const int row_in_tile = quad * 32 + lane;
    constexpr int CPT = C::CPT;
    constexpr int NCH = C::NCH;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int nb_count = p.N / 128;
    const int phases_per_tile = C::PROMOTE ? num_kb : 1;
    int buf = 0;
    uint32_t buf_phase = 0;
    bool ok = true;
    int tile_parity = 0;
    for (int t = sched_id; t < num_tiles && ok; t += sched_stride, tile_parity ^= 1) {
      const TileCoord tc = decode_tile(sched, t);
      const bool row_ok = rank * BM + row_in_tile < tc.rows_valid;
      const int64_t grow = static_cast<int64_t>(tc.row_start) + rank * BM + row_in_tile;
      float acc[CPT];
      float ta[32], tb[32];
      // Scales.  The tile touches at most two 128-column weight-scale blocks; their K/128
      // values are staged in shared memory once per tile (one round trip to L2/DRAM instead
      // of one on the critical path of every K block).  The row's activation scales are
      // contiguous in K and are fetched four K blocks at a time, four ahead of use.
      int sel0 = 0, sel1 = 0;
      const float* sa_ptr = nullptr;
      float4 sa_cur = make_float4(0.f, 0.f, 0.f, 0.f), sa_next = sa_cur;
      const bool sa_vec = (num_kb & 3) == 0;
      const float* sbs = sb_smem[tile_parity];
      auto load_sa4 = [&](int ph0) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!row_ok || ph0 >= num_kb) return v;
        if (sa_vec) return *reinterpret_cast<const float4*>(sa_ptr + ph0);
        v.x = sa_ptr[ph0];
        if (ph0 + 1 < num_kb) v.y = sa_ptr[ph0 + 1];
        if (ph0 + 2 < num_kb) v.z = sa_ptr[ph0 + 2];
        if (ph0 + 3 < num_kb) v.w = sa_ptr[ph0 + 3];
        return v;
      };
      if constexpr (C::PROMOTE) {
#pragma unroll
        for (int j = 0; j < CPT; ++j) acc[j] = 0.f;
        int nb_lo = problem_col<C>(tc.n_tile, 0, p.N) / 128;
        int nb_hi = problem_col<C>(tc.n_tile, C::BN - 1, p.N) / 128;
        nb_lo = nb_lo < nb_count ? nb_lo : nb_count - 1;
        nb_hi = nb_hi < nb_count ? nb_hi : nb_count - 1;
        int nb0 = problem_col<C>(tc.n_tile, chunk_tmem_col<C>(g, 0), p.N) / 128;
        int nb1 = problem_col<C>(tc.n_tile, chunk_tmem_col<C>(g, NCH / 2), p.N) / 128;
        sel0 = nb0 >= nb_hi ? 1 : 0;   // both halves fall in one of the two blocks
        sel1 = nb1 >= nb_hi ? 1 : 0;
        const float* sb_ptr = p.b_scale + static_cast<int64_t>(tc.expert) * num_kb * nb_count;
        float* dst = sb_smem[tile_parity];
        for (int i = threadIdx.x - 128; i < 2 * num_kb; i += C::EPI_WARPS * 32)
          dst[i] = sb_ptr[(i >> 1) * nb_count + ((i & 1) ? nb_hi : nb_lo)];
        sa_ptr = p.a_scale + grow * num_kb;
        sa_cur = load_sa4(0);
        sa_next = load_sa4(4);
        // hand-over of the staged buffer: one arrival per warp and a bounded wait (a warp that
        // gave up on some wait must not leave the others parked on a plain barrier)
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.sready);
        ok = mbar_wait(&bars.sready, static_cast<uint32_t>(tile_parity), abort_p);
        if (!ok) break;
      }
      ok = mbar_wait(&bars.tfull[buf], buf_phase, abort_p);
      if (!ok) break;
      tc_fence_after();
      if constexpr (!C::PROMOTE) {
        // One accumulation phase per tile: the finished accumulator goes straight into the
        // registers the epilogue works on, every chunk in flight at once, and the buffer is
        // handed back after a single round trip.
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tmem_ld_32x32(tmem_base + lane_addr + buf * C::BN + chunk_tmem_col<C>(g, c),
                        *reinterpret_cast<float(*)[32]>(acc + c * 32));
#pragma unroll
        for (int c = 0; c < NCH; ++c) tmem_ld_wait_on(*reinterpret_cast<float(*)[32]>(acc + c * 32));
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (C::PAIR) mbar_arrive_cluster(&bars.tempty[buf], 0);
          else mbar_arrive(&bars.tempty[buf]);
        }
        if (++buf == C::ACC_BUFS) { buf = 0; buf_phase ^= 1u; }
        tile_epilogue<C>(p, tc, g, row_ok, grow, acc, xchg[tile_parity], epi_buf[ew]);
        continue;
      }
      // first two loads of the tile
      tmem_ld_32x32(tmem_base + lane_addr + buf * C::BN + chunk_tmem_col<C>(g, 0), ta);
      tmem_ld_32x32(tmem_base + lane_addr + buf * C::BN + chunk_tmem_col<C>(g, 1), tb);

      // Two 32-column loads are kept in flight: both are waited for together, then
      // each buffer is consumed and immediately refilled with the chunk after next.
      for (int ph = 0; ph < phases_per_tile && ok; ++ph) {
        float s0 = 1.f, s1 = 1.f;
        if constexpr (C::PROMOTE) {
          const int w = ph & 3;
          if (w == 0 && ph > 0) {
            sa_cur = sa_next;
            sa_next = load_sa4(ph + 4);
          }
          const float sa = w == 0 ? sa_cur.x : (w == 1 ? sa_cur.y : (w == 2 ? sa_cur.z : sa_cur.w));
          s0 = sa * sbs[2 * ph + sel0];
          s1 = sa * sbs[2 * ph + sel1];
        }
#pragma unroll
        for (int q = 0; q < NCH / 2; ++q) {
          tmem_ld_wait();
          const bool last_pair = q + 1 == NCH / 2;
          const int c0 = 2 * q, c1 = 2 * q + 1;
          const float sc0 = c0 < NCH / 2 ? s0 : s1;
          const float sc1 = c1 < NCH / 2 ? s0 : s1;
          if (!last_pair) {
            // consume a staged chunk, refill it with the chunk after next of the same buffer
            accumulate32<C::PROMOTE>(acc + c0 * 32, ta, sc0);
            tmem_ld_32x32(tmem_base + lane_addr + buf * C::BN + chunk_tmem_col<C>(g, c0 + 2), ta);
            accumulate32<C::PROMOTE>(acc + c1 * 32, tb, sc1);
            tmem_ld_32x32(tmem_base + lane_addr + buf * C::BN + chunk_tmem_col<C>(g, c1 + 2), tb);
          } else {
            // every column of this buffer is in registers: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (C::PAIR) mbar_arrive_cluster(&bars.tempty[buf], 0);
              else mbar_arrive(&bars.tempty[buf]);
            }
            // The last two chunks are accumulated while the next partial is still being
            // computed, so that the moment it is ready both staging buffers are free and its
            // first two loads go out at once: from "accumulator complete" to "accumulator
            // free again" is on the critical path of every K block (two buffers in flight).
            accumulate32<C::PROMOTE>(acc + c0 * 32, ta, sc0);
            accumulate32<C::PROMOTE>(acc + c1 * 32, tb, sc1);
            if (++buf == C::ACC_BUFS) { buf = 0; buf_phase ^= 1u; }
            if (ph + 1 < phases_per_tile) {
              ok = mbar_wait(&bars.tfull[buf], buf_phase, abort_p);
              if (ok) {
                tc_fence_after();
                tmem_ld_32x32(tmem_base + lane_addr + buf * C::BN + chunk_tmem_col<C>(g, 0), ta);
                tmem_ld_32x32(tmem_base + lane_addr + buf * C::BN + chunk_tmem_col<C>(g, 1), tb);
              }
            }
          }
        }
      }
      if (!ok) break;
      if constexpr (C::OFFLOAD) {
        // the tile leaves through shared memory; the store warps write it out while this
        // warp is back at the accumulators of the next tile
        add_bias<C>(p, tc, g, acc);
        ok = mbar_wait(&bars.oempty, static_cast<uint32_t>(tile_parity) ^ 1u, abort_p);
        if (!ok) break;
        if (row_ok) stage_row<C>(tiles + C::STAGES * C::STAGE_BYTES + C::SF_BYTES, row_in_tile, g, p.d_dtype, acc);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.ofull);
      } else {
        tile_epilogue<C>(p, tc, g, row_ok, grow, acc, xchg[tile_parity], epi_buf[ew]);
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    if (threadIdx.x == 0) atomicExch(&g_device_status, B200MOE_TIMEOUT);
    // Let copies that are still in flight land before shared memory is released.
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
    __syncthreads();
  }
  if constexpr (C::PAIR) cluster_sync();  // neither CTA leaves while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (C::PAIR) tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    else tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---- host side ---------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

CUtensorMapDataType tm_dtype(int dtype) {
  switch (dtype) {
    case B200MOE_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case B200MOE_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

// Row-major [rows, cols] (2-D) or [batch, rows, cols] (3-D) tensor, box of
// `box_cols` x `box_rows` elements, 128-byte swizzle, zero fill out of bounds.
int make_map(CUtensorMap* map, int dtype, const void* base, uint64_t cols, uint64_t rows,
             uint64_t batch, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return B200MOE_CUDA_ERROR;
  const uint64_t elt = dtype_size(dtype);
  cuuint64_t dims[3] = {cols, rows, batch ? batch : 1};
  cuuint64_t strides[2] = {cols * elt, cols * rows * elt};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const cuuint32_t rank = batch ? 3 : 2;
  CUresult r = fn(map, tm_dtype(dtype), rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled", cudaErrorInvalidValue);
    return B200MOE_CUDA_ERROR;
  }
  return B200MOE_OK;
}

template <typename C>
int launch_config(const b200moe_gemm_args& a, const void* B, int b_dtype, cudaStream_t st) {
  CUtensorMap map_a, map_b;
  int rc = make_map(&map_a, a.a_dtype, a.A, a.K, a.R, 0, C::BK, BM);
  if (rc != B200MOE_OK) return rc;
  if (C::B_MN_MAJOR)
    rc = make_map(&map_b, b_dtype, B, a.N, a.K, a.E, C::CHUNK_COLS, C::BK);
  else
    rc = make_map(&map_b, b_dtype, B, a.K, a.N, a.E, C::BK,
                  (C::GATED_SPLIT || C::PAIR) ? C::BN / 2 : C::BN);
  if (rc != B200MOE_OK) return rc;

  GemmParams p;
  p.a_scale = a.a_scale;
  p.b_scale = reinterpret_cast<const float*>(a.b_scale);
  p.bias = a.bias;
  p.bias_dtype = a.bias_dtype;
  p.D = a.D;
  p.d_scale = a.d_scale;
  p.d_dtype = a.d_dtype;
  p.rows_per_expert = a.rows_per_expert;
  p.R = a.R;
  p.N = a.N;
  p.K = a.K;
  p.E = a.E;
  p.ldd = a.epilogue == B200MOE_EPI_STORE ? a.N : a.N / 2;  // elements (bytes for e4m3)
  p.alpha = a.alpha;
  p.limit = a.limit;
  p.act = a.gated_act;
  p.act_p0 = a.act_param0;
  p.act_p1 = a.act_param1;
  p.clamp = a.clamp_limit;
  p.pow2_scales = a.scales_pow2;
  p.d_row_ptr = a.epilogue == B200MOE_EPI_STORE ? a.d_row_ptr : nullptr;
  p.ab_fmt = a.a_dtype == B200MOE_BF16 ? 1 : 0;  // kind::f16: 0 f16, 1 bf16; kind::f8f6f4: 0 e4m3

  rc = ensure_dynamic_smem<C>(grouped_gemm_kernel<C>, C::SMEM_BYTES, "cudaFuncSetAttribute");
  if (rc != B200MOE_OK) return rc;
  const int n_tiles = C::GATED_SPLIT ? (a.N / 2 + C::BN / 2 - 1) / (C::BN / 2)
                                     : (a.N + C::BN - 1) / C::BN;
  const int64_t max_m_tiles = (a.R + C::TILE_M - 1) / C::TILE_M + a.E;
  int64_t grid = max_m_tiles * n_tiles * (C::PAIR ? 2 : 1);
  if (grid > kNumSMs) grid = kNumSMs;
  // B200MOE_GEMM_SMS caps the persistent grid (read per call): a caller that runs the exchange
  // kernels of one wave of tokens beside the GEMMs of another leaves them a few SMs this way
  if (const char* cap = getenv("B200MOE_GEMM_SMS")) {
    const int c = atoi(cap);
    if (c >= 2 && c < grid) grid = c;
  }
  if (grid < 1) grid = 1;
  if (C::PAIR) {
    grid = grid < 2 ? 2 : grid & ~1ll;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<C>, map_a, map_b, p);
    if (e != cudaSuccess) {
      set_last_error("grouped_gemm_kernel (cluster launch)", e);
      return B200MOE_CUDA_ERROR;
    }
    return launch_status("grouped_gemm_kernel");
  }
  grouped_gemm_kernel<C><<<static_cast<int>(grid), C::THREADS, C::SMEM_BYTES, st>>>(map_a, map_b, p);
  return launch_status("grouped_gemm_kernel");
}

// ---- CUDA-core evaluation of the same contract (checking aid) --------------------------

__global__ void gemm_check_kernel(b200moe_gemm_args a, int b_layout_nk) {
  // one thread per (row, col); expert of the row by linear scan
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (idx >= a.R * a.N) return;
  const int64_t row = idx / a.N;
  const int col = static_cast<int>(idx % a.N);
  int e = -1;
  int64_t off = 0;
  for (int i = 0; i < a.E; ++i) {
    const int64_t n = a.rows_per_expert[i];
    if (row < off + n) { e = i; break; }
    off += n;
  }
  if (e < 0) return;
  float acc = 0.f;
  const int nkb = a.K / 128;
  for (int k = 0; k < a.K; ++k) {
    float av;
    if (a.a_dtype == B200MOE_E4M3) {
      av = e4m3_to_f32(reinterpret_cast<const uint8_t*>(a.A)[row * a.K + k]);
      if (a.a_scale) av *= a.a_scale[row * nkb + k / 128];
    } else if (a.a_dtype == B200MOE_BF16) {
      av = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.A)[row * a.K + k]);
    } else {
      av = __half2float(reinterpret_cast<const __half*>(a.A)[row * a.K + k]);
    }
    float bv;
    if (a.recipe == B200MOE_RECIPE_BF16) {
      const int64_t at = b_layout_nk ? (static_cast<int64_t>(e) * a.N + col) * a.K + k
                                     : (static_cast<int64_t>(e) * a.K + k) * a.N + col;
      bv = a.a_dtype == B200MOE_F16 ? __half2float(reinterpret_cast<const __half*>(a.B)[at])
                                    : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.B)[at]);
    } else if (a.recipe == B200MOE_RECIPE_FP8_BLOCK) {
      bv = e4m3_to_f32(reinterpret_cast<const uint8_t*>(a.B)[(static_cast<int64_t>(e) * a.K + k) * a.N + col]);
      bv *= reinterpret_cast<const float*>(a.b_scale)[(static_cast<int64_t>(e) * nkb + k / 128) * (a.N / 128) + col / 128];
    } else {
      const uint8_t byte = reinterpret_cast<const uint8_t*>(a.B)[(static_cast<int64_t>(e) * a.N + col) * (a.K / 2) + k / 2];
      const int code = (k & 1) ? (byte >> 4) : (byte & 0xF);
      const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
      bv = (code & 8) ? -mag[code & 7] : mag[code & 7];
      const uint8_t sc = reinterpret_cast<const uint8_t*>(a.b_scale)[(static_cast<int64_t>(e) * a.N + col) * (a.K / 32) + k / 32];
      bv *= exp2f(static_cast<float>(sc) - 127.f);
    }
    acc = fmaf(av, bv, acc);
  }
  if (a.bias) acc += load_bias(a.bias, a.bias_dtype, static_cast<int64_t>(e) * a.N + col);
  if (a.d_dtype == B200MOE_F32) reinterpret_cast<float*>(a.D)[idx] = acc;
  else if (a.d_dtype == B200MOE_BF16) reinterpret_cast<__nv_bfloat16*>(a.D)[idx] = __float2bfloat16_rn(acc);
  else reinterpret_cast<__half*>(a.D)[idx] = __float2half_rn(acc);
}

// ---- weight dequantisation to 16-bit (compatibility paths) ------------------------------

__global__ void dequant_fp8_block_kernel(const uint8_t* __restrict__ w, const float* __restrict__ s,
                                         __nv_bfloat16* __restrict__ out, int64_t E, int K, int N) {
  const int64_t total = E * K * static_cast<int64_t>(N) / 8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t at = i * 8;
    const int col = static_cast<int>(at % N);
    const int64_t ek = at / N;
    const int k = static_cast<int>(ek % K);
    const int64_t e = ek / K;
    const float sc = s[(e * (K / 128) + k / 128) * (N / 128) + col / 128];
    const uint2 raw = *reinterpret_cast<const uint2*>(w + at);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
    Vec<__nv_bfloat16, 8> o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16_rn(e4m3_to_f32(b[j]) * sc);
    *reinterpret_cast<Vec<__nv_bfloat16, 8>*>(out + at) = o;
  }
}

// [E,N,K/2] e2m1 pairs + [E,N,K/32] e8m0 -> [E,N,K] bf16 (exact: every product
// of an e2m1 value and a power of two is a bf16 number).
__global__ void dequant_mxfp4_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ s,
                                     __nv_bfloat16* __restrict__ out, int64_t rows, int K) {
  const int64_t total = rows * (K / 8);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / (K / 8);
    const int k0 = static_cast<int>(i % (K / 8)) * 8;
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(w + row * (K / 2) + k0 / 2);
    const float sc = exp2f(static_cast<float>(s[row * (K / 32) + k0 / 32]) - 127.f);
    Vec<__nv_bfloat16, 8> o;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int code = (raw >> (4 * j)) & 0xF;
      const int m = code & 7;
      float mag = m < 4 ? 0.5f * m : (m == 4 ? 2.f : (m == 5 ? 3.f : (m == 6 ? 4.f : 6.f)));
      o.v[j] = __float2bfloat16_rn((code & 8) ? -mag * sc : mag * sc);
    }
    *reinterpret_cast<Vec<__nv_bfloat16, 8>*>(out + row * K + k0) = o;
  }
}

#include "grouped_gemm_decode.cuh"
#include "grouped_gemm_mx.cuh"

}  // namespace
}  // namespace b200moe

using namespace b200moe;

static int validate(const b200moe_gemm_args* a) {
  if (!a) return B200MOE_INVALID_ARG;
  if (a->R < 0 || a->N <= 0 || a->K <= 0 || a->E <= 0 || a->E > kMaxExpertsSmem) return B200MOE_INVALID_ARG;
  if (a->N % 8 != 0) return B200MOE_INVALID_ARG;
  if (a->R == 0) return B200MOE_OK;
  if (!a->A || !a->B || (!a->D && !a->d_row_ptr) || !a->rows_per_expert) return B200MOE_INVALID_ARG;
  if (a->R >= (1ll << 31)) return B200MOE_UNSUPPORTED;
  return B200MOE_OK;
}

extern "C" size_t b200moe_grouped_gemm_workspace_bytes(const b200moe_gemm_args* a) {
  if (!a) return 0;
  const size_t full = static_cast<size_t>(a->E) * a->N * a->K * 2;
  if (a->recipe == B200MOE_RECIPE_MXFP4) return full;
  if (a->recipe == B200MOE_RECIPE_FP8_BLOCK && a->a_dtype != B200MOE_E4M3) return full;
  return 0;
}

extern "C" int b200moe_dequant_weights(int recipe, const void* B, const void* b_scale, void* out,
                                       int E, int N, int K, void* stream) {
  if (!B || !b_scale || !out || E <= 0 || N <= 0 || K <= 0) return B200MOE_INVALID_ARG;
  cudaStream_t st = as_stream(stream);
  const int grid = kNumSMs * 8;
  if (recipe == B200MOE_RECIPE_FP8_BLOCK) {
    if (K % 128 || N % 128) return B200MOE_INVALID_ARG;
    dequant_fp8_block_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint8_t*>(B),
                                                   reinterpret_cast<const float*>(b_scale),
                                                   reinterpret_cast<__nv_bfloat16*>(out), E, K, N);
  } else if (recipe == B200MOE_RECIPE_MXFP4) {
    if (K % 32) return B200MOE_INVALID_ARG;
    dequant_mxfp4_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint8_t*>(B),
                                               reinterpret_cast<const uint8_t*>(b_scale),
                                               reinterpret_cast<__nv_bfloat16*>(out),
                                               static_cast<int64_t>(E) * N, K);
  } else {
    return B200MOE_UNSUPPORTED;
  }
  return launch_status("dequant_weights");
}

// the split gated epilogue with something other than plain SiLU
static bool gated_any(const b200moe_gemm_args& a) {
  return a.epilogue == B200MOE_EPI_SILU_MUL && (a.gated_act != B200MOE_ACT_SILU || a.clamp_limit > 0.0f);
}

template <int KIND, bool MN, bool PROMOTE, int BN, int STAGES, bool PAIR = false>
static int launch_epi(const b200moe_gemm_args& a, const void* B, int b_dtype, cudaStream_t st) {
  switch (a.epilogue) {
    case B200MOE_EPI_STORE:
      if constexpr (KIND == KIND_F8 && PROMOTE && PAIR && BN == 256) {
        // The tile leaves through a staging tile in shared memory and the spare warps; four
        // operand stages instead of six make room for it.  Measured on tiles of 16 K blocks
        // (K = 2048): +5 % with 32 experts of 1024 or 4096 rows, +2-4 % on 256 ragged experts
        // of ~512 rows; on tiles of 112 K blocks, where the store is 2 % of a tile, -5 %.
        // So: short tiles only.  B200MOE_STORE_OFFLOAD=0 / 1 forces the choice (tests).
        // Rows with a home of their own (d_row_ptr) keep the reader-warp store.
        const char* off = getenv("B200MOE_STORE_OFFLOAD");
        const bool on = off ? off[0] != '0' : a.K <= 4096;
        if (on && !a.d_row_ptr)
          return launch_config<Config<KIND, MN, PROMOTE, BN, B200MOE_EPI_STORE, 4, PAIR, true>>(a, B, b_dtype, st);
      }
      return launch_config<Config<KIND, MN, PROMOTE, BN, B200MOE_EPI_STORE, STAGES, PAIR>>(a, B, b_dtype, st);
    case B200MOE_EPI_SILU_MUL:
      // an MN-major split tile needs one weight box for the gate half and one for the up half
      if constexpr (MN && !PAIR && BN * (KIND == KIND_F16 ? 2 : 1) < 256) {
        return B200MOE_UNSUPPORTED;
      } else if (gated_any(a)) {
        if constexpr (PAIR) return B200MOE_UNSUPPORTED;  // the caller does not pair these
        else return launch_config<Config<KIND, MN, PROMOTE, BN, kEpiGatedAny, STAGES, false>>(a, B, b_dtype, st);
      } else {
        return launch_config<Config<KIND, MN, PROMOTE, BN, B200MOE_EPI_SILU_MUL, STAGES, PAIR>>(a, B, b_dtype, st);
      }
    case B200MOE_EPI_SWIGLU_OAI:
      return launch_config<Config<KIND, MN, PROMOTE, BN, B200MOE_EPI_SWIGLU_OAI, STAGES, PAIR>>(a, B, b_dtype, st);
    default:
      return B200MOE_INVALID_ARG;
  }
}

// 128x256 tiles halve the shared-memory and L2 traffic per flop; 128x128 tiles
// give more CTAs something to do when the problem is small.
static bool want_pair(const b200moe_gemm_args& a, bool wide) {
  const char* force = getenv("B200MOE_PAIR");  // test hook: forces a tile shape for one call
  if (force) return atoi(force) != 0 && wide;
  // CTA pairs schedule 256-row tiles and halve the weight bytes each CTA stages per flop (a
  // single CTA's 128x256 tile asks shared memory for more than it can deliver at the full MMA
  // rate); worth it once the experts are tall enough that the 256-row tiles are not mostly
  // padding.  Measured: +3 % for 16-bit operands on the Mixtral shapes; for the block-scaled
  // FP8 recipe, whose per-K-block accumulator hand-off gets slower across two CTAs, +6-7 %
  // with the store epilogue from 512 rows per expert on (second GEMM of the DeepSeek-V3 and
  // Mixtral shapes), +2 % with the fused activation epilogue at 1024 rows per expert and
  // -6 % at 512.
  const bool promote = a.recipe == B200MOE_RECIPE_FP8_BLOCK && a.a_dtype == B200MOE_E4M3;
  const int64_t rows = a.R / a.E;
  if (promote) return wide && rows >= (a.epilogue == B200MOE_EPI_STORE ? 512 : 1024);
  return wide && rows >= 1024;
}

static bool want_wide_tile(const b200moe_gemm_args& a) {
  const char* force = getenv("B200MOE_TILE_N");  // test hook, as above
  if (force) return atoi(force) == 256;
  const int64_t n_eff = a.epilogue == B200MOE_EPI_SILU_MUL ? a.N / 2 : a.N;
  const int64_t m_tiles = (a.R + BM - 1) / BM;
  return n_eff % 128 == 0 && n_eff >= 256 && m_tiles * (n_eff / 128) >= 2 * kNumSMs;
}

extern "C" int b200moe_grouped_gemm(const b200moe_gemm_args* args, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  int rc = validate(args);
  if (rc != B200MOE_OK || args->R == 0) return rc;
  b200moe_gemm_args a = *args;
  cudaStream_t st = as_stream(stream);
  if (a.epilogue != B200MOE_EPI_STORE && (a.N % 2 != 0)) return B200MOE_INVALID_ARG;
  const bool quant_out = a.d_dtype == B200MOE_E4M3;
  if (!quant_out && a.d_dtype != B200MOE_BF16 && a.d_dtype != B200MOE_F16) return B200MOE_UNSUPPORTED;
  if (quant_out && (a.epilogue != B200MOE_EPI_SILU_MUL || !a.d_scale || (a.N / 2) % 128 != 0))
    return B200MOE_UNSUPPORTED;
  const bool wide = want_wide_tile(a);
  const bool pair = want_pair(a, wide) && !gated_any(a);

  if (a.gated_act < B200MOE_ACT_SILU || a.gated_act > B200MOE_ACT_SITU) return B200MOE_INVALID_ARG;
  if (a.a_scale_layout == B200MOE_A_SCALE_KBLOCK_MAJOR || a.a_scale_layout == B200MOE_A_SCALE_ROW_MAJOR_DECODE) {
    if (gated_any(a) || a.clamp_limit > 0.0f) return B200MOE_UNSUPPORTED;  // SiLU only on that kernel
    return grouped_gemm_decode(a, st);
  }
  if (a.recipe == B200MOE_RECIPE_FP8_BLOCK && a.a_dtype == B200MOE_E4M3 && !a.a_scale && !a.b_scale) {
    // Unit scales: a plain e4m3 x e4m3 contraction with one accumulation phase per tile.
    // No recipe of the layer uses it; it is the same-dtype ceiling the block-scaled
    // kernel is measured against.
    if (a.K % 128 || a.N % 128 || quant_out || a.epilogue != B200MOE_EPI_STORE) return B200MOE_UNSUPPORTED;
    if (pair) return launch_config<Config<KIND_F8, true, false, 256, B200MOE_EPI_STORE, 6, true>>(a, a.B, B200MOE_E4M3, st);
    return launch_config<Config<KIND_F8, true, false, 256, B200MOE_EPI_STORE, 4>>(a, a.B, B200MOE_E4M3, st);
  }
  if (a.recipe == B200MOE_RECIPE_FP8_BLOCK && a.a_dtype == B200MOE_E4M3) {
    if (!a.a_scale || !a.b_scale || a.K % 128 || a.N % 128) return B200MOE_INVALID_ARG;
    if (a.K / 128 > kMaxKBlocks) return B200MOE_UNSUPPORTED;
    if (a.epilogue == B200MOE_EPI_SILU_MUL && (a.N / 2) % 128 != 0) return B200MOE_UNSUPPORTED;
    if (a.scales_pow2) {
      // power-of-two scales: the tensor core applies them, one accumulation phase per tile
      if (a.epilogue == B200MOE_EPI_SWIGLU_OAI) return B200MOE_UNSUPPORTED;
      if (a.epilogue == B200MOE_EPI_STORE)
        return launch_config<Config<KIND_F8S, true, false, 256, B200MOE_EPI_STORE, 4>>(a, a.B, B200MOE_E4M3, st);
      if (gated_any(a))
        return launch_config<Config<KIND_F8S, true, false, 256, kEpiGatedAny, 4>>(a, a.B, B200MOE_E4M3, st);
      return launch_config<Config<KIND_F8S, true, false, 256, B200MOE_EPI_SILU_MUL, 4>>(a, a.B, B200MOE_E4M3, st);
    }
    if (pair) return launch_epi<KIND_F8, true, true, 256, 6, true>(a, a.B, B200MOE_E4M3, st);
    if (wide || a.epilogue == B200MOE_EPI_SILU_MUL)
      return launch_epi<KIND_F8, true, true, 256, 4>(a, a.B, B200MOE_E4M3, st);
    return launch_epi<KIND_F8, true, true, 128, 6>(a, a.B, B200MOE_E4M3, st);
  }
  if (quant_out) return B200MOE_UNSUPPORTED;

  // 16-bit activations: weights must be 16-bit too; quantised weights are
  // expanded into the workspace first (slow path kept for API compatibility).
  if (a.a_dtype != B200MOE_BF16 && a.a_dtype != B200MOE_F16) return B200MOE_UNSUPPORTED;
  const void* B = a.B;
  bool b_nk = a.recipe == B200MOE_RECIPE_BF16 && a.b_layout == B200MOE_B_LAYOUT_NK;
  if (a.recipe != B200MOE_RECIPE_BF16) {
    if (a.a_dtype != B200MOE_BF16) return B200MOE_UNSUPPORTED;
    const size_t need = b200moe_grouped_gemm_workspace_bytes(&a);
    if (!workspace || workspace_bytes < need) return B200MOE_WORKSPACE_TOO_SMALL;
    rc = b200moe_dequant_weights(a.recipe, a.B, a.b_scale, workspace, a.E, a.N, a.K, stream);
    if (rc != B200MOE_OK) return rc;
    B = workspace;
    b_nk = a.recipe == B200MOE_RECIPE_MXFP4;
  }
  if (a.K % 8 != 0) return B200MOE_INVALID_ARG;
  if (b_nk) {
    if (pair) return launch_epi<KIND_F16, false, false, 256, 6, true>(a, B, a.a_dtype, st);
    if (wide) return launch_epi<KIND_F16, false, false, 256, 4>(a, B, a.a_dtype, st);
    return launch_epi<KIND_F16, false, false, 128, 6>(a, B, a.a_dtype, st);
  }
  if (pair) return launch_epi<KIND_F16, true, false, 256, 6, true>(a, B, a.a_dtype, st);
  if (wide) return launch_epi<KIND_F16, true, false, 256, 4>(a, B, a.a_dtype, st);
  return launch_epi<KIND_F16, true, false, 128, 6>(a, B, a.a_dtype, st);
}

extern "C" size_t b200moe_mx_weight_scales_bytes(int E, int N, int K) {
  if (E <= 0 || N <= 0 || K <= 0) return 0;
  const size_t num_kb = (static_cast<size_t>(K) + kMxBK - 1) / kMxBK;
  const size_t atoms = (static_cast<size_t>(N) + 127) / 128 + 1;
  return static_cast<size_t>(E) * num_kb * atoms * kMxAtomBytes;
}

extern "C" int b200moe_mx_prepare_weight_scales(const uint8_t* scales, int E, int N, int K,
                                                uint8_t* out, void* stream) {
  if (!scales || !out || E <= 0 || N <= 0 || K < kMxBK || K % 32) return B200MOE_INVALID_ARG;
  const int64_t words = static_cast<int64_t>(b200moe_mx_weight_scales_bytes(E, N, K) / 4);
  int64_t blocks = (words + 255) / 256;
  if (blocks > kNumSMs * 16) blocks = kNumSMs * 16;
  mx_prepare_weight_scales_kernel<<<static_cast<int>(blocks), 256, 0, as_stream(stream)>>>(
      scales, out, E, N, K, words);
  return launch_status("mx_prepare_weight_scales_kernel");
}

extern "C" int b200moe_grouped_gemm_mx(const b200moe_mx_gemm_args* a, void* stream) {
  if (!a) return B200MOE_INVALID_ARG;
  if (a->R < 0 || a->N <= 0 || a->K < kMxBK || a->E <= 0 || a->E > kMaxExpertsSmem)
    return B200MOE_INVALID_ARG;
  if (a->K % 64 || a->N % 8) return B200MOE_UNSUPPORTED;  // packed 4-bit rows: 32-byte pitch
  if (a->R == 0) return B200MOE_OK;
  if (a->R >= (1ll << 31)) return B200MOE_UNSUPPORTED;
  if (!a->A || !a->a_sf || !a->B || !a->b_sf || !a->D || !a->rows_per_expert) return B200MOE_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(a->B) % 32 || reinterpret_cast<uintptr_t>(a->A) % 16 ||
      reinterpret_cast<uintptr_t>(a->a_sf) % 16 || reinterpret_cast<uintptr_t>(a->b_sf) % 16)
    return B200MOE_INVALID_ARG;
  const int64_t groups = (a->K + 511) / 512;
  if (a->a_sf_pitch % 16 || a->a_sf_pitch < groups * 16) return B200MOE_INVALID_ARG;
  cudaStream_t st = as_stream(stream);
  if (a->epilogue == B200MOE_EPI_STORE) {
    if (a->d_dtype != B200MOE_BF16 && a->d_dtype != B200MOE_F16) return B200MOE_UNSUPPORTED;
    return launch_mx<MxConfig<192, B200MOE_EPI_STORE, 5>>(*a, st);
  }
  if (a->epilogue == B200MOE_EPI_SWIGLU_OAI) {
    if (a->N % 2) return B200MOE_INVALID_ARG;
    if (a->d_dtype == B200MOE_E4M3) {
      if (!a->d_sf || (a->N / 2) % 32 || a->d_sf_pitch < (a->N / 2) / 32) return B200MOE_INVALID_ARG;
    } else if (a->d_dtype != B200MOE_BF16 && a->d_dtype != B200MOE_F16) {
      return B200MOE_UNSUPPORTED;
    }
    return launch_mx<MxConfig<192, B200MOE_EPI_SWIGLU_OAI, 5>>(*a, st);
  }
  return B200MOE_UNSUPPORTED;
}

extern "C" int b200moe_grouped_gemm_check(const b200moe_gemm_args* args, void* stream) {
  int rc = validate(args);
  if (rc != B200MOE_OK || args->R == 0) return rc;
  const int64_t total = args->R * args->N;
  const bool b_nk = args->recipe == B200MOE_RECIPE_BF16 && args->b_layout == B200MOE_B_LAYOUT_NK;
  gemm_check_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, as_stream(stream)>>>(*args, b_nk ? 1 : 0);
  return launch_status("gemm_check_kernel");
}

// A wait that can never be satisfied, with a budget of `budget_cycles`: exercises the path
// every tensor-core kernel takes when a barrier does not complete (flag raised, status word
// written, kernel returns) without involving tensor memory or TMA.
__global__ void wait_timeout_selftest_kernel(long long budget_cycles) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    b200moe::sm100::mbar_init(&bar, 1);
    b200moe::sm100::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    bool done = false;
    while (!done && clock64() - t0 < budget_cycles) done = b200moe::sm100::mbar_try_wait(&bar, 0);
    if (!done) atomicExch(&b200moe::g_device_status, B200MOE_TIMEOUT);
  }
  __syncthreads();
}

extern "C" int b200moe_selftest_wait_timeout(long long budget_cycles, void* stream) {
  if (budget_cycles <= 0 || budget_cycles > 2000000000ll) return B200MOE_INVALID_ARG;
  wait_timeout_selftest_kernel<<<1, 32, 0, as_stream(stream)>>>(budget_cycles);
  return launch_status("wait_timeout_selftest_kernel");
}

int* b200moe::device_status_word() {
  // one address per device; looked up each time (a handful of host calls per layer)
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, b200moe::g_device_status) != cudaSuccess) return nullptr;
  return reinterpret_cast<int*>(p);
}

extern "C" int b200moe_device_status(void* stream, int* status_host) {
  if (!status_host) return B200MOE_INVALID_ARG;
  cudaStream_t st = as_stream(stream);
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(status_host, g_device_status, sizeof(int), 0,
                                            cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e == cudaSuccess && *status_host != 0)
    e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  if (e != cudaSuccess) {
    set_last_error("device_status", e);
    return B200MOE_CUDA_ERROR;
  }
  return B200MOE_OK;
}
