// Block-scaled grouped GEMM: microscaling (MX) operands on tcgen05.mma
// kind::mxf8f6f4.block_scale.  Included by grouped_gemm.cu inside its namespace.
//
//   A  [R, K]      e4m3, rows grouped by expert, with e8m0 scales per 32 of K
//                  (row-major bytes [R, a_sf_pitch]);
//   B  [E, N, K/2] e2m1 pairs (the MXFP4 weight layout of the operator), read by a
//                  tensor map of the "16 x 4 bit, 16-byte aligned" type, which
//                  expands every element to a byte container on the way into shared
//                  memory -- HBM and L2 carry 4 bits per weight, the tensor core
//                  sees the element layout kind::mxf8f6f4 wants;
//   SFB            the weight scales, rearranged once per layer by
//                  mx_prepare_weight_scales_kernel into 512-byte pieces per
//                  (expert, 128 of K, 128 rows of N) in tensor-memory order.
//
// The scales never touch the accumulators: tcgen05.cp moves them from shared memory
// into tensor memory and the MMA applies them, so a tile is one uninterrupted chain
// of MMAs into one accumulator buffer, and the reader warps only run epilogues
// (bias, SwigluOAI, MXFP8 quantisation of the result for the second GEMM).
//
// Roles (one persistent CTA per SM): warp 0 TMA producer (A, B and SFB), warp 1 MMA
// issuer, warp 2 activation-scale loader (the tile's 128 rows start at an arbitrary
// row, so their scale words are fetched with plain loads, transposed into the
// tensor-memory order in shared memory and published with a proxy fence), warps 4..
// accumulator readers.  K need not be a multiple of 128: the last stage is loaded at
// K-128 and only its new 32-wide sub-blocks are issued.

constexpr int kMxBK = 128;            // elements of K per stage (128 bytes per row for both operands)
constexpr int kMxSfaBytes = 512;      // one scale word per row of the A tile
constexpr int kMxAtomBytes = 512;     // scales of 128 rows of B for one stage
constexpr int kMxSfaCol = 448;        // tensor-memory columns of the scale words
constexpr int kMxSfbCol = 456;

struct MxParams {
  const uint8_t* a_sf;
  int64_t a_sf_pitch;
  const uint8_t* b_sf;  // prepared layout
  int b_atoms;          // 128-row pieces per (expert, K block) in b_sf
  const void* bias;
  int bias_dtype;
  void* D;
  int d_dtype;
  int64_t ldd;          // row pitch of D in elements
  uint8_t* d_sf;
  int64_t d_sf_pitch;
  const int32_t* rows_per_expert;
  int64_t R;
  int N, K, E;
  float alpha, limit;
};

template <int BN_, int EPI_, int STAGES_>
struct MxConfig {
  static constexpr int BN = BN_;
  static constexpr int EPI = EPI_;
  static constexpr int STAGES = STAGES_;
  static constexpr int A_BYTES = BM * kStageRowBytes;
  static constexpr int B_BYTES = BN * kStageRowBytes;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // the barrier counts what TMA read: the packed 4-bit source, half of what lands in shared memory
  static constexpr int STAGE_TX_BYTES = A_BYTES + B_BYTES / 2;
  static constexpr int B_ATOMS = (BN + 127) / 128;           // pieces copied per stage
  static constexpr int SFB_BYTES = B_ATOMS * kMxAtomBytes;
  static constexpr int COL_GROUPS = BN / 64;                 // reader warps per lane quadrant
  static constexpr int EPI_WARPS = 4 * COL_GROUPS;
  static constexpr int THREADS = 128 + EPI_WARPS * 32;
  static constexpr int ACC_STRIDE = 256;                     // tensor-memory columns between the two accumulators
  static constexpr int TMEM_COLS = 512;
  static constexpr size_t SMEM_BYTES =
      1024 + static_cast<size_t>(STAGES) * (STAGE_BYTES + kMxSfaBytes + SFB_BYTES);
  static_assert(BN % 64 == 0 && BN <= 192, "two accumulators and the scale words share 512 columns");
  static_assert(STAGE_BYTES % 1024 == 0, "swizzled tiles start on 1 KiB boundaries");
};

struct alignas(8) MxBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tfull[2];
  uint64_t tempty[2];
};

// e8m0 byte of the smallest power of two >= max(amax, eps) / 448, floored like
// per_token_group_fp8_quant floors its scale, and that power of two.
__device__ __forceinline__ uint32_t mx_scale_byte(float amax, float* scale) {
  float s = fmaxf(fmaxf(amax, 1e-10f) * (1.0f / 448.0f), 1.0f / (448.0f * 512.0f));
  uint32_t bits = __float_as_uint(s);
  uint32_t e = bits >> 23;
  if (bits & 0x7FFFFFu) ++e;
  *scale = __uint_as_float(e << 23);
  return e;
}

// The reader warps only run epilogues here (the scales are applied inside the MMA), one tile
// behind the tensor pipe, so a row's results leave with plain 16-byte stores from the thread
// that owns the row: no shared-memory staging, which leaves room for a fifth operand stage.
template <typename C>
__device__ __forceinline__ void mx_tile_epilogue(const MxParams& p, const TileCoord& tc, int g,
                                                 bool row_ok, int64_t grow, float (&acc)[64]) {
  const int col0 = tc.n_tile * C::BN + g * 64;  // first accumulator column of this thread
  if (col0 >= p.N) return;
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 64; ++j)
      if (col0 + j < p.N)
        acc[j] += load_bias(p.bias, p.bias_dtype, static_cast<int64_t>(tc.expert) * p.N + col0 + j);
  }
  if constexpr (C::EPI == B200MOE_EPI_STORE) {
    if (row_ok) store_row16<64>(p.D, p.d_dtype, grow * p.ldd + col0, acc, p.N - col0);
  } else {  // SWIGLU_OAI: (gate, up) pairs are adjacent columns -> 32 results
    float o[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) o[j] = swiglu_oai_f32(acc[2 * j], acc[2 * j + 1], p.alpha, p.limit);
    const int ocol0 = col0 / 2;
    const int n_valid = (p.N - col0) / 2;
    if (p.d_dtype == B200MOE_E4M3) {
      // the 32 results are one MX group of the second GEMM's A operand
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) amax = fmaxf(amax, j < n_valid ? fabsf(o[j]) : 0.f);
      float s;
      const uint32_t sbyte = mx_scale_byte(amax, &s);
      const float inv_s = 1.0f / s;  // exact: s is a power of two
      if (row_ok) {
        p.d_sf[grow * p.d_sf_pitch + (ocol0 >> 5)] = static_cast<uint8_t>(sbyte);
        uint8_t* dst = reinterpret_cast<uint8_t*>(p.D) + grow * p.ldd + ocol0;
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float v0 = fmaxf(-448.0f, fminf(o[4 * i + 0] * inv_s, 448.0f));
          const float v1 = fmaxf(-448.0f, fminf(o[4 * i + 1] * inv_s, 448.0f));
          const float v2 = fmaxf(-448.0f, fminf(o[4 * i + 2] * inv_s, 448.0f));
          const float v3 = fmaxf(-448.0f, fminf(o[4 * i + 3] * inv_s, 448.0f));
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v0, v1), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v2, v3), __NV_SATFINITE, __NV_E4M3);
          w[i] = lo | (hi << 16);
        }
        if (n_valid >= 32) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(dst + 16) = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
          const uint8_t* b = reinterpret_cast<const uint8_t*>(w);
          for (int j = 0; j < n_valid; ++j) dst[j] = b[j];
        }
      }
    } else if (row_ok) {
      store_row16<32>(p.D, p.d_dtype, grow * p.ldd + ocol0, o, n_valid);
    }
  }
}

template <typename C>
__global__ void __launch_bounds__(C::THREADS, 1)
grouped_gemm_mx_kernel(const __grid_constant__ CUtensorMap map_a,
                       const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_b_tail, MxParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Schedule sched;
  __shared__ MxBarriers bars;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  uint8_t* sfa_smem = tiles + C::STAGES * C::STAGE_BYTES;
  uint8_t* sfb_smem = sfa_smem + C::STAGES * kMxSfaBytes;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = (p.N + C::BN - 1) / C::BN;
  const int num_kb = (p.K + kMxBK - 1) / kMxBK;
  // K % 128 != 0: the last stage covers [K-128, K) and repeats `tail_skip` 32-wide
  // sub-blocks of the stage before it, which are not issued again.
  const int tail_skip = (p.K % kMxBK) ? (kMxBK - p.K % kMxBK) / 32 : 0;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&bars.full[s], 2);  // producer (with the byte count) + scale loader
      mbar_init(&bars.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars.tfull[b], 1);
      mbar_init(&bars.tempty[b], C::EPI_WARPS);
    }
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    prefetch_tensormap(&map_b_tail);
  }
  build_schedule(sched, p.rows_per_expert, p.E, p.R, n_tiles, BM);
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const int num_tiles = total_tiles(sched);
  volatile int* abort_p = &abort_flag;
  const int sched_id = blockIdx.x, sched_stride = gridDim.x;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = sched_id; t < num_tiles && ok; t += sched_stride) {
        const TileCoord tc = decode_tile(sched, t);
        const int n0 = tc.n_tile * C::BN;
        const uint8_t* sfb_tile =
            p.b_sf + (static_cast<int64_t>(tc.expert) * num_kb * p.b_atoms + n0 / 128) * kMxAtomBytes;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          ok = mbar_wait_spin(&bars.empty[stage], phase ^ 1u, abort_p);
          if (!ok) break;
          const bool tail = tail_skip && kb == num_kb - 1;
          uint8_t* a_dst = tiles + stage * C::STAGE_BYTES;
          mbar_arrive_expect_tx(&bars.full[stage], C::STAGE_TX_BYTES + C::SFB_BYTES);
          tma_load_2d(a_dst, &map_a, &bars.full[stage], tail ? p.K - kMxBK : kb * kMxBK, tc.row_start);
          if (tail) tma_load_3d(a_dst + C::A_BYTES, &map_b_tail, &bars.full[stage], 0, n0, tc.expert);
          else tma_load_3d(a_dst + C::A_BYTES, &map_b, &bars.full[stage], kb * kMxBK, n0, tc.expert);
          bulk_load(sfb_smem + stage * C::SFB_BYTES,
                    sfb_tile + static_cast<int64_t>(kb) * p.b_atoms * kMxAtomBytes, C::SFB_BYTES,
                    &bars.full[stage]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      // One thread feeds the tensor pipe, and an MMA of this shape takes about 100 cycles:
      // the scalar instructions between two tcgen05.mma decide whether the pipe stays busy.
      // So the stage index is a compile-time constant (the K loop is unrolled over the ring
      // and runs across tile boundaries), every descriptor is a register base plus an
      // immediate, and the instruction descriptors are constants.  Control flow around the
      // MMAs is kept to whole blocks of straight-line issues: a per-instruction guard inside
      // the unrolled loop (skip sub-block kk when kk < n) made the tail stage read the wrong
      // sub-blocks whenever it fell on the first or last slot of the ring.
      const uint32_t a0 = smem_u32(tiles);
      const uint32_t sw_hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version, 128-byte swizzle
      const uint32_t sf_hi = (128u >> 4) | (1u << 14);                // SBO 128, version, no swizzle
      const uint32_t a_lo0 = ((a0 & 0x3FFFFu) >> 4) | ((16u >> 4) << 16);
      const uint32_t b_lo0 = a_lo0 + (C::A_BYTES >> 4);
      const uint32_t sfa_lo0 = (smem_u32(sfa_smem) & 0x3FFFFu) >> 4;
      const uint32_t sfb_lo0 = (smem_u32(sfb_smem) & 0x3FFFFu) >> 4;
      const uint32_t sfa_t = tmem_base + kMxSfaCol;
      auto desc = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      int t = sched_id;
      int kb = 0;
      uint32_t d_tmem = 0, sfb_t = 0, accum = 0;
      bool more = t < num_tiles;
      while (more && ok) {
#pragma unroll
        for (int s = 0; s < C::STAGES; ++s) {
          if (kb == 0) {
            // next tile: its accumulator buffer must have been read out
            const int n_tile = decode_tile(sched, t).n_tile;
            // a tile that starts inside a 128-row piece of the scales (192-column tiles: every
            // odd one starts at row 64) reads its scale columns from that offset on
            sfb_t = tmem_base + kMxSfbCol + ((n_tile * C::BN) % 128) / 32;
            ok = mbar_wait(&bars.tempty[buf], buf_phase ^ 1u, abort_p);
            if (!ok) break;
            d_tmem = tmem_base + buf * C::ACC_STRIDE;
            accum = 0;
          }
          ok = mbar_wait_spin(&bars.full[s], phase, abort_p);
          if (!ok) break;
          tc_fence_after();
          tmem_cp_32x128b_x4(sfa_t, desc(sfa_lo0 + s * (kMxSfaBytes >> 4), sf_hi));
#pragma unroll
          for (int a = 0; a < C::B_ATOMS; ++a)
            tmem_cp_32x128b_x4(tmem_base + kMxSfbCol + 4 * a,
                               desc(sfb_lo0 + (s * C::SFB_BYTES + a * kMxAtomBytes) / 16, sf_hi));
          const uint32_t a_lo = a_lo0 + s * (C::STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + s * (C::STAGE_BYTES >> 4);
          if (tail_skip && kb == num_kb - 1) {
            // K % 128 == 64 (rows of packed 4-bit weights have a 32-byte pitch, so K is a multiple
            // of 64): the stage was loaded at K-128 and its first two sub-blocks were issued with
            // the stage before
            mma_mxf8f6f4(d_tmem, desc(a_lo + 4, sw_hi), desc(b_lo + 4, sw_hi),
                         make_idesc_mx(0u, 5u, 0u, BM, C::BN, 2, 2), sfa_t, sfb_t, accum);
            mma_mxf8f6f4(d_tmem, desc(a_lo + 6, sw_hi), desc(b_lo + 6, sw_hi),
                         make_idesc_mx(0u, 5u, 0u, BM, C::BN, 3, 3), sfa_t, sfb_t, 1u);
            accum = 1;
          } else {
            mma_mxf8f6f4(d_tmem, desc(a_lo, sw_hi), desc(b_lo, sw_hi),
                         make_idesc_mx(0u, 5u, 0u, BM, C::BN, 0, 0), sfa_t, sfb_t, accum);
            accum = 1;
#pragma unroll
            for (int kk = 1; kk < 4; ++kk)
              mma_mxf8f6f4(d_tmem, desc(a_lo + kk * 2, sw_hi), desc(b_lo + kk * 2, sw_hi),
                           make_idesc_mx(0u, 5u, 0u, BM, C::BN, kk, kk), sfa_t, sfb_t, 1u);
          }
          mma_commit(&bars.empty[s]);
          if (++kb == num_kb) {
            mma_commit(&bars.tfull[buf]);
            kb = 0;
            if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
            t += sched_stride;
            if (t >= num_tiles) { more = false; break; }
          }
        }
        phase ^= 1u;
      }
    }
  } else if (warp == 2) {
    // ---------------- activation-scale loader ----------------
    // Lane l owns rows l, 32+l, 64+l, 96+l of the tile.  One 16-byte load per row brings
    // the scale words of four K blocks; they are fetched one group (four stages) ahead.
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const int groups = (num_kb + 3) / 4;
    auto load_group = [&](int t, int grp, uint4 (&w)[4]) {
      const TileCoord tc = decode_tile(sched, t);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        int64_t row = static_cast<int64_t>(tc.row_start) + c * 32 + lane;
        if (row >= p.R) row = p.R - 1;  // rows past the end are never stored
        w[c] = *reinterpret_cast<const uint4*>(p.a_sf + row * p.a_sf_pitch + grp * 16);
      }
    };
    auto word = [](const uint4& v, int j) { return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w)); };
    uint4 cur[4], nxt[4];
    uint32_t prev_last[4] = {0u, 0u, 0u, 0u};
    int t = sched_id;
    if (t < num_tiles) load_group(t, 0, nxt);
    for (; t < num_tiles && ok; t += sched_stride) {
      for (int grp = 0; grp < groups && ok; ++grp) {
#pragma unroll
        for (int c = 0; c < 4; ++c) cur[c] = nxt[c];
        if (grp + 1 < groups) load_group(t, grp + 1, nxt);
        else if (t + sched_stride < num_tiles) load_group(t + sched_stride, 0, nxt);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kb = grp * 4 + j;
          if (kb >= num_kb) break;
          uint4 o;
          uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t v = word(cur[c], j);
            if (tail_skip && kb == num_kb - 1) {
              // bytes of sub-blocks [K/32 - 4, K/32): the last (4 - tail_skip) bytes of the
              // previous word followed by the first tail_skip... of this one
              const uint32_t before = j > 0 ? word(cur[c], j - 1) : prev_last[c];
              v = __funnelshift_r(before, v, 8 * (4 - tail_skip));
            }
            ow[c] = v;
          }
          ok = mbar_wait_spin(&bars.empty[stage], phase ^ 1u, abort_p);
          if (!ok) break;
          *reinterpret_cast<uint4*>(sfa_smem + stage * kMxSfaBytes + lane * 16) = o;
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.full[stage]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) prev_last[c] = cur[c].w;
      }
    }
  } else if (warp >= 4) {
    // ---------------- accumulator readers / epilogue ----------------
    const int quad = warp & 3;
    const int g = (warp - 4) >> 2;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    int buf = 0;
    uint32_t buf_phase = 0;
    bool ok = true;
    for (int t = sched_id; t < num_tiles && ok; t += sched_stride) {
      const TileCoord tc = decode_tile(sched, t);
      const bool row_ok = row_in_tile < tc.rows_valid;
      const int64_t grow = static_cast<int64_t>(tc.row_start) + row_in_tile;
      float acc[64];
      ok = mbar_wait(&bars.tfull[buf], buf_phase, abort_p);
      if (!ok) break;
      tc_fence_after();
      const uint32_t src = tmem_base + lane_addr + buf * C::ACC_STRIDE + g * 64;
      tmem_ld_32x32(src, *reinterpret_cast<float(*)[32]>(acc));
      tmem_ld_32x32(src + 32, *reinterpret_cast<float(*)[32]>(acc + 32));
      tmem_ld_wait_on2(*reinterpret_cast<float(*)[32]>(acc), *reinterpret_cast<float(*)[32]>(acc + 32));
      // the accumulator is in registers: the MMA warp may start the tile after next
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.tempty[buf]);
      if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
      mx_tile_epilogue<C>(p, tc, g, row_ok, grow, acc);
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    if (threadIdx.x == 0) atomicExch(&g_device_status, B200MOE_TIMEOUT);
    for (int i = 0; i < 64; ++i) __nanosleep(10000);  // copies in flight land before smem is released
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// Tensor map over packed e2m1 pairs, [batch, rows, cols] with `cols` 4-bit elements per
// row (a multiple of 128), box 128 x box_rows; elements arrive in shared memory one per
// byte container (16 elements = 8 bytes of data + 8 bytes of padding), 128-byte swizzle.
inline int make_map_fp4(CUtensorMap* map, const void* base, uint64_t cols, uint64_t row_pitch_bytes,
                        uint64_t rows, uint64_t batch, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return B200MOE_CUDA_ERROR;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {row_pitch_bytes, row_pitch_bytes * rows};
  cuuint32_t box[3] = {128, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, const_cast<void*>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled (packed 4-bit)", cudaErrorInvalidValue);
    return B200MOE_CUDA_ERROR;
  }
  return B200MOE_OK;
}

template <typename C>
int launch_mx(const b200moe_mx_gemm_args& a, cudaStream_t st) {
  CUtensorMap map_a, map_b, map_b_tail;
  int rc = make_map(&map_a, B200MOE_E4M3, a.A, a.K, a.R, 0, kMxBK, BM);
  if (rc != B200MOE_OK) return rc;
  const uint64_t pitch = static_cast<uint64_t>(a.K) / 2;
  const uint64_t k_main = static_cast<uint64_t>(a.K / kMxBK) * kMxBK;
  rc = make_map_fp4(&map_b, a.B, k_main, pitch, a.N, a.E, C::BN);
  if (rc != B200MOE_OK) return rc;
  // the last 128 elements of every row, for a K that is not a multiple of 128
  rc = make_map_fp4(&map_b_tail, reinterpret_cast<const uint8_t*>(a.B) + (a.K - kMxBK) / 2, kMxBK,
                    pitch, a.N, a.E, C::BN);
  if (rc != B200MOE_OK) return rc;

  MxParams p;
  p.a_sf = a.a_sf;
  p.a_sf_pitch = a.a_sf_pitch;
  p.b_sf = a.b_sf;
  p.b_atoms = (a.N + 127) / 128 + 1;
  p.bias = a.bias;
  p.bias_dtype = a.bias_dtype;
  p.D = a.D;
  p.d_dtype = a.d_dtype;
  p.ldd = a.epilogue == B200MOE_EPI_STORE ? a.N : a.N / 2;
  p.d_sf = a.d_sf;
  p.d_sf_pitch = a.d_sf_pitch;
  p.rows_per_expert = a.rows_per_expert;
  p.R = a.R;
  p.N = a.N;
  p.K = a.K;
  p.E = a.E;
  p.alpha = a.alpha;
  p.limit = a.limit;
  rc = ensure_dynamic_smem<C>(grouped_gemm_mx_kernel<C>, C::SMEM_BYTES, "cudaFuncSetAttribute (mx)");
  if (rc != B200MOE_OK) return rc;
  const int n_tiles = (a.N + C::BN - 1) / C::BN;
  int64_t grid = ((a.R + BM - 1) / BM + a.E) * n_tiles;
  if (grid > kNumSMs) grid = kNumSMs;
  if (grid < 1) grid = 1;
  grouped_gemm_mx_kernel<C><<<static_cast<int>(grid), C::THREADS, C::SMEM_BYTES, st>>>(
      map_a, map_b, map_b_tail, p);
  return launch_status("grouped_gemm_mx_kernel");
}

// Weight scales [E, N, K/32] (e8m0 bytes) -> [E, ceil(K/128), ceil(N/128)+1, 512]: per
// (expert, K block, 128 rows) the 512 bytes tcgen05.cp wants, byte (n%32)*16 + (n%128/32)*4 + j
// holding the scale of row n and sub-block j of that K block.  A last K block that starts at
// K-128 gets the sub-blocks it really covers.  Rows past N and the extra piece hold 1.0.
__global__ void mx_prepare_weight_scales_kernel(const uint8_t* __restrict__ s, uint8_t* __restrict__ out,
                                                int E, int N, int K, int64_t total_words) {
  const int num_kb = (K + kMxBK - 1) / kMxBK;
  const int atoms = (N + 127) / 128 + 1;
  const int sub_total = K / 32;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total_words;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int in_atom = static_cast<int>(i % 128);  // word index: lane * 4 + column
    int64_t rest = i / 128;
    const int atom = static_cast<int>(rest % atoms);
    rest /= atoms;
    const int kb = static_cast<int>(rest % num_kb);
    const int e = static_cast<int>(rest / num_kb);
    const int n = atom * 128 + (in_atom & 3) * 32 + (in_atom >> 2);
    const int sub0 = (kb == num_kb - 1 && (K % kMxBK)) ? sub_total - 4 : kb * 4;
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t b = 127;
      if (n < N && sub0 + j < sub_total)
        b = s[(static_cast<int64_t>(e) * N + n) * sub_total + sub0 + j];
      w |= b << (8 * j);
    }
    reinterpret_cast<uint32_t*>(out)[i] = w;
  }
}
