// Grouped GEMM for the decode regime (a handful of rows per expert), FP8 block-scaled.
//
// With 1..32 rows per expert a 128-row activation tile is almost all padding and the
// layer is pure weight streaming.  This kernel swaps the operands of the MMA: the
// WEIGHT tile is the M side (128 output features x 128 of K, read in the operator's own
// [E,K,N] layout as an MN-major operand) and the expert's tokens are the N side (32
// columns).  A pipeline stage is then 16 KB (32 KB for gate+up) of weights from HBM plus
// 4 KB of tokens from L2, so almost every byte in flight is a weight byte, and the tile
// count (experts x feature tiles x token chunks) is large enough to balance 148 SMs.
//
// Measured on the DeepSeek-V3 shape: with all scales of a tile staged in shared memory and
// the output quantised in the epilogue, a layer of 1..32 tokens is 4-6 % faster on this
// kernel than on the 128-row-tile kernel; from about four rows per expert on it is slower
// (hot experts need several 32-token chunks, each streaming the weights again).  Callers
// select it with the activation-scale layout code.
//
//   accumulator (tensor memory): lanes = output features, columns = tokens
//   per 128 of K:  acc[f][t] += a_scale[kb][t] * b_scale[kb][f/128] * partial[f][t]
//   epilogue:      store (+bias) or silu(gate)*up, written token-major so that the 32
//                  lanes of a warp store 32 neighbouring features of one token.
//
// Activation scales are taken K-block-major ([K/128, R]) or row-major ([R, K/128]); either
// way they are read once per tile into shared memory.  Warp roles, mbarrier protocol and the bounded waits
// are those of the prefill kernel (grouped_gemm.cu).
// (included by grouped_gemm.cu inside its translation-unit-local namespace)

constexpr int kNTok = 32;          // tokens per tile (MMA N)
constexpr int kFeat = 128;         // output features per tile (MMA M)
constexpr int kBK = 128;           // K per stage (fp8: one 128-byte swizzle row)
constexpr int kWBytes = kBK * 128; // one weight tile: 128 K rows x 128 feature bytes
constexpr int kTokBytes = kNTok * 128;
constexpr int kMaxExperts = 1024;

struct DecodeParams {
  const float* a_scale_t;  // [K/128, R] K-block-major, or [R, K/128] when a_row_major
  int a_row_major;
  float* d_scale;          // [R, N_out/128] when D is e4m3 (gated epilogue only)
  const float* b_scale;    // [E, K/128, N/128]
  const void* bias;
  int bias_dtype;
  void* D;
  int d_dtype;
  const int32_t* rows_per_expert;
  int64_t R;
  int N, K, E;
  int ldd;
};

struct DecodeSchedule {
  int tile_prefix[kMaxExperts + 1];  // tiles (feature tiles x token chunks) before expert e
  int row_prefix[kMaxExperts + 1];
  int num_experts;
  int f_tiles;
};

__device__ __forceinline__ void build_decode_schedule(DecodeSchedule& s, const int32_t* rows_per_expert,
                                                      int E, int64_t R, int f_tiles) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int tile_run = 0;
    long long row_run = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + lane;
      long long rows = e < E ? rows_per_expert[e] : 0;
      if (rows < 0) rows = 0;
      long long incl_rows = rows;
      const int tiles = static_cast<int>((rows + kNTok - 1) / kNTok) * f_tiles;
      int incl_tiles = tiles;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const long long r = __shfl_up_sync(0xffffffffu, incl_rows, off);
        const int t = __shfl_up_sync(0xffffffffu, incl_tiles, off);
        if (lane >= off) { incl_rows += r; incl_tiles += t; }
      }
      if (e < E) {
        const long long rs = row_run + incl_rows - rows;
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
      s.f_tiles = f_tiles;
    }
  }
}

struct DecodeTile {
  int expert, row_start, rows_valid, f_tile;
};

// Tiles of one expert are ordered feature tile major, token chunk minor, so the chunks that
// share a weight tile run next to each other.
__device__ __forceinline__ DecodeTile decode_tile(const DecodeSchedule& s, int t) {
  int lo = 0, hi = s.num_experts;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s.tile_prefix[mid] <= t) lo = mid; else hi = mid;
  }
  // skip experts without tiles that share the prefix value
  while (lo + 1 < s.num_experts && s.tile_prefix[lo + 1] <= t) ++lo;
  const int rows_e = s.row_prefix[lo + 1] - s.row_prefix[lo];
  const int chunks = (rows_e + kNTok - 1) / kNTok;
  const int within = t - s.tile_prefix[lo];
  DecodeTile d;
  d.expert = lo;
  d.f_tile = within / (chunks > 0 ? chunks : 1);
  const int c = within - d.f_tile * chunks;
  d.row_start = s.row_prefix[lo] + c * kNTok;
  const int left = rows_e - c * kNTok;
  d.rows_valid = left < kNTok ? (left < 0 ? 0 : left) : kNTok;
  return d;
}

__device__ __forceinline__ void store16(void* D, int dtype, int64_t at, float v) {
  if (dtype == B200MOE_BF16) reinterpret_cast<__nv_bfloat16*>(D)[at] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(D)[at] = __float2half_rn(v);
}

struct alignas(8) DecodeBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tfull[4];
  uint64_t tempty[4];
  uint64_t sfree, sready;  // hand-over of the staged-scales buffer between tiles (4 reader warps)
  uint64_t qready;         // quantising epilogue: every warp's per-token maxima are in shared memory
};

// GATED: two weight tiles per stage (gate features f, up features N/2 + f), epilogue
// silu(gate)*up into D [R, N/2].  Otherwise one weight tile and a plain store into D [R, N].
template <bool GATED>
struct DecodeConfig {
  static constexpr int W_TILES = GATED ? 2 : 1;
  static constexpr int STAGE_BYTES = W_TILES * kWBytes + kTokBytes;
  static constexpr int STAGES = GATED ? 5 : 8;
  static constexpr int ACC_COLS = 64;   // per buffer: gate 32 | up 32 (plain uses the first 32)
  static constexpr int ACC_BUFS = 4;
  static constexpr int TMEM_COLS = 256;
  static constexpr int THREADS = 256;   // warp 0 producer, warp 1 MMA, warps 4..7 readers
  static constexpr size_t SMEM_BYTES = 1024 + static_cast<size_t>(STAGES) * STAGE_BYTES;
  static_assert(SMEM_BYTES > 116 * 1024, "one CTA per SM is assumed");
};

template <bool GATED>
__global__ void __launch_bounds__(256, 1)
decode_gemm_kernel(const __grid_constant__ CUtensorMap map_tok,
                   const __grid_constant__ CUtensorMap map_w, DecodeParams p) {
  using C = DecodeConfig<GATED>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ DecodeSchedule sched;
  __shared__ DecodeBarriers bars;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float qmax[4][kNTok];  // quantising epilogue: per reader warp, per token

  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_out = GATED ? p.N / 2 : p.N;            // output features
  const int f_tiles = (n_out + kFeat - 1) / kFeat;
  const int num_kb = p.K / kBK;
  // after the operand stages: this tile's activation scales [K/128][32] and weight scales [K/128][2]
  float* sa_s = reinterpret_cast<float*>(tiles + C::STAGES * C::STAGE_BYTES);
  float* sb_s = sa_s + num_kb * kNTok;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&bars.full[s], 1);
      mbar_init(&bars.empty[s], 1);
    }
    for (int b = 0; b < C::ACC_BUFS; ++b) {
      mbar_init(&bars.tfull[b], 1);
      mbar_init(&bars.tempty[b], 4);
    }
    mbar_init(&bars.sfree, 4);
    mbar_init(&bars.sready, 4);
    mbar_init(&bars.qready, 4);
    mbar_fence_init();
    prefetch_tensormap(&map_tok);
    prefetch_tensormap(&map_w);
  }
  build_decode_schedule(sched, p.rows_per_expert, p.E, p.R, f_tiles);
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const int num_tiles = sched.tile_prefix[sched.num_experts];
  volatile int* abort_p = &abort_flag;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const DecodeTile tc = decode_tile(sched, t);
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        ok = mbar_wait(&bars.empty[stage], phase ^ 1u, abort_p);
        if (!ok) break;
        uint8_t* w_dst = tiles + stage * C::STAGE_BYTES;
        uint8_t* tok_dst = w_dst + C::W_TILES * kWBytes;
        mbar_arrive_expect_tx(&bars.full[stage], C::STAGE_BYTES);
        tma_load_3d(w_dst, &map_w, &bars.full[stage], tc.f_tile * kFeat, kb * kBK, tc.expert);
        if (GATED)
          tma_load_3d(w_dst + kWBytes, &map_w, &bars.full[stage], p.N / 2 + tc.f_tile * kFeat,
                      kb * kBK, tc.expert);
        tma_load_2d(tok_dst, &map_tok, &bars.full[stage], kb * kBK, tc.row_start);
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    // A = weights, MN-major (features contiguous); B = tokens, K-major; e4m3 x e4m3 -> fp32
    const uint32_t idesc = make_idesc(0u, 0u, 1u, 0u, kFeat, kNTok);
    const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version, 128-byte swizzle
    const uint32_t w_lo0 = ((smem_u32(tiles) & 0x3FFFFu) >> 4) | ((kWBytes >> 4) << 16);
    const uint32_t tok_lo0 = (((smem_u32(tiles) + C::W_TILES * kWBytes) & 0x3FFFFu) >> 4) | ((16u >> 4) << 16);
    int stage = 0;
    uint32_t phase = 0;
    int buf = 0;
    uint32_t buf_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        ok = mbar_wait(&bars.tempty[buf], buf_phase ^ 1u, abort_p);
        if (!ok) break;
        ok = mbar_wait(&bars.full[stage], phase, abort_p);
        if (!ok) break;
        tc_fence_after();
        // descriptors: constant high word, low words = base + stage * constant (+ an
        // immediate per K slice): what this one thread computes between two MMAs is time
        // the tensor pipe idles
        const uint32_t w_lo = w_lo0 + stage * (C::STAGE_BYTES >> 4);
        const uint32_t tok_lo = tok_lo0 + stage * (C::STAGE_BYTES >> 4);
        const uint32_t d_tmem = tmem_base + buf * C::ACC_COLS;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t b_desc = (static_cast<uint64_t>(desc_hi) << 32) | (tok_lo + kk * 2);
          const uint64_t a_gate = (static_cast<uint64_t>(desc_hi) << 32) | (w_lo + kk * ((32 * 128) >> 4));
          mma_f8(d_tmem, a_gate, b_desc, idesc, kk > 0 ? 1u : 0u);
          if (GATED) {
            const uint64_t a_up = (static_cast<uint64_t>(desc_hi) << 32) |
                                  (w_lo + (kWBytes >> 4) + kk * ((32 * 128) >> 4));
            mma_f8(d_tmem + kNTok, a_up, b_desc, idesc, kk > 0 ? 1u : 0u);
          }
        }
        mma_commit(&bars.empty[stage]);
        mma_commit(&bars.tfull[buf]);
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        if (++buf == C::ACC_BUFS) { buf = 0; buf_phase ^= 1u; }
      }
    }
  } else if (warp >= 4) {
    // ---------------- accumulator readers / epilogue ----------------
    const int quad = warp & 3;
    const int f_local = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int nb_count = p.N / 128;
    int buf = 0;
    uint32_t buf_phase = 0;
    uint32_t tile_parity = 0;
    uint32_t quant_parity = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const DecodeTile tc = decode_tile(sched, t);
      float accg[kNTok], accu[GATED ? kNTok : 1];
#pragma unroll
      for (int j = 0; j < kNTok; ++j) accg[j] = 0.f;
      if (GATED) {
#pragma unroll
        for (int j = 0; j < kNTok; ++j) accu[GATED ? j : 0] = 0.f;
      }
      const int f0 = tc.f_tile * kFeat;
      const int nb_g = f0 / 128 < nb_count ? f0 / 128 : nb_count - 1;
      const int nb_u = GATED ? ((p.N / 2 + f0) / 128 < nb_count ? (p.N / 2 + f0) / 128 : nb_count - 1) : 0;
      const float* sb_ptr = p.b_scale + static_cast<int64_t>(tc.expert) * num_kb * nb_count;
      // All scales of the tile go to shared memory first (one round trip to L2 per tile):
      // a load per K block would put that latency on every step of the readers' chain,
      // which is what paces this kernel.
      // (mbarriers with the bounded wait rather than a named barrier: a warp that gave up on
      // a wait must not leave the others parked)
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.sfree);   // this warp is done with the last tile's scales
      ok = mbar_wait(&bars.sfree, tile_parity, abort_p);
      if (!ok) break;
      {
        const int rt = threadIdx.x - 128;
        for (int i = rt; i < num_kb * kNTok; i += 128) {
          const int j = i & (kNTok - 1);
          const int kb = i / kNTok;
          sa_s[i] = j >= tc.rows_valid ? 0.f
                    : p.a_row_major    ? p.a_scale_t[static_cast<int64_t>(tc.row_start + j) * num_kb + kb]
                                       : p.a_scale_t[static_cast<int64_t>(kb) * p.R + tc.row_start + j];
        }
        for (int i = rt; i < 2 * num_kb; i += 128)
          sb_s[i] = sb_ptr[(i >> 1) * nb_count + ((i & 1) ? nb_u : nb_g)];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.sready);
      ok = mbar_wait(&bars.sready, tile_parity, abort_p);
      if (!ok) break;
      tile_parity ^= 1u;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        // scales of this K block: one per token (same for every lane) and one per weight block
        float sa[kNTok];
#pragma unroll
        for (int j = 0; j < kNTok; j += 4) {
          const float4 v = *reinterpret_cast<const float4*>(sa_s + kb * kNTok + j);
          sa[j] = v.x; sa[j + 1] = v.y; sa[j + 2] = v.z; sa[j + 3] = v.w;
        }
        const float sbg = sb_s[2 * kb];
        const float sbu = GATED ? sb_s[2 * kb + 1] : 0.f;
        ok = mbar_wait(&bars.tfull[buf], buf_phase, abort_p);
        if (!ok) break;
        tc_fence_after();
        float vg[32], vu[32];
        const uint32_t t_addr = tmem_base + lane_addr + buf * C::ACC_COLS;
        tmem_ld_32x32(t_addr, vg);
        if (GATED) tmem_ld_32x32(t_addr + kNTok, vu);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.tempty[buf]);
        if (++buf == C::ACC_BUFS) { buf = 0; buf_phase ^= 1u; }
#pragma unroll
        for (int j = 0; j < kNTok; ++j) {
          accg[j] = fmaf(sa[j] * sbg, vg[j], accg[j]);
          if (GATED) accu[GATED ? j : 0] = fmaf(sa[j] * sbu, vu[j], accu[GATED ? j : 0]);
        }
      }
      if (!ok) break;
      const int f = f0 + f_local;
      float bg = 0.f, bu = 0.f;
      if (p.bias && f < n_out) {
        bg = load_bias(p.bias, p.bias_dtype, static_cast<int64_t>(tc.expert) * p.N + f);
        if (GATED) bu = load_bias(p.bias, p.bias_dtype, static_cast<int64_t>(tc.expert) * p.N + p.N / 2 + f);
      }
#pragma unroll
      for (int j = 0; j < kNTok; ++j) {
        float v = accg[j] + bg;
        if (GATED) {
          const float u = accu[GATED ? j : 0] + bu;
          v = v * fast_sigmoid(v) * u;
        }
        accg[j] = v;
      }
      if (GATED && p.d_dtype == B200MOE_E4M3) {
        // Per-token-group-128 quantisation: the tile's 128 features are one group of each of
        // its tokens.  Per token: maximum over the warp's 32 features by shuffles, over the
        // four warps through shared memory, then one e4m3 byte per (token, feature).
#pragma unroll
        for (int j = 0; j < kNTok; ++j) {
          if (j < tc.rows_valid) {
            float m = f < n_out ? fabsf(accg[j]) : 0.f;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
            if (lane == 0) qmax[quad][j] = m;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.qready);
        ok = mbar_wait(&bars.qready, quant_parity, abort_p);
        if (!ok) break;
        quant_parity ^= 1u;
        uint8_t* out = reinterpret_cast<uint8_t*>(p.D);
#pragma unroll
        for (int j = 0; j < kNTok; ++j) {
          if (j < tc.rows_valid) {
            const float amax = fmaxf(fmaxf(qmax[0][j], qmax[1][j]), fmaxf(qmax[2][j], qmax[3][j]));
            const float sc = fmaxf(amax * (1.0f / 448.0f), 1.0f / (448.0f * 512.0f));
            const int64_t row = tc.row_start + j;
            if (f < n_out) {
              const float q = fmaxf(-448.0f, fminf(accg[j] * (1.0f / sc), 448.0f));
              out[row * p.ldd + f] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3));
            }
            if (f_local == 0) p.d_scale[row * (n_out / 128) + tc.f_tile] = sc;
          }
        }
        // qmax is rewritten by the next tile only after every warp passed that tile's
        // scale hand-over, i.e. after it finished reading here
      } else if (f < n_out) {
#pragma unroll
        for (int j = 0; j < kNTok; ++j)
          if (j < tc.rows_valid)
            store16(p.D, p.d_dtype, static_cast<int64_t>(tc.row_start + j) * p.ldd + f, accg[j]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    if (threadIdx.x == 0) atomicExch(&g_device_status, B200MOE_TIMEOUT);
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <bool GATED>
int launch_decode(const b200moe_gemm_args& a, cudaStream_t st) {
  using C = DecodeConfig<GATED>;
  CUtensorMap map_tok, map_w;
  int rc = make_map(&map_tok, B200MOE_E4M3, a.A, a.K, a.R, 0, kBK, kNTok);
  if (rc != B200MOE_OK) return rc;
  rc = make_map(&map_w, B200MOE_E4M3, a.B, a.N, a.K, a.E, 128, kBK);
  if (rc != B200MOE_OK) return rc;
  DecodeParams p;
  p.a_scale_t = a.a_scale;
  p.a_row_major = a.a_scale_layout == B200MOE_A_SCALE_ROW_MAJOR_DECODE;
  p.d_scale = a.d_scale;
  p.b_scale = reinterpret_cast<const float*>(a.b_scale);
  p.bias = a.bias;
  p.bias_dtype = a.bias_dtype;
  p.D = a.D;
  p.d_dtype = a.d_dtype;
  p.rows_per_expert = a.rows_per_expert;
  p.R = a.R;
  p.N = a.N;
  p.K = a.K;
  p.E = a.E;
  p.ldd = GATED ? a.N / 2 : a.N;
  constexpr int kMaxDecodeKBlocks = 160;  // K <= 20480: the staged scales fit beside the stages
  if (a.K / kBK > kMaxDecodeKBlocks) return B200MOE_UNSUPPORTED;
  const size_t smem = C::SMEM_BYTES + static_cast<size_t>(a.K / kBK) * (kNTok + 2) * sizeof(float);
  struct Tag {};  // one record per instantiation of this function
  const int arc = ensure_dynamic_smem<Tag>(
      decode_gemm_kernel<GATED>, C::SMEM_BYTES + kMaxDecodeKBlocks * (kNTok + 2) * sizeof(float),
      "cudaFuncSetAttribute");
  if (arc != B200MOE_OK) return arc;
  decode_gemm_kernel<GATED><<<kNumSMs, C::THREADS, smem, st>>>(map_tok, map_w, p);
  return launch_status("decode_gemm_kernel");
}

// Entry used by b200moe_grouped_gemm when the caller asks for the decode form
// (a_scale_layout = K-block-major, or row-major with the decode selector).
int grouped_gemm_decode(const b200moe_gemm_args& a, cudaStream_t st) {
  if (a.recipe != B200MOE_RECIPE_FP8_BLOCK || a.a_dtype != B200MOE_E4M3 || !a.a_scale || !a.b_scale)
    return B200MOE_UNSUPPORTED;
  if (a.K % 128 || a.N % 128 || a.E > kMaxExperts) return B200MOE_INVALID_ARG;
  const bool quant_out = a.d_dtype == B200MOE_E4M3;
  if (!quant_out && a.d_dtype != B200MOE_BF16 && a.d_dtype != B200MOE_F16) return B200MOE_UNSUPPORTED;
  if (quant_out && (a.epilogue != B200MOE_EPI_SILU_MUL || !a.d_scale)) return B200MOE_UNSUPPORTED;
  if (a.d_row_ptr) return B200MOE_UNSUPPORTED;
  if (a.epilogue == B200MOE_EPI_STORE) return launch_decode<false>(a, st);
  if (a.epilogue == B200MOE_EPI_SILU_MUL) {
    if ((a.N / 2) % 128) return B200MOE_UNSUPPORTED;
    return launch_decode<true>(a, st);
  }
  return B200MOE_UNSUPPORTED;
}
