"""Grouped GEMM on the tensor cores against the CPU oracle (dequantise, then
fp32 matmul per expert) and, at sizes a CPU cannot reach, against the plain
CUDA-core evaluation of the same contract.  Tolerance: 2e-2 absolute+relative,
the reference's bf16 bound (tests/fused_moe/test_grouped_gemm.py there)."""
import ctypes

import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
EPI_STORE, EPI_SILU, EPI_OAI = 0, 1, 2
KN, NK = 0, 1


def ragged_rows(E, avg, seed, zero_some=True):
    g = torch.Generator().manual_seed(seed)
    rows = torch.randint(0, 2 * avg + 1, (E,), generator=g).to(torch.int32)
    if zero_some and E > 2:
        rows[1] = 0
        rows[E - 1] = 0
    return rows


def close(out, ref, tol=2e-2):
    out, ref = out.float().cpu(), ref.float().cpu()
    err = (out - ref).abs()
    bound = tol + tol * ref.abs()
    assert (err <= bound).all(), (
        f"max err {err.max().item():.4g} at {torch.nonzero(err > bound)[:5].tolist()} "
        f"({int((err > bound).sum())} of {err.numel()} outside {tol})")


def make_bf16(E, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(E, K, N, generator=g) / K ** 0.5).to(torch.bfloat16)


@pytest.mark.parametrize("E,avg,K,N", [(1, 64, 64, 128), (4, 100, 256, 256), (8, 16, 1024, 4096),
                                       (3, 200, 72, 136), (16, 4, 512, 384), (2, 300, 4096, 1024)])
@pytest.mark.parametrize("layout", [KN, NK])
def test_bf16_store(ops, E, avg, K, N, layout):
    rows = ragged_rows(E, avg, E + K)
    R = int(rows.sum())
    if R == 0:
        rows[0] = 5
        R = 5
    g = torch.Generator().manual_seed(N)
    A = torch.randn(R, K, generator=g).to(torch.bfloat16)
    B = make_bf16(E, K, N, K)
    bias = (torch.randn(E, N, generator=g) * 0.1).to(torch.bfloat16)
    ref = O.grouped_gemm("bf16", A, B, None, bias, rows, torch.float32)
    Bdev = B.to(DEV) if layout == KN else B.transpose(1, 2).contiguous().to(DEV)
    D = torch.zeros(R, N, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.b200_grouped_gemm(A.to(DEV), None, Bdev, None, bias.to(DEV), D, rows.to(DEV), N, K, E,
                                 EPI_STORE, layout)
    close(D, ref)
    if layout == KN:  # the reference-named entry is the same path
        D2 = torch.zeros_like(D)
        r = ops._xpu_C.cutlass_grouped_gemm_interface(A.to(DEV), None, Bdev, None, bias.to(DEV), D2,
                                                      rows.to(DEV), N, K, E)
        assert r.data_ptr() == D2.data_ptr() and torch.equal(D, D2)


def test_rows_beyond_an_expert_are_untouched(ops):
    E, K, N = 3, 128, 128
    rows = torch.tensor([5, 0, 130], dtype=torch.int32)
    R = 200                                     # more rows than the experts own
    A = torch.randn(R, K).to(torch.bfloat16)
    B = make_bf16(E, K, N, 1)
    D = torch.full((R, N), 7.0, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.b200_grouped_gemm(A.to(DEV), None, B.to(DEV), None, None, D, rows.to(DEV), N, K, E,
                                 EPI_STORE, KN)
    assert (D[135:] == 7.0).all()
    ref = O.grouped_gemm("bf16", A[:135], B, None, None, rows, torch.float32)
    close(D[:135], ref)


@pytest.mark.parametrize("epi", [EPI_SILU, EPI_OAI])
@pytest.mark.parametrize("layout", [KN, NK])
@pytest.mark.parametrize("E,avg,K,N", [(4, 90, 256, 512), (8, 40, 1024, 4096), (2, 150, 192, 5760)])
def test_bf16_gated_epilogue(ops, epi, layout, E, avg, K, N):
    rows = ragged_rows(E, avg, 3)
    R = int(rows.sum())
    g = torch.Generator().manual_seed(5)
    A = torch.randn(R, K, generator=g).to(torch.bfloat16)
    B = make_bf16(E, K, N, 9)
    bias = (torch.randn(E, N, generator=g) * 0.1).to(torch.bfloat16)
    h = O.grouped_gemm("bf16", A, B, None, bias, rows, torch.float32)
    ref = O.silu_mul_fp32(h) if epi == EPI_SILU else O.swigluoai_and_mul(h)
    Bdev = B.to(DEV) if layout == KN else B.transpose(1, 2).contiguous().to(DEV)
    D = torch.zeros(R, N // 2, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.b200_grouped_gemm(A.to(DEV), None, Bdev, None, bias.to(DEV), D, rows.to(DEV), N, K, E,
                                 epi, layout, 1.702, 7.0)
    close(D, ref)


@pytest.mark.parametrize("E,avg,K,N", [(1, 128, 128, 128), (4, 100, 512, 256), (8, 30, 4096, 1024),
                                       (2, 260, 7168, 512)])
def test_fp8_block(ops, E, avg, K, N):
    rows = ragged_rows(E, avg, K)
    R = max(int(rows.sum()), 1)
    if int(rows.sum()) == 0:
        rows[0] = 1
    g = torch.Generator().manual_seed(N + 1)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    Aq, As = O.per_token_group_fp8_quant(x, 128)
    Bq, Bs = zip(*[O.quant_fp8_block_weight(torch.randn(K, N, generator=g) / K ** 0.5) for _ in range(E)])
    Bq, Bs = torch.stack(Bq), torch.stack(Bs)
    # distinct scales per block so that a mis-indexed scale shows
    Bs = Bs * (1.0 + 0.25 * torch.rand(Bs.shape, generator=g))
    ref = O.grouped_gemm("fp8block", O.dequant_fp8_group_act(Aq, As), Bq, Bs, None, rows, torch.float32)
    D = torch.zeros(R, N, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), None, D, rows.to(DEV),
                                 N, K, E, EPI_STORE, KN)
    close(D, ref)


@pytest.mark.parametrize("pair", ["0", "1"])
@pytest.mark.parametrize("E,avg,K,N", [(1, 300, 512, 256), (3, 700, 1024, 512)])
def test_fp8_unit_scales(ops, E, avg, K, N, pair, monkeypatch):
    """No scales at all: the plain e4m3 x e4m3 contraction (one accumulation phase per tile)
    that the benchmark uses as its same-dtype ceiling.  Exact products, fp32 sums."""
    monkeypatch.setenv("B200MOE_PAIR", pair)
    monkeypatch.setenv("B200MOE_TILE_N", "256")
    rows = ragged_rows(E, avg, K)
    if int(rows.sum()) == 0:
        rows[0] = 1
    R = int(rows.sum())
    g = torch.Generator().manual_seed(K)
    A = torch.randn(R, K, generator=g).to(torch.float8_e4m3fn)
    B = (torch.randn(E, K, N, generator=g) / K ** 0.5).to(torch.float8_e4m3fn)
    ref = O.grouped_gemm("bf16", A.float(), B.float(), None, None, rows, torch.float32)
    D = torch.zeros(R, N, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.b200_grouped_gemm(A.to(DEV), None, B.to(DEV), None, None, D, rows.to(DEV), N, K, E,
                                 EPI_STORE, KN)
    close(D, ref)


@pytest.mark.parametrize("tile_n,pair", [("128", "0"), ("256", "0"), ("256", "1")])
@pytest.mark.parametrize("kind", ["bf16_kn", "bf16_nk", "fp8"])
def test_every_tile_shape(ops, tile_n, pair, kind, monkeypatch):
    """Tile width and CTA pairing (two CTAs sharing one 256-row MMA) are normally
    picked from the problem size; force each combination."""
    monkeypatch.setenv("B200MOE_TILE_N", tile_n)
    monkeypatch.setenv("B200MOE_PAIR", pair)
    E, K, N = 3, 512, 768
    rows = torch.tensor([130, 0, 257], dtype=torch.int32)
    R = 387
    g = torch.Generator().manual_seed(11)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    D = torch.zeros(R, N, dtype=torch.bfloat16, device=DEV)
    if kind == "fp8":
        Aq, As = O.per_token_group_fp8_quant(x, 128)
        Bq, Bs = zip(*[O.quant_fp8_block_weight(torch.randn(K, N, generator=g) / K ** 0.5) for _ in range(E)])
        Bq, Bs = torch.stack(Bq), torch.stack(Bs) * (1.0 + 0.25 * torch.rand(E, K // 128, N // 128, generator=g))
        ref = O.grouped_gemm("fp8block", O.dequant_fp8_group_act(Aq, As), Bq, Bs, None, rows, torch.float32)
        ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), None, D, rows.to(DEV),
                                     N, K, E, EPI_STORE, KN)
    else:
        B = make_bf16(E, K, N, 3)
        bias = (torch.randn(E, N, generator=g) * 0.1).to(torch.bfloat16)
        ref = O.grouped_gemm("bf16", x, B, None, bias, rows, torch.float32)
        layout = KN if kind == "bf16_kn" else NK
        Bd = B.to(DEV) if layout == KN else B.transpose(1, 2).contiguous().to(DEV)
        ops._xpu_C.b200_grouped_gemm(x.to(DEV), None, Bd, None, bias.to(DEV), D, rows.to(DEV), N, K, E,
                                     EPI_STORE, layout)
        for epi in (EPI_SILU, EPI_OAI):
            D2 = torch.zeros(R, N // 2, dtype=torch.bfloat16, device=DEV)
            ops._xpu_C.b200_grouped_gemm(x.to(DEV), None, Bd, None, bias.to(DEV), D2, rows.to(DEV), N, K, E,
                                         epi, layout, 1.702, 7.0)
            close(D2, O.silu_mul_fp32(ref) if epi == EPI_SILU else O.swigluoai_and_mul(ref))
    close(D, ref)


@pytest.mark.parametrize("offload", ["0", "1"])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("E,rows_list,K,N", [(3, [130, 0, 257], 512, 768), (4, [1, 255, 256, 300], 384, 384),
                                            (2, [700, 129], 1280, 1152)])
def test_fp8_pair_store_through_the_spare_warps(ops, E, rows_list, K, N, out_dtype, offload, monkeypatch):
    """Block-scaled FP8 store GEMM on CTA pairs: the finished tile leaves through a staging tile
    in shared memory and the two spare warps (default), or through the reader warps
    (B200MOE_STORE_OFFLOAD=0).  Ragged experts (an empty one, one row, a row more than a tile),
    a tile that hangs over the right edge (N = 384, 1152), several tiles per CTA pair so that
    the staging tile is reused, a bias.  Both ways give the same bits."""
    monkeypatch.setenv("B200MOE_TILE_N", "256")
    monkeypatch.setenv("B200MOE_PAIR", "1")
    monkeypatch.setenv("B200MOE_STORE_OFFLOAD", offload)
    rows = torch.tensor(rows_list, dtype=torch.int32)
    R = int(rows.sum())
    g = torch.Generator().manual_seed(K + N)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    Aq, As = O.per_token_group_fp8_quant(x, 128)
    Bq, Bs = zip(*[O.quant_fp8_block_weight(torch.randn(K, N, generator=g) / K ** 0.5) for _ in range(E)])
    Bq, Bs = torch.stack(Bq), torch.stack(Bs) * (1.0 + 0.25 * torch.rand(E, K // 128, N // 128, generator=g))
    bias = (torch.randn(E, N, generator=g) * 0.1).to(torch.bfloat16)
    ref = O.grouped_gemm("fp8block", O.dequant_fp8_group_act(Aq, As), Bq, Bs, bias, rows, torch.float32)
    guard = 64  # rows after the last expert must stay untouched
    D = torch.full((R + guard, N), 7.0, dtype=out_dtype, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), bias.to(DEV), D[:R],
                                 rows.to(DEV), N, K, E, EPI_STORE, KN)
    close(D[:R], ref)
    assert bool((D[R:] == 7.0).all())
    monkeypatch.setenv("B200MOE_STORE_OFFLOAD", "0")
    D0 = torch.zeros(R, N, dtype=out_dtype, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), bias.to(DEV), D0,
                                 rows.to(DEV), N, K, E, EPI_STORE, KN)
    assert torch.equal(D0, D[:R])


@pytest.mark.parametrize("pair", ["0", "1"])
@pytest.mark.parametrize("E,avg,K,N", [(2, 100, 256, 512), (8, 60, 4096, 2048), (3, 200, 512, 28672 // 8)])
def test_fp8_fused_silu_quant_epilogue(ops, E, avg, K, N, pair, monkeypatch):
    monkeypatch.setenv("B200MOE_PAIR", pair)
    monkeypatch.setenv("B200MOE_TILE_N", "256")
    # GEMM1 of the block-FP8 layer: SiLU*mul and the per-token-group-128
    # re-quantisation happen in the epilogue; output is e4m3 [R, N/2] + f32 scales.
    rows = ragged_rows(E, avg, K + 1)
    R = int(rows.sum())
    g = torch.Generator().manual_seed(N)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    Aq, As = O.per_token_group_fp8_quant(x, 128)
    Bq, Bs = zip(*[O.quant_fp8_block_weight(torch.randn(K, N, generator=g) / K ** 0.5) for _ in range(E)])
    Bq, Bs = torch.stack(Bq), torch.stack(Bs)
    h = O.grouped_gemm("fp8block", O.dequant_fp8_group_act(Aq, As), Bq, Bs, None, rows, torch.float32)
    act = O.silu_mul_fp32(h)
    I = N // 2
    gact = act.view(R, I // 128, 128)
    rs = torch.maximum(gact.abs().amax(-1) / 448.0, torch.tensor(O.FP8_MIN_SCALE))
    Dq = torch.zeros(R, I, dtype=torch.float8_e4m3fn, device=DEV)
    Ds = torch.zeros(R, I // 128, dtype=torch.float32, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), None, Dq, rows.to(DEV),
                                 N, K, E, EPI_SILU, KN, 1.702, 7.0, Ds)
    assert torch.allclose(Ds.cpu(), rs, rtol=1e-3, atol=1e-9)
    deq = Dq.cpu().float().view(R, -1, 128) * Ds.cpu().unsqueeze(-1)
    # within one e4m3 step of the exact activation (half a step of rounding + accumulation order)
    assert ((deq - gact).abs() <= 0.07 * gact.abs() + 2e-3 * rs.unsqueeze(-1) + 1e-6).all()


@pytest.mark.parametrize("epi", [EPI_STORE, EPI_SILU])
@pytest.mark.parametrize("E,max_rows,K,N", [(4, 5, 256, 512), (16, 70, 512, 1024), (64, 33, 1024, 256),
                                            (3, 1, 7168, 512)])
def test_fp8_decode_kernel(ops, epi, E, max_rows, K, N):
    """Few rows per expert: weights on the M side of the MMA, 32 tokens per tile,
    activation scales K-block-major ([K/128, R])."""
    g = torch.Generator().manual_seed(E * 7 + K)
    rows = torch.randint(0, max_rows + 1, (E,), generator=g).to(torch.int32)
    rows[0] = max_rows
    R = int(rows.sum())
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    Aq, As = O.per_token_group_fp8_quant(x, 128)
    Bq, Bs = zip(*[O.quant_fp8_block_weight(torch.randn(K, N, generator=g) / K ** 0.5) for _ in range(E)])
    Bq, Bs = torch.stack(Bq), torch.stack(Bs) * (1.0 + 0.25 * torch.rand(E, K // 128, N // 128, generator=g))
    bias = (torch.randn(E, N, generator=g) * 0.1).to(torch.bfloat16)
    ref = O.grouped_gemm("fp8block", O.dequant_fp8_group_act(Aq, As), Bq, Bs, bias, rows, torch.float32)
    if epi == EPI_SILU:
        ref = O.silu_mul_fp32(ref)
    D = torch.full((R + 3, ref.shape[1]), 9.0, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.t().contiguous().to(DEV), Bq.to(DEV), Bs.to(DEV), bias.to(DEV),
                                 D, rows.to(DEV), N, K, E, epi, KN, 1.702, 7.0, None, None, 1)
    close(D[:R], ref)
    assert (D[R:] == 9.0).all()


@pytest.mark.parametrize("E,max_rows,K,N", [(4, 5, 256, 512), (16, 70, 512, 1024), (3, 1, 7168, 512)])
def test_fp8_decode_kernel_row_major_scales_and_quantised_output(ops, E, max_rows, K, N):
    """The decode-regime kernel fed like the default one (row-major activation scales) and
    writing what the default w13 kernel writes: e4m3 [R, N/2] + one f32 scale per token per
    128 columns."""
    g = torch.Generator().manual_seed(E * 11 + K)
    rows = torch.randint(0, max_rows + 1, (E,), generator=g).to(torch.int32)
    rows[0] = max_rows
    R = int(rows.sum())
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    Aq, As = O.per_token_group_fp8_quant(x, 128)
    Bq, Bs = zip(*[O.quant_fp8_block_weight(torch.randn(K, N, generator=g) / K ** 0.5) for _ in range(E)])
    Bq, Bs = torch.stack(Bq), torch.stack(Bs) * (1.0 + 0.25 * torch.rand(E, K // 128, N // 128, generator=g))
    h = O.grouped_gemm("fp8block", O.dequant_fp8_group_act(Aq, As), Bq, Bs, None, rows, torch.float32)
    # 16-bit output with row-major scales
    D = torch.full((R + 2, N), 9.0, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), None, D, rows.to(DEV), N, K, E,
                                 EPI_STORE, KN, 1.702, 7.0, None, None, 2)
    close(D[:R], h)
    assert (D[R:] == 9.0).all()
    # quantised gated output
    act = O.silu_mul_fp32(h)
    I = N // 2
    gact = act.view(R, I // 128, 128)
    rs = torch.maximum(gact.abs().amax(-1) / 448.0, torch.tensor(O.FP8_MIN_SCALE))
    Dq = torch.zeros(R, I, dtype=torch.float8_e4m3fn, device=DEV)
    Ds = torch.zeros(R, I // 128, dtype=torch.float32, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), None, Dq, rows.to(DEV), N, K, E,
                                 EPI_SILU, KN, 1.702, 7.0, Ds, None, 2)
    assert torch.allclose(Ds.cpu(), rs, rtol=1e-3, atol=1e-9)
    deq = Dq.cpu().float().view(R, -1, 128) * Ds.cpu().unsqueeze(-1)
    assert ((deq - gact).abs() <= 0.07 * gact.abs() + 2e-3 * rs.unsqueeze(-1) + 1e-6).all()


def test_fp8_weights_with_16bit_activations(ops):
    # what the reference kernel does natively: weights expanded, activations untouched
    E, K, N = 3, 256, 384
    rows = torch.tensor([70, 0, 33], dtype=torch.int32)
    g = torch.Generator().manual_seed(2)
    A = torch.randn(103, K, generator=g).to(torch.bfloat16)
    Bq, Bs = zip(*[O.quant_fp8_block_weight(torch.randn(K, N, generator=g) / 16) for _ in range(E)])
    Bq, Bs = torch.stack(Bq), torch.stack(Bs)
    ref = O.grouped_gemm("fp8block", A, Bq, Bs, None, rows, torch.float32)
    D = torch.zeros(103, N, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.cutlass_grouped_gemm_interface(A.to(DEV), None, Bq.to(DEV), Bs.to(DEV), None, D,
                                              rows.to(DEV), N, K, E)
    close(D, ref)


def test_mxfp4_weights(ops):
    E, K, N = 4, 320, 256
    rows = torch.tensor([50, 7, 0, 131], dtype=torch.int32)
    g = torch.Generator().manual_seed(4)
    A = torch.randn(188, K, generator=g).to(torch.bfloat16)
    q, s = zip(*[O.quant_mxfp4_weight(torch.randn(N, K, generator=g) / 16) for _ in range(E)])
    q, s = torch.stack(q), torch.stack(s)
    bias = (torch.randn(E, N, generator=g) * 0.02).to(torch.bfloat16)
    ref = O.grouped_gemm("mxfp4", A, q, s, bias, rows, torch.float32)
    D = torch.zeros(188, N, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.cutlass_grouped_gemm_interface(A.to(DEV), None, q.to(DEV).view(torch.float4_e2m1fn_x2),
                                              s.to(DEV), bias.to(DEV), D, rows.to(DEV), N, K, E)
    close(D, ref)
    # the one-time expansion is exact
    w16 = ops._xpu_C.b200_dequant_weights(q.to(DEV), s.to(DEV))
    assert torch.equal(w16.cpu().float(), torch.stack([O.dequant_mxfp4(q[e], s[e]) for e in range(E)]))


def test_c_abi_direct_call():
    """Through ctypes with raw pointers: what a non-torch host would do."""
    from vllm_xpu_kernels import capi
    lib = capi.lib()
    E, K, N = 2, 128, 256
    rows = torch.tensor([100, 60], dtype=torch.int32, device=DEV)
    A = torch.randn(160, K, device=DEV).to(torch.bfloat16)
    B = (torch.randn(E, K, N, device=DEV) / 11).to(torch.bfloat16)
    D = torch.zeros(160, N, dtype=torch.bfloat16, device=DEV)
    a = capi.GemmArgs(recipe=capi.RECIPE_BF16, epilogue=capi.EPI_STORE, a_dtype=capi.BF16,
                      d_dtype=capi.BF16, A=A.data_ptr(), B=B.data_ptr(), b_layout=capi.B_LAYOUT_KN,
                      D=D.data_ptr(), rows_per_expert=rows.data_ptr(), R=160, N=N, K=K, E=E)
    assert lib.b200moe_grouped_gemm_workspace_bytes(ctypes.byref(a)) == 0
    st = torch.cuda.current_stream().cuda_stream
    assert lib.b200moe_grouped_gemm(ctypes.byref(a), None, 0, st) == capi.OK
    torch.cuda.synchronize()
    ref = O.grouped_gemm("bf16", A.cpu(), B.cpu(), None, None, rows.cpu(), torch.float32)
    close(D, ref)
    a.N = 7
    assert lib.b200moe_grouped_gemm(ctypes.byref(a), None, 0, st) == capi.INVALID_ARG


@pytest.mark.parametrize("recipe", ["bf16", "fp8block"])
def test_large_against_cuda_core_check(ops, recipe):
    """Mixtral-sized K and a slice of N: too big for the CPU oracle, so the
    tensor-core result is compared with one-thread-per-element CUDA arithmetic."""
    E, K, N, R = 8, 4096, 2048, 8192
    g = torch.Generator().manual_seed(0)
    rows = torch.tensor([1000, 1100, 900, 1024, 1050, 998, 1120, 1000], dtype=torch.int32, device=DEV)
    x = torch.randn(R, K, generator=g).to(torch.bfloat16)
    D = torch.zeros(R, N, dtype=torch.bfloat16, device=DEV)
    ref = torch.zeros(R, N, dtype=torch.float32, device=DEV)
    if recipe == "bf16":
        B = (torch.randn(E, K, N, generator=g) / 64).to(torch.bfloat16).to(DEV)
        ops._xpu_C.b200_grouped_gemm(x.to(DEV), None, B, None, None, D, rows, N, K, E, EPI_STORE, KN)
        ops._xpu_C.b200_grouped_gemm_check(x.to(DEV), None, B, None, None, ref, rows, N, K, E, KN)
    else:
        Aq, As = O.per_token_group_fp8_quant(x, 128)
        Bq = (torch.randn(E, K, N, generator=g) * 100).clamp(-448, 448).to(torch.float8_e4m3fn).to(DEV)
        Bs = (torch.rand(E, K // 128, N // 128, generator=g) * 2e-4 + 1e-4).to(DEV)
        ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq, Bs, None, D, rows, N, K, E, EPI_STORE, KN)
        ops._xpu_C.b200_grouped_gemm_check(Aq.to(DEV), As.to(DEV), Bq, Bs, None, ref, rows, N, K, E, KN)
    close(D, ref)


# ---- block-FP8 with power-of-two scales: scales applied by the tensor core -------------------
def _pow2_case(E, rows, K, N, seed):
    R = sum(rows)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(R + 3, K, generator=g) * torch.exp2(torch.randint(-3, 4, (R + 3, 1), generator=g).float())
    Aq, As = O.per_token_group_fp8_quant(x.to(torch.bfloat16), 128, scale_ue8m0=True)
    Bq, Bs = [], []
    for _ in range(E):
        w = torch.randn(K, N, generator=g) / K ** 0.5
        w = w * torch.exp2(torch.randint(-2, 3, (K // 128, N // 128), generator=g).float()
                           ).repeat_interleave(128, 0).repeat_interleave(128, 1)
        blk = w.view(K // 128, 128, N // 128, 128)
        sc = torch.exp2(torch.ceil(torch.log2((blk.abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-12))))
        q = (blk / sc.view(K // 128, 1, N // 128, 1)).clamp(-448, 448).reshape(K, N).to(torch.float8_e4m3fn)
        Bq.append(q)
        Bs.append(sc)
    return Aq, As, torch.stack(Bq), torch.stack(Bs), torch.tensor(rows, dtype=torch.int32), R


@pytest.mark.parametrize("E,rows,K,N", [
    (1, [128], 128, 256),                          # one tile, one stage
    (1, [100], 512, 512),                          # the four stages of the ring once
    (2, [140, 90], 640, 256),                      # five K blocks: a second scale group with one block in it
    (2, [64, 200], 896, 512),                      # seven: the ring wraps inside the second group
    (3, [130, 0, 257], 1024, 768),                 # ring wraps; three column tiles
    (2, [77, 300], 2048, 7168),                    # second GEMM of the DeepSeek-V3 layer
    (6, [500, 513, 1, 640, 390, 128], 1536, 1280), # 100 tiles... several per CTA
])
def test_fp8_pow2_scales_store(ops, E, rows, K, N):
    Aq, As, Bq, Bs, rpe, R = _pow2_case(E, rows, K, N, K + N)
    ref = O.grouped_gemm("fp8block", O.dequant_fp8_group_act(Aq, As)[:R], Bq, Bs, None, rpe, torch.float32)
    D = torch.full((R + 3, N), 3.0, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), None, D, rpe.to(DEV),
                                 N, K, E, EPI_STORE, KN, 1.702, 7.0, None, None, 0, 0, 0.0, 0.0, 0.0, True)
    close(D[:R], ref)
    assert (D[R:] == 3.0).all()
    # the same problem through the promotion kernel agrees (same contract, other arithmetic order)
    D2 = torch.empty(R + 3, N, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), None, D2, rpe.to(DEV),
                                 N, K, E, EPI_STORE, KN)
    close(D2[:R], ref)


@pytest.mark.parametrize("E,rows,K,N", [(2, [100, 60], 256, 512), (3, [200, 129, 300], 7168, 1024)])
def test_fp8_pow2_scales_fused_silu_quant(ops, E, rows, K, N):
    """First GEMM of the layer on the tensor-core-scaled kernel: SiLU*mul and the group-128
    quantisation in the epilogue, with power-of-two output scales."""
    Aq, As, Bq, Bs, rpe, R = _pow2_case(E, rows, K, N, 7)
    h = O.grouped_gemm("fp8block", O.dequant_fp8_group_act(Aq, As)[:R], Bq, Bs, None, rpe, torch.float32)
    gact = O.silu_mul_fp32(h)
    Dq = torch.zeros(R + 3, N // 2, dtype=torch.float8_e4m3fn, device=DEV)
    Ds = torch.zeros(R + 3, N // 2 // 128, dtype=torch.float32, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), None, Dq, rpe.to(DEV),
                                 N, K, E, EPI_SILU, KN, 1.702, 7.0, Ds, None, 0, 0, 0.0, 0.0, 0.0, True)
    ds = Ds.cpu()[:R]
    assert torch.equal(torch.exp2(torch.log2(ds).round()), ds)          # exact powers of two
    _, rs = O.per_token_group_fp8_quant(gact, 128, scale_ue8m0=True)
    amax = gact.view(R, -1, 128).abs().amax(-1)
    frac = torch.log2(amax.clamp_min(1e-10) / 448)
    clear = (frac - frac.round()).abs() > 1e-3                           # not within rounding of a power of two
    assert torch.equal(ds[clear], rs[clear])
    deq = Dq.cpu()[:R].float().view(R, -1, 128) * ds.unsqueeze(-1)
    assert ((deq.view(R, -1) - gact).abs() <= 0.07 * gact.abs() + 2e-3 * ds.repeat_interleave(128, 1) * 448 / 16 + 1e-6).all()


def test_fp8_pow2_scales_refuse_other_scales(ops):
    """A scale that is not a power of two cannot go through the tensor core's scaling: the kernel
    says so in the device status word instead of applying it wrongly in silence."""
    Aq, As, Bq, Bs, rpe, R = _pow2_case(1, [64], 256, 256, 3)
    As = As.clone()
    As[5, 1] *= 1.5
    D = torch.empty(R + 3, 256, dtype=torch.bfloat16, device=DEV)
    ops._xpu_C.b200_grouped_gemm(Aq.to(DEV), As.to(DEV), Bq.to(DEV), Bs.to(DEV), None, D, rpe.to(DEV),
                                 256, 256, 1, EPI_STORE, KN, 1.702, 7.0, None, None, 0, 0, 0.0, 0.0, 0.0, True)
    assert ops._xpu_C.b200_device_status() == -1      # B200MOE_INVALID_ARG, and the word is cleared
    assert ops._xpu_C.b200_device_status() == 0
