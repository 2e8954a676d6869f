"""Block-scaled (MX) grouped GEMM: MXFP8 activations x MXFP4 weights on the tensor
cores against the CPU oracle (dequantise both operands, then fp32 matmul per
expert; tests/fused_moe/test_grouped_gemm.py of the reference does the same for its
MXFP4 recipe).  The oracle is fed the same quantised A, so the tolerance (2e-2
absolute + relative, the stated layer bound) covers the contraction only."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
EPI_STORE, EPI_OAI = 0, 2


def close(out, ref, tol=2e-2):
    out, ref = out.float().cpu(), ref.float().cpu()
    err = (out - ref).abs()
    bound = tol + tol * ref.abs()
    assert (err <= bound).all(), (
        f"max err {err.max().item():.4g} at {torch.nonzero(err > bound)[:5].tolist()} "
        f"({int((err > bound).sum())} of {err.numel()} outside {tol})")


def make_case(E, rows, K, N, seed, spread_scales=True):
    g = torch.Generator().manual_seed(seed)
    R = int(sum(rows))
    x = torch.randn(R, K, generator=g)
    if spread_scales:  # rows and column groups of different magnitude: a mis-indexed scale shows
        x = x * torch.exp2(torch.randint(-3, 4, (R, K // 32), generator=g).float()).repeat_interleave(32, 1)
    Aq, Asf = O.quant_mxfp8_act(x.to(torch.bfloat16))
    Bq, Bs = [], []
    for _ in range(E):
        w = torch.randn(N, K, generator=g) / K ** 0.5
        if spread_scales:
            w = w * torch.exp2(torch.randint(-2, 3, (N, K // 32), generator=g).float()).repeat_interleave(32, 1)
        q, s = O.quant_mxfp4_weight(w)
        Bq.append(q)
        Bs.append(s)
    return Aq, Asf, torch.stack(Bq), torch.stack(Bs), torch.tensor(rows, dtype=torch.int32)


def padded_sf(sf, K):
    pitch = (K + 511) // 512 * 16
    out = torch.full((sf.shape[0], pitch), 0xFF, dtype=torch.uint8)   # padding must never be read as a scale
    out[:, :K // 32] = sf
    return out


def run_mx(ops, Aq, Asf, Bq, Bs, rows, N, K, epi, bias=None, quant_out=False):
    E, R = Bq.shape[0], Aq.shape[0]
    bsf = ops._xpu_C.b200_mx_prepare_weight_scales(Bs.to(DEV), K)
    b = None if bias is None else bias.to(DEV)
    cols = N if epi == EPI_STORE else N // 2
    if quant_out:
        D = torch.zeros(R, cols, dtype=torch.float8_e4m3fn, device=DEV)
        Dsf = torch.full((R, (cols + 511) // 512 * 16), 0xFF, dtype=torch.uint8, device=DEV)
    else:
        D = torch.full((R, cols), 7.0, dtype=torch.bfloat16, device=DEV)
        Dsf = None
    ops._xpu_C.b200_grouped_gemm_mx(Aq.to(DEV), padded_sf(Asf, K).to(DEV), Bq.to(DEV), bsf, b, D, Dsf,
                                    rows.to(DEV), N, K, E, epi, 1.702, 7.0)
    return D, Dsf


@pytest.mark.parametrize("E,rows,K,N", [
    (1, [128], 128, 192),                       # one tile, one stage
    (1, [128], 512, 384),                       # the odd 192-column tile starts inside a scale piece
    (1, [300], 256, 576),
    (1, [77], 192, 200),                        # K tail of 64, ragged N
    (5, [100, 300, 0, 129, 171], 384, 384),
    (3, [1, 0, 260], 2880, 2880),               # the gpt-oss widths: K = 22.5 stages
    (8, [40, 0, 13, 128, 129, 255, 256, 257], 1024, 640),
    (1, [128], 576, 192),                       # K tail in the last slot of the five-stage ring
    (1, [128], 704, 192),                       # K tail in the first slot of the next round
    (3, [700, 900, 704], 704, 1728),            # 171 tiles on 148 CTAs: two tiles per CTA, K tail
    (2, [1100, 1204], 2880, 1728),              # the same with the gpt-oss K
])
def test_mxfp4_native_store(ops, E, rows, K, N):
    Aq, Asf, Bq, Bs, rpe = make_case(E, rows, K, N, seed=K + N)
    g = torch.Generator().manual_seed(1)
    bias = (torch.randn(E, N, generator=g) * 0.1).to(torch.bfloat16)
    ref = O.grouped_gemm("mxfp4", O.dequant_mxfp8_act(Aq, Asf), Bq, Bs, bias, rpe, torch.float32)
    D, _ = run_mx(ops, Aq, Asf, Bq, Bs, rpe, N, K, EPI_STORE, bias)
    close(D, ref)


def test_mxfp4_native_rows_beyond_the_experts_are_untouched(ops):
    E, K, N = 2, 256, 384
    Aq, Asf, Bq, Bs, rpe = make_case(E, [60, 90], K, N, seed=3)
    pad = torch.zeros(50, K, dtype=torch.float8_e4m3fn)
    Aq2 = torch.cat([Aq.view(torch.uint8), pad.view(torch.uint8)]).view(torch.float8_e4m3fn)
    Asf2 = torch.cat([Asf, torch.full((50, K // 32), 0xFF, dtype=torch.uint8)])  # NaN scales in unused rows
    D, _ = run_mx(ops, Aq2, Asf2, Bq, Bs, rpe, N, K, EPI_STORE)
    assert (D[150:] == 7.0).all()
    ref = O.grouped_gemm("mxfp4", O.dequant_mxfp8_act(Aq, Asf), Bq, Bs, None, rpe, torch.float32)
    close(D[:150], ref)


@pytest.mark.parametrize("E,rows,K,N", [(3, [200, 150, 250], 512, 1152), (2, [129, 64], 2880, 5760)])
def test_mxfp4_native_swigluoai_epilogue(ops, E, rows, K, N):
    Aq, Asf, Bq, Bs, rpe = make_case(E, rows, K, N, seed=11, spread_scales=False)
    g = torch.Generator().manual_seed(2)
    bias = (torch.randn(E, N, generator=g) * 0.1).to(torch.bfloat16)
    h = O.grouped_gemm("mxfp4", O.dequant_mxfp8_act(Aq, Asf), Bq, Bs, bias, rpe, torch.float32)
    act = O.swigluoai_and_mul(h)
    D, _ = run_mx(ops, Aq, Asf, Bq, Bs, rpe, N, K, EPI_OAI, bias)
    close(D, act)
    # the same epilogue leaving MXFP8: codes and scale bytes against the oracle's quantiser run
    # on the kernel's own bf16-free fp32 activation is not available on the CPU, so compare the
    # dequantised result with the fp32 activation at e4m3 resolution (half an ulp = 1/16 of the
    # group maximum at worst) and the scale bytes with the oracle's where the group maximum is
    # not within rounding of a power of two
    Dq, Dsf = run_mx(ops, Aq, Asf, Bq, Bs, rpe, N, K, EPI_OAI, bias, quant_out=True)
    deq = O.dequant_mxfp8_act(Dq.cpu(), Dsf.cpu())
    gmax = act.view(act.shape[0], -1, 32).abs().amax(-1)
    err = (deq - act).abs().view(act.shape[0], -1, 32).amax(-1)
    assert (err <= gmax / 16 + 1e-6).all()
    _, ref_sf = O.quant_mxfp8_act(act)
    frac = torch.log2(gmax.clamp_min(1e-10) / 448)
    clear = (frac - frac.round()).abs() > 1e-3
    assert torch.equal(Dsf.cpu()[:, :ref_sf.shape[1]][clear], ref_sf[clear])


def test_quant_mxfp8_matches_the_oracle(ops):
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(257, 2880, generator=g) * torch.exp2(torch.randint(-6, 6, (257, 1), generator=g).float()))
    x = x.to(torch.bfloat16)
    q, sf = ops._xpu_C.b200_quant_mxfp8(x.to(DEV))
    rq, rsf = O.quant_mxfp8_act(x)
    assert sf.shape == (257, 96)
    assert torch.equal(sf.cpu()[:, :90], rsf)
    assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))


def test_mx_argument_checks(ops):
    Aq, Asf, Bq, Bs, rpe = make_case(1, [32], 160, 192, seed=1)   # K = 160 is not a multiple of 64
    with pytest.raises(RuntimeError):
        run_mx(ops, Aq, Asf, Bq, Bs, rpe, 192, 160, EPI_STORE)
