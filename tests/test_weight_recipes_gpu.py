"""The 16-bit-activation weight recipes (per-tensor FP8 in e4m3 and e5m2,
MXFP8, INT4): the one-time widening against the dequantisation rules of the
reference (vllm_xpu_kernels/moe_utils.py:206-217 and
tests/fused_moe/test_fused_moe.py:37-50 there), and the layer built from each
against the layer oracle within the 2e-2 bf16 bound."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make(recipe, E, K, N, g, fp8=torch.float8_e4m3fn):
    """Quantised [.., K, N]-contract weights of one GEMM: (w, scale) in the API layout."""
    ws, ss = [], []
    for _ in range(E):
        w = torch.randn(K, N, generator=g) / K ** 0.5
        if recipe == "fp8":
            s = torch.tensor(2.0 ** float(torch.randint(-3, 4, (1,), generator=g)) * 1.25)
            ws.append((w / s).to(fp8)); ss.append(s)
        elif recipe == "mxfp8":
            q, s = O.quant_mxfp8_weight(w); ws.append(q); ss.append(s)
        else:
            q, s = O.quant_int4_weight(w.t().contiguous()); ws.append(q); ss.append(s)
    return torch.stack(ws), torch.stack(ss)


@pytest.mark.parametrize("recipe,fp8", [("fp8", torch.float8_e4m3fn), ("fp8", torch.float8_e5m2),
                                        ("mxfp8", torch.float8_e4m3fn), ("int4", None)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_widening_matches_the_dequantisation_rule(ops, recipe, fp8, out_dtype):
    g = torch.Generator().manual_seed(2)
    E, K, N = 3, 256, 384
    w, s = make(recipe, E, K, N, g, fp8)
    out = ops._xpu_C.b200_expand_weights(w.to(DEV), s.to(DEV), recipe, out_dtype).cpu()
    ref = torch.stack([O.dequant_expert_weight(recipe, w[e], s[e]) for e in range(E)])  # [E, K, N]
    if recipe == "int4":
        ref = ref.transpose(1, 2)
    assert out.dtype == out_dtype and out.shape == ref.shape
    assert torch.equal(out, ref.to(out_dtype))


@pytest.mark.parametrize("recipe,fp8", [("fp8", torch.float8_e4m3fn), ("fp8", torch.float8_e5m2),
                                        ("mxfp8", torch.float8_e4m3fn), ("int4", None)])
@pytest.mark.parametrize("has_bias", [False, True])
def test_layer(ops, recipe, fp8, has_bias):
    from vllm_xpu_kernels.fused_moe_interface import XpuFusedMoe
    E, H, I, T, k = 4, 256, 384, 40, 2
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(T, H, generator=g) / 2).to(torch.bfloat16)
    w13, s13 = make(recipe, E, H, 2 * I, g, fp8)
    w2, s2 = make(recipe, E, I, H, g, fp8)
    b13 = (torch.randn(E, 2 * I, generator=g) / 16).to(torch.bfloat16) if has_bias else None
    b2 = (torch.randn(E, H, generator=g) / 16).to(torch.bfloat16) if has_bias else None
    tw, ti = O.topk_softmax(torch.randn(T, E, generator=g), k, True)
    ti = ti.to(torch.int32)
    dev = lambda t: None if t is None else t.to(DEV)
    moe = XpuFusedMoe(dev(w13), dev(s13), dev(b13), dev(w2), dev(s2), dev(b2), k, "silu", E)
    assert moe.recipe == recipe and moe.inter_size == I
    out = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    moe.apply(out, dev(x), dev(tw), dev(ti))
    ref = O.fused_moe(recipe, x, w13, s13, b13, w2, s2, b2, tw, ti, "silu", quant_act=False,
                      out_dtype=torch.float32)
    err = (out.float().cpu() - ref).abs()
    assert (err <= 2e-2 + 2e-2 * ref.abs()).all(), f"max err {err.max():.4g}"
