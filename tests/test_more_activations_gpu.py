"""The other activations of the layer (gelu, gelu_tanh, swiglustep, situ,
relu2_no_mul) against the reference's own torch oracles (golden vectors) and
the CPU restatement, the gemm1 clamp folded into the activation kernel, and the
layer built with each of them.  Tolerances are the reference's
(tests/test_activation.py:70-73, tests/test_swiglustep_and_mul.py:24-29 there):
atol 1e-3 / rtol 1.6e-2 for bf16, 1e-3 / 1e-3 for f16, 1e-5 / 1.3e-6 for f32."""
import pytest
import torch

from conftest import load_golden
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"bf16": (1e-3, 1.6e-2), "f16": (1e-3, 1e-3), "f32": (1e-5, 1.3e-6)}
DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def _t(g, key, tag):
    a = g[key + "_" + tag]
    return a.view(torch.bfloat16) if tag == "bf16" else a


def _run(ops, name, x):
    gated = name != "relu2"
    out = torch.empty(x.shape[0], x.shape[1] // 2 if gated else x.shape[1], dtype=x.dtype, device=DEV)
    xd = x.to(DEV)
    if name == "gelu":
        ops._C.gelu_and_mul(out, xd)
    elif name == "gelu_tanh":
        ops._C.gelu_tanh_and_mul(out, xd)
    elif name == "relu2":
        ops._C.relu2_no_mul(out, xd)
    elif name == "swiglustep":
        ops._C.swiglustep_and_mul(out, xd, 7.0)
    elif name == "situ_raw":
        ops._C.situ_and_mul(out, xd, 1.7, -1.0)
    elif name == "situ_lin":
        ops._C.situ_and_mul(out, xd, 1.7, 2.0)
    return out.cpu()


@pytest.mark.parametrize("tag", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("name", ["gelu", "gelu_tanh", "relu2", "swiglustep", "situ_raw", "situ_lin"])
def test_against_reference_oracles(ops, name, tag):
    g = load_golden("act_more")
    x = _t(g, "x", tag)
    ref = _t(g, name, tag)
    out = _run(ops, name, x)
    atol, rtol = TOL[tag]
    if name == "relu2":
        assert torch.equal(out, ref)
    else:
        torch.testing.assert_close(out, ref, atol=atol, rtol=rtol)
    if name in ("gelu", "gelu_tanh") and tag != "f32":
        # Same two roundings as the reference, so most elements are bit-identical.  The rest
        # sit where 1 + erf(x/sqrt2) cancels (x < -3): there one ulp between the CPU's and the
        # GPU's erf is percents of the result.
        assert (out == ref).float().mean() > 0.9


@pytest.mark.parametrize("d", [8, 100, 1800, 13824])
@pytest.mark.parametrize("name", ["gelu", "swiglustep", "situ_lin", "relu2"])
def test_ragged_widths_against_restatement(ops, name, d):
    g = torch.Generator().manual_seed(d)
    x = (torch.randn(7, 2 * d, generator=g) * 4).to(torch.bfloat16)
    ref = {"gelu": lambda: O.gelu_and_mul(x), "swiglustep": lambda: O.swiglustep_and_mul(x),
           "situ_lin": lambda: O.situ_and_mul(x, 1.7, 2.0), "relu2": lambda: O.relu2_no_mul(x)}[name]()
    torch.testing.assert_close(_run(ops, name, x), ref, atol=1e-3, rtol=1.6e-2)


def test_empty_and_leading_dims(ops):
    out = torch.empty(0, 8, dtype=torch.bfloat16, device=DEV)
    ops._C.gelu_and_mul(out, torch.empty(0, 16, dtype=torch.bfloat16, device=DEV))
    x = torch.randn(3, 5, 64, device=DEV, dtype=torch.float16)
    out = torch.empty(3, 5, 32, device=DEV, dtype=torch.float16)
    ops._C.swiglustep_and_mul(out, x, 7.0)
    torch.testing.assert_close(out.cpu(), O.swiglustep_and_mul(x.cpu()), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("case,error", [
    ("odd_width", "last dimension must be positive and even"),
    ("noncontiguous_input", "input must be contiguous"),
    ("noncontiguous_output", "output must be contiguous"),
    ("wrong_output_shape", "output last dimension must be half"),
    ("wrong_output_dtype", "input and output must have the same dtype"),
])
def test_situ_rejects_invalid_tensor_contract(ops, case, error):
    # the cases and texts of tests/test_activation.py:117-148 of the reference
    x = torch.randn(2, 8, device=DEV)
    out = torch.empty(2, 4, device=DEV)
    if case == "odd_width":
        x, out = torch.randn(2, 7, device=DEV), torch.empty(2, 3, device=DEV)
    elif case == "noncontiguous_input":
        x = torch.randn(2, 16, device=DEV)[:, ::2]
    elif case == "noncontiguous_output":
        out = torch.empty(2, 8, device=DEV)[:, ::2]
    elif case == "wrong_output_shape":
        out = torch.empty(2, 3, device=DEV)
    elif case == "wrong_output_dtype":
        out = out.to(torch.bfloat16)
    with pytest.raises(RuntimeError, match=error):
        ops._C.situ_and_mul(out, x, 1.7, 2.0)


@pytest.mark.parametrize("beta", [0.0, -1.0, float("nan"), float("inf")])
def test_situ_rejects_invalid_beta(ops, beta):
    with pytest.raises(RuntimeError, match="finite and greater than zero"):
        ops._C.situ_and_mul(torch.empty(2, 4, device=DEV), torch.randn(2, 8, device=DEV), beta, 2.0)


@pytest.mark.parametrize("linear_beta", [float("nan"), float("inf"), float("-inf")])
def test_situ_rejects_invalid_linear_beta(ops, linear_beta):
    with pytest.raises(RuntimeError, match="linear_beta must be finite"):
        ops._C.situ_and_mul(torch.empty(2, 4, device=DEV), torch.randn(2, 8, device=DEV), 1.7, linear_beta)


@pytest.mark.parametrize("act,code", [("silu", 0), ("gelu", 1), ("swiglustep", 3), ("relu2", 5)])
def test_clamp_folded_into_the_activation(ops, act, code):
    """clamp_limit > 0 gives what clamping the input first (gate <= limit, |up| <= limit,
    halves of the row) and then the plain activation gives."""
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(33, 512, generator=g) * 6).to(torch.bfloat16).to(DEV)
    lim = 5.0
    xc = x.clone()
    xc[:, :256].clamp_(max=lim)
    xc[:, 256:].clamp_(min=-lim, max=lim)
    width = 512 if act == "relu2" else 256
    a = torch.empty(33, width, dtype=torch.bfloat16, device=DEV)
    b = torch.empty_like(a)
    ops._C.b200_act_and_mul(a, x, code, 7.0, 0.0, lim)
    ops._C.b200_act_and_mul(b, xc, code, 7.0, 0.0, 0.0)
    assert torch.equal(a, b)
    assert not torch.equal(x, xc)


def _layer(E, H, I, T, k, seed, w2_rows=None):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, H, generator=g) / 2).to(torch.bfloat16)
    w13 = (torch.randn(E, H, 2 * I, generator=g) / H ** 0.5).to(torch.bfloat16)
    w2 = (torch.randn(E, w2_rows or I, H, generator=g) / (w2_rows or I) ** 0.5).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    tw, ti = O.topk_softmax(logits, k, True)
    return x, w13, w2, tw, ti.to(torch.int32)


@pytest.mark.parametrize("activation", ["silu", "gelu", "gelu_tanh", "swiglustep", "situ", "relu2_no_mul"])
@pytest.mark.parametrize("clamp", [None, 1.0])
@pytest.mark.parametrize("fused", [True, False])
def test_layer_with_each_activation(ops, activation, clamp, fused, monkeypatch):
    """Every gated activation (and the layer's clamp) both ways: evaluated in the first GEMM's
    epilogue, and as the stand-alone kernel between the two GEMMs (relu2_no_mul is not gated
    and always takes the second way)."""
    from vllm_xpu_kernels.fused_moe_interface import XpuFusedMoe
    if not fused:
        monkeypatch.setenv("B200MOE_UNFUSED_ACT", "1")
    E, H, I, T, k = 4, 256, 384, 40, 2
    x, w13, w2, tw, ti = _layer(E, H, I, T, k, 11, w2_rows=2 * I if activation == "relu2_no_mul" else None)
    kw = dict(activation_situ_beta=4.0, activation_situ_linear_beta=25.0) if activation == "situ" else {}
    moe = XpuFusedMoe(w13.to(DEV), None, None, w2.to(DEV), None, None, k, activation, E,
                      gemm1_clamp_limit=clamp, **kw)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    moe.apply(out, x.to(DEV), tw.to(DEV), ti.to(DEV))
    ref = O.fused_moe("bf16", x, w13, None, None, w2, None, None, tw, ti, activation,
                      gemm1_clamp_limit=clamp, out_dtype=torch.float32,
                      situ_beta=4.0, situ_linear_beta=25.0)
    err = (out.float().cpu() - ref).abs()
    assert (err <= 2e-2 + 2e-2 * ref.abs()).all(), f"max err {err.max():.4g}"


def test_situ_needs_beta():
    from vllm_xpu_kernels.fused_moe_interface import XpuFusedMoe
    w13 = torch.zeros(2, 128, 256, dtype=torch.bfloat16, device=DEV)
    w2 = torch.zeros(2, 128, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError, match="SITU requires activation_situ_beta"):
        XpuFusedMoe(w13, None, None, w2, None, None, 2, "situ", 2)
    with pytest.raises(ValueError, match="must be positive"):
        XpuFusedMoe(w13, None, None, w2, None, None, 2, "situ", 2, activation_situ_beta=-1.0)
    with pytest.raises(ValueError, match="Unsupported FusedMoe activation"):
        XpuFusedMoe(w13, None, None, w2, None, None, 2, "tanh", 2)


@pytest.mark.parametrize("activation,clamp", [("silu", 0.5), ("gelu", None), ("relu2_no_mul", None),
                                              ("swiglustep", 2.0), ("situ", None), ("gelu_tanh", 1.0)])
@pytest.mark.parametrize("fused", [True, False])
def test_block_fp8_layer_with_each_activation(ops, activation, clamp, fused, monkeypatch):
    """Block-FP8 layer: activation (+ clamp) and the group-128 quantisation of its result in the
    first GEMM's epilogue, or as separate kernels on the bf16 output of that GEMM."""
    from vllm_xpu_kernels.fused_moe_interface import XpuFusedMoe
    if not fused:
        monkeypatch.setenv("B200MOE_UNFUSED_ACT", "1")
    kw = dict(activation_situ_beta=4.0, activation_situ_linear_beta=25.0) if activation == "situ" else {}
    E, H, I, T, k = 4, 256, 256, 48, 2
    g = torch.Generator().manual_seed(5)
    K2 = 2 * I if activation == "relu2_no_mul" else I
    x = (torch.randn(T, H, generator=g)).to(torch.bfloat16)
    q13, s13 = zip(*[O.quant_fp8_block_weight(torch.randn(H, 2 * I, generator=g) / H ** 0.5) for _ in range(E)])
    q2, s2 = zip(*[O.quant_fp8_block_weight(torch.randn(K2, H, generator=g) / K2 ** 0.5) for _ in range(E)])
    q13, s13, q2, s2 = (torch.stack(t) for t in (q13, s13, q2, s2))
    tw, ti = O.topk_softmax(torch.randn(T, E, generator=g), k, True)
    ti = ti.to(torch.int32)
    moe = XpuFusedMoe(q13.to(DEV), s13.to(DEV), None, q2.to(DEV), s2.to(DEV), None, k, activation, E,
                      gemm1_clamp_limit=clamp, **kw)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    moe.apply(out, x.to(DEV), tw.to(DEV), ti.to(DEV))
    ref = O.fused_moe("fp8block", x, q13, s13, None, q2, s2, None, tw, ti, activation,
                      gemm1_clamp_limit=clamp, out_dtype=torch.float32,
                      situ_beta=4.0, situ_linear_beta=25.0)
    err = (out.float().cpu() - ref).abs()
    # Unfused, the layer rounds the activation to bf16 before quantising it (as the reference
    # does), the oracle keeps fp32: an e4m3 code flips now and then, and a flipped code of a
    # squared value is worth more, hence the wider element bound for relu2.  Fused, the
    # activation is quantised from fp32 like the oracle's.
    tol = 0.15 if activation == "relu2_no_mul" else (2e-2 if fused else 5e-2)
    assert (err <= tol + tol * ref.abs()).all(), f"max err {err.max():.4g}"
    assert err.mean() < 2e-2 * ref.abs().mean()
