"""Checks at the benchmark's full sizes, where the CPU oracle cannot evaluate the whole
layer: properties that do not depend on size (permutation validity, conservation of rows,
idempotence of the stable order) plus the oracle on a sample of tokens."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_c3_routing_and_permutation_full_size(ops):
    T, E, k, H = 16384, 256, 8, 7168
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(T, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.01
    w, ids = ops._moe_C.grouped_topk(logits.to(DEV), 8, 4, 8, True, 2.5, bias.to(DEV), 1)
    rw, rids = O.grouped_topk(logits, k, True, 8, 4, "sigmoid", 2.5, bias)
    if not torch.equal(ids.cpu(), rids):
        # diagnosis only: a differing row is excusable when the oracle's own selection margin on
        # it is a few fp32 ulps (two correct evaluations of the sigmoid may then disagree)
        bad = (ids.cpu() != rids).any(dim=1)
        keys = torch.sigmoid(logits) + bias
        margin = O.routing_margin(keys[bad], k)
        raise AssertionError(f"{int(bad.sum())} of {T} rows differ from the oracle; their selection "
                             f"margins: {margin[:8].tolist()}")
    # align: a permutation of the flat indices plus padding, blocks labelled by their expert
    n, nb = O.align_sizes(T * k, E, 128)
    s = torch.empty(n, dtype=torch.int32, device=DEV)
    e = torch.empty(nb, dtype=torch.int32, device=DEV)
    t = torch.empty(1, dtype=torch.int32, device=DEV)
    ops._moe_C.moe_align_block_size(ids, E, 128, s, e, t, None)
    total = int(t.item())
    valid = s[:total]
    real = valid[valid < T * k]
    assert real.numel() == T * k and torch.equal(torch.sort(real).values.cpu(), torch.arange(T * k, dtype=torch.int32))
    flat = ids.flatten()
    owner = e[: total // 128].repeat_interleave(128)
    mask = valid < T * k
    assert torch.equal(flat[valid[mask].long()], owner[mask])            # every index sits in its expert's blocks
    seg = valid.view(-1, 128)
    assert ((seg[:, 1:] > seg[:, :-1]) | (seg[:, 1:] == T * k)).all()   # stable: ascending inside a block
    rs, re, rt = O.moe_align_block_size(ids.cpu(), 128, E)
    assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re) and total == int(rt)
    # remap on fp8 rows with scales: rows_per_expert = histogram, row map = a permutation, rows copied bit-exact
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    xq = torch.empty(T, H, dtype=torch.float8_e4m3fn, device=DEV)
    xs = torch.empty(T, H // 128, dtype=torch.float32, device=DEV)
    ops._C.per_token_group_fp8_quant(x, xq, xs, 128, 1e-10, -448.0, 448.0, False, False, False)
    out = torch.empty(T * k, H, dtype=torch.float8_e4m3fn, device=DEV)
    so = torch.empty(T * k, H // 128, dtype=torch.float32, device=DEV)
    rows = torch.zeros(E, dtype=torch.int32, device=DEV)
    rmap = torch.empty(T, k, dtype=torch.int32, device=DEV)
    ops._moe_C.remap_hidden_states(xq, xs, out, so, None, rows, rmap, ids, E, E)
    assert torch.equal(rows.cpu().long(), torch.bincount(flat.cpu().long(), minlength=E))
    assert torch.equal(torch.sort(rmap.flatten()).values.cpu(), torch.arange(T * k, dtype=torch.int32))
    src = torch.arange(T, device=DEV).repeat_interleave(k)
    assert torch.equal(out.view(torch.uint8)[rmap.flatten().long()], xq.view(torch.uint8)[src])
    assert torch.equal(so[rmap.flatten().long()], xs[src])
    # gather with weights 1/k of the permuted copies gives the row back (fp32 accumulate, one rounding)
    back = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    y = out.to(torch.bfloat16)
    ops._moe_C.moe_gather(back, y, torch.full((T, k), 1.0 / k, device=DEV), rmap, E)
    assert torch.allclose(back.float(), xq.float(), rtol=1e-2, atol=1e-2)


def test_c1_layer_full_size_sampled_tokens(ops):
    """The full Mixtral-shaped layer on the GPU; the oracle on 24 of its 4096 tokens (a token's
    output depends only on that token), plus row conservation over the whole batch."""
    import bench
    from vllm_xpu_kernels.fused_moe_interface import XpuFusedMoe
    from vllm_xpu_kernels.moe_utils import quant_fp8_block_act
    cfg = bench.CONFIGS["c1"]
    dev = torch.device(DEV)
    weights = bench.make_device_layer(cfg, dev)
    x, logits = bench.make_inputs(cfg, cfg["T"], seed=0)
    layer = bench.Layer(cfg, weights, cfg["T"], dev)
    out = layer.step(x.to(dev), logits.to(dev)).float().cpu()
    assert torch.ops._xpu_C.b200_device_status() == 0
    assert torch.isfinite(out).all()
    rw, rids = O.topk_softmax(logits, cfg["k"], True)
    assert torch.equal(layer.ids.cpu(), rids)
    pick = torch.randperm(cfg["T"], generator=torch.Generator().manual_seed(1))[:24]
    cpu_w = {k: (v.cpu() if v is not None else None) for k, v in weights.items()}
    ref = O.fused_moe("fp8block", x[pick], cpu_w["w13"], cpu_w["w13_scale"], None, cpu_w["w2"],
                      cpu_w["w2_scale"], None, rw[pick], rids[pick], "silu", out_dtype=torch.float32)
    err = (out[pick] - ref).abs()
    assert (err <= 2e-2 + 2e-2 * ref.abs()).all(), f"max err {err.max():.4g}"
    assert err.mean() < 1e-2 * ref.abs().mean() + 1e-3
    # the same batch through already-quantised inputs is bit-identical (no hidden state between calls)
    xq, xs = quant_fp8_block_act(x.to(dev))
    out2 = torch.empty_like(layer.out)
    layer.moe.apply(out2, xq, layer.w, layer.ids, a1q_scale=xs)
    assert torch.equal(out2.float().cpu(), out)


# ---- the other configurations at full size ------------------------------------------------
# Same pattern: the whole layer on the GPU, the CPU oracle on a sample of its tokens with only
# the experts those tokens hit rebuilt and dequantised (bench.parity_check), bound 2e-2
# absolute + relative against the quantise-dequantise oracle.

def _full_layer(key, T=None, skew=False):
    import bench
    cfg = dict(bench.CONFIGS[key], key=key)
    if skew:
        cfg["skew"] = True
    if T:
        cfg["T"] = T
    return bench, cfg


def _check(res):
    assert res["routing_ids_equal"], res
    assert res["ok"], res
    assert res["mean_err"] < 1e-2 * res["mean_abs_ref"] + 1e-3, res


def test_c2_layer_full_size_sampled_tokens(ops):
    """gpt-oss shape, 8192 tokens, 128 experts, MXFP4 weights on the block-scaled tensor-core
    path: 16 sampled tokens against the oracle fed the same MXFP8-quantised activations."""
    bench, cfg = _full_layer("c2")
    dev = torch.device(DEV)
    weights = bench.make_device_layer(cfg, dev)
    layer = bench.Layer(cfg, weights, cfg["T"], dev)
    assert layer.moe._mx_native
    x, logits = bench.make_inputs(cfg, cfg["T"], seed=0)
    out = layer.step(x.to(dev), logits.to(dev)).clone()
    assert torch.ops._xpu_C.b200_device_status() == 0
    assert torch.isfinite(out.float()).all()
    _check(bench.parity_check(cfg, layer, x, logits, out, dev, n_tokens=16))


@pytest.fixture(scope="module")
def c3_weights():
    import bench
    dev = torch.device(DEV)
    cfg = dict(bench.CONFIGS["c3"], key="c3")
    w = bench.make_device_layer(cfg, dev)
    yield cfg, w
    del w
    torch.cuda.empty_cache()


def test_c3_layer_full_size_sampled_tokens(ops, c3_weights):
    """DeepSeek-V3 shape, 16384 tokens, 256 experts, grouped routing: 16 sampled tokens."""
    import bench
    cfg, weights = c3_weights
    dev = torch.device(DEV)
    layer = bench.Layer(cfg, weights, cfg["T"], dev)
    x, logits = bench.make_inputs(cfg, cfg["T"], seed=0)
    out = layer.step(x.to(dev), logits.to(dev)).clone()
    assert torch.ops._xpu_C.b200_device_status() == 0
    assert torch.isfinite(out.float()).all()
    _check(bench.parity_check(cfg, layer, x, logits, out, dev, n_tokens=16))


def test_c3_layer_with_power_of_two_scales_full_size(ops):
    """The same layer with its 128x128 block scales rounded up to powers of two: the layer picks
    the kernel that lets the tensor core apply the scales (and quantises activations the same
    way); 16 sampled tokens against the oracle quantising likewise."""
    import bench
    dev = torch.device(DEV)
    cfg = dict(bench.CONFIGS["c3"], key="c3", pow2_scales=True)
    weights = bench.make_device_layer(cfg, dev)
    layer = bench.Layer(cfg, weights, cfg["T"], dev)
    assert layer.moe.act_scales_pow2
    x, logits = bench.make_inputs(cfg, cfg["T"], seed=0)
    out = layer.step(x.to(dev), logits.to(dev)).clone()
    assert torch.ops._xpu_C.b200_device_status() == 0
    assert torch.isfinite(out.float()).all()
    _check(bench.parity_check(cfg, layer, x, logits, out, dev, n_tokens=16))
    del layer, weights
    torch.cuda.empty_cache()


@pytest.mark.parametrize("T", [1, 8, 32, 128, 256])
def test_c4_decode_sweep_with_zipf_routing(ops, c3_weights, T):
    """The decode regime on the same weights: few tokens and router logits offset by
    1.5*log(1/rank) so that a handful of experts take most rows (hot experts span several
    32-token chunks of the decode-regime kernel).  Every token is checked for T <= 8."""
    import bench
    cfg, weights = c3_weights
    cfg = dict(cfg, T=T, skew=True)
    dev = torch.device(DEV)
    layer = bench.Layer(cfg, weights, T, dev)
    x, logits = bench.make_inputs(cfg, T, seed=0)
    out = layer.step(x.to(dev), logits.to(dev)).clone()
    assert torch.ops._xpu_C.b200_device_status() == 0
    res = bench.parity_check(cfg, layer, x, logits, out, dev, n_tokens=8)
    _check(res)
