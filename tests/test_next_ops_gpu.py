"""The operators either side of the hot path that share its registry: softplus-sqrt routing
(with hash routing), the batched align variant, and the MX activation-scale re-layout."""
import ctypes

import pytest
import torch

from conftest import load_golden
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_softplus(ops, logits, k, renorm, scale, bias=None, iid=None, table=None, pad=None):
    T = logits.shape[0]
    w = torch.empty(T, k, dtype=torch.float32, device=DEV)
    ids = torch.empty(T, k, dtype=torch.int32, device=DEV)
    src = torch.empty(T, k, dtype=torch.int32, device=DEV)
    d = lambda t: None if t is None else t.to(DEV)  # noqa: E731
    ops._moe_C.topk_softplus_sqrt(w, ids, src, logits.to(DEV), renorm, scale, d(bias), d(iid), d(table), d(pad))
    return w.cpu(), ids.cpu()


def test_softplus_sqrt_golden(ops):
    g = load_golden("softplus_sqrt")
    w, i = run_softplus(ops, g["logits"], 6, True, 2.5, g["bias"], None, None, g["pad"])
    assert torch.equal(i, g["i1"]) and torch.allclose(w, g["w1"], atol=2e-2, rtol=0)
    w, i = run_softplus(ops, g["logits"], 6, False, 1.0, None, g["iid"], g["table"], None)
    assert torch.equal(i, g["i2"]) and torch.allclose(w, g["w2"], atol=2e-2, rtol=0)


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (513, 256, 8), (64, 384, 6)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softplus_sqrt_vs_oracle(ops, T, E, k, dtype):
    g = torch.Generator().manual_seed(E)
    logits = (torch.randn(T, E, generator=g) * 3).to(dtype)
    bias = torch.randn(E, generator=g) * 0.05
    rw, ri = O.topk_softplus_sqrt(logits, k, True, 1.5, bias)
    w, i = run_softplus(ops, logits, k, True, 1.5, bias)
    keys = torch.nn.functional.softplus(logits.float()).sqrt() + bias
    bad = (i != ri).any(dim=1)
    assert not (bad & (O.routing_margin(keys, k) > 1e-6)).any()
    assert torch.allclose(w[~bad], rw[~bad], atol=2e-2, rtol=0)


@pytest.mark.parametrize("max_tokens,E,bs,empty", [(13, 8, 8, False), (16, 64, 16, True), (512, 32, 64, False),
                                                  (512, 16, 32, True)])
def test_batched_align_vs_oracle(ops, max_tokens, E, bs, empty):
    g = torch.Generator().manual_seed(max_tokens + E)
    n = torch.randint(0, max_tokens, (E,), generator=g).to(torch.int32)
    if empty:
        n[torch.randperm(E, generator=g)[: E // 2]] = 0
    rs, rb, rn = O.batched_moe_align_block_size(max_tokens, bs, n)
    s = torch.empty_like(rs, device=DEV)
    b = torch.empty_like(rb, device=DEV)
    t = torch.empty(1, dtype=torch.int32, device=DEV)
    ops._moe_C.batched_moe_align_block_size(max_tokens, bs, n.to(DEV), s, b, t)
    assert torch.equal(s.cpu(), rs) and torch.equal(b.cpu(), rb) and torch.equal(t.cpu(), rn)


@pytest.mark.parametrize("rows", [[0, 1, 2, 3, 4, 5, 7, 8], [16, 0, 33, 100], [1], [0, 0, 0], [128, 256, 200, 137]])
@pytest.mark.parametrize("scale_k", [4, 8, 40])
def test_reorder_mxfp_scales_vs_oracle(ops, rows, scale_k):
    total = sum(rows)
    g = torch.Generator().manual_seed(scale_k)
    sc = torch.randint(0, 256, (max(total, 1), scale_k), generator=g, dtype=torch.uint8)[:total]
    upper = total + 3 * len(rows)
    ref = O.reorder_mxfp_scales(sc, torch.tensor(rows), upper)
    out = ops._moe_C.reorder_mxfp_scales(sc.view(torch.float8_e8m0fnu).to(DEV),
                                         torch.tensor(rows, dtype=torch.int32, device=DEV), upper)
    assert out.shape == (upper, scale_k)
    assert torch.equal(out.cpu().view(torch.uint8), ref)


def test_reorder_scales_golden(ops):
    g = load_golden("reorder_scales")
    out = ops._moe_C.reorder_mxfp_scales(g["scales"].view(torch.float8_e8m0fnu).to(DEV), g["rows"].to(DEV),
                                         g["total"])
    assert torch.equal(out.cpu().view(torch.uint8), g["out"])


def test_bounded_wait_gives_up_and_reports():
    """A device-side wait that nothing will ever satisfy returns after its budget and leaves
    B200MOE_TIMEOUT in the status word; the context stays usable."""
    from vllm_xpu_kernels import capi
    lib = capi.lib()
    st = torch.cuda.current_stream().cuda_stream
    assert lib.b200moe_selftest_wait_timeout(2_000_000, st) == capi.OK      # ~1 ms of cycles
    status = ctypes.c_int(0)
    assert lib.b200moe_device_status(st, ctypes.byref(status)) == capi.OK
    assert status.value == capi.TIMEOUT
    assert lib.b200moe_device_status(st, ctypes.byref(status)) == capi.OK and status.value == 0  # cleared
    x = torch.ones(8, device=DEV)
    assert float((x * 2).sum()) == 16.0
