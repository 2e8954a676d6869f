"""Routing kernels against the CPU oracle and the committed golden vectors.
Ids must be bit-exact; weights within 2e-2 (the reference's own tolerance,
tests/test_topk.py:56-59 there)."""
import glob
import os

import pytest
import torch

from conftest import GOLDEN, as_bf16, load_golden
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


def run_topk(ops, kind, logits, k, renorm, bias=None, pad=None, scale=1.0, ids_dtype=torch.int32):
    T = logits.shape[0]
    w = torch.empty(T, k, dtype=torch.float32, device=DEV)
    ids = torch.empty(T, k, dtype=ids_dtype, device=DEV)
    src = torch.empty(T, k, dtype=torch.int32, device=DEV)
    lg = logits.to(DEV)
    b = None if bias is None else bias.to(DEV)
    p = None if pad is None else pad.to(DEV)
    if kind == "softmax":
        ops._moe_C.topk_softmax(w, ids, src, lg, renorm, b, p)
    else:
        ops._moe_C.topk_sigmoid(w, ids, src, lg, renorm, b, scale, p)
    return w.cpu(), ids.cpu(), src.cpu()


def assert_ids(ids, ref_ids, margin, what):
    """Expert ids are bit-exact.  When a row differs, the message says whether the oracle's own
    k-th/(k+1)-th keys on that row are within a few ulp (there two correct fp32 evaluations may
    differ) -- a diagnosis, not an excuse: the test fails either way."""
    bad = (ids.to(torch.int64) != ref_ids.to(torch.int64)).any(dim=1)
    if bad.any():
        near = int((bad & (margin <= 4e-7)).sum())
        raise AssertionError(f"{what}: {int(bad.sum())} rows with different expert ids "
                             f"({near} of them with a selection margin below 4e-7)")
    return 0


@pytest.mark.parametrize("name", _names("topk_"))
def test_topk_golden(ops, name):
    g = load_golden(name)
    k = g["k"]
    renorm = bool(g.get("renorm", True))
    w, i, src = run_topk(ops, "softmax", g["logits"], k, renorm)
    assert torch.equal(i, g["i"])
    assert torch.allclose(w, g["w"], atol=2e-2, rtol=0)
    assert torch.equal(src, O.token_expert_indices(g["logits"].shape[0], k))
    if "ib" in g:
        w, i, _ = run_topk(ops, "softmax", g["logits"], k, renorm, g["bias"], g["pad"])
        assert torch.equal(i, g["ib"]) and torch.allclose(w, g["wb"], atol=2e-2, rtol=0)
        assert (w[g["pad"]] == 0).all()
        w, i, _ = run_topk(ops, "sigmoid", g["logits"], k, renorm, g["bias"], None, 2.5)
        assert torch.equal(i, g["is_"]) and torch.allclose(w, g["ws"], atol=2e-2, rtol=0)


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (64, 8, 2), (4096, 8, 2), (8192, 128, 4), (333, 60, 6),
                                   (257, 256, 8), (100, 512, 10), (31, 1024, 32), (5, 4, 4), (9, 3, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_topk_softmax_vs_oracle(ops, T, E, k, dtype):
    g = torch.Generator().manual_seed(T * 1000 + E)
    logits = torch.randn(T, E, generator=g).to(dtype)
    for renorm in (True, False):
        rw, ri = O.topk_softmax(logits, k, renorm)
        w, i, _ = run_topk(ops, "softmax", logits, k, renorm, ids_dtype=torch.int64)
        margin = O.routing_margin(torch.softmax(logits.float(), -1), k)
        flips = assert_ids(i, ri, margin, "topk_softmax")
        if flips == 0:
            assert torch.allclose(w, rw, atol=2e-2, rtol=0)


@pytest.mark.parametrize("T,E,k", [(64, 8, 2), (2048, 256, 8), (77, 96, 5)])
def test_topk_sigmoid_vs_oracle(ops, T, E, k):
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(T, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.01
    rw, ri = O.topk_sigmoid(logits, k, True, bias, 2.5)
    w, i, _ = run_topk(ops, "sigmoid", logits, k, True, bias, None, 2.5)
    margin = O.routing_margin(torch.sigmoid(logits) + bias, k)
    if assert_ids(i, ri, margin, "topk_sigmoid") == 0:
        assert torch.allclose(w, rw, atol=2e-2, rtol=0)


def test_topk_ties_go_to_lower_index(ops):
    logits = torch.zeros(5, 64)
    w, i, _ = run_topk(ops, "softmax", logits, 4, True)
    assert i.tolist() == [[0, 1, 2, 3]] * 5


def test_topk_empty(ops):
    w, i, _ = run_topk(ops, "softmax", torch.zeros(0, 8), 2, True)
    assert w.shape == (0, 2)


def run_grouped(ops, logits, bias, ng, tg, k, renorm, scale, scoring=1):
    v, i = ops._moe_C.grouped_topk(logits.to(DEV), ng, tg, k, renorm, scale, bias.to(DEV), scoring)
    assert v.dtype == torch.float32 and i.dtype == torch.int32
    return v.cpu(), i.cpu()


@pytest.mark.parametrize("name", _names("grouped_"))
def test_grouped_topk_golden(ops, name):
    g = load_golden(name)
    logits = as_bf16(g["logits"]) if name == "grouped_bf16" else g["logits"]
    renorm = bool(g.get("renorm", True))
    v, i = run_grouped(ops, logits, g["bias"], g["ng"], g["tg"], g["k"], renorm, 2.5)
    assert torch.equal(i, g["i"])
    assert torch.allclose(v, g["w"], atol=2e-2, rtol=0)
    if "i_softmax" in g:
        # scoring_func 0: scores activated by the caller
        sm = torch.softmax(logits, dim=-1)
        v, i = run_grouped(ops, sm, g["bias"], g["ng"], g["tg"], g["k"], renorm, 1.0, scoring=0)
        assert torch.equal(i, g["i_softmax"])
        assert torch.allclose(v, g["w_softmax"], atol=2e-2, rtol=0)


@pytest.mark.parametrize("T", [1, 8, 256, 16384])
def test_grouped_topk_deepseek_shape(ops, T):
    cfg = O.CONFIGS["c3"]
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(T, 256, generator=g)
    bias = torch.randn(256, generator=g) * 0.01
    rw, ri = O.grouped_topk(logits, 8, True, 8, 4, "sigmoid", 2.5, bias)
    v, i = run_grouped(ops, logits, bias, 8, 4, 8, True, 2.5)
    keys = torch.sigmoid(logits) + bias
    bad = (i != ri).any(dim=1)
    if bad.any():  # ids are bit-exact; the gaps are printed to tell a near-tie from a wrong selection
        srt = torch.sort(keys[bad], dim=-1).values
        gaps = (srt[:, 1:] - srt[:, :-1]).min(dim=-1).values
        raise AssertionError(f"{int(bad.sum())} of {T} rows differ from the oracle; smallest key gaps "
                             f"on those rows: {gaps[:8].tolist()}")
    assert torch.allclose(v, rw, atol=2e-2, rtol=0)
    # properties that hold at any size: ids distinct, at most topk_group groups used, weights sum to scale
    assert (torch.sort(i, dim=1).values.diff(dim=1) > 0).all()
    assert ((i // 32).to(torch.int64).unsqueeze(-1) == torch.arange(8)).any(1).sum(1).max() <= 4
    assert torch.allclose(v.sum(1), torch.full((T,), 2.5), atol=1e-4)


def test_grouped_topk_edge_rows_of_the_reference_kernel(ops):
    """Rows the torch oracle of the reference does not define but its kernel does
    (csrc/moe/grouped_topk.cpp:608-624, 659-662, 678-687): too few groups with a finite score,
    all-zero scores under renormalisation, -inf scores inside the kept groups."""
    E, n_group, topk_group, k = 64, 8, 4, 4
    g = torch.Generator().manual_seed(5)
    scores = torch.rand(6, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.01
    scores[0, 24:] = float("-inf")              # 3 finite groups < topk_group: degenerate row
    scores[1] = 0.0                             # selected scores sum to zero
    scores[2, ::3] = float("-inf")              # holes inside every group
    scores[3, :56] = float("-inf")              # one finite group only: degenerate
    scores[4, 8:16] = float("-inf")             # one dead group among eight: still a normal row
    zero_bias = torch.zeros(E)
    for b in (bias, zero_bias):
        w, ids = ops._moe_C.grouped_topk(scores.to(DEV), n_group, topk_group, k, True, 2.5, b.to(DEV), 0)
        rw, rids = O.grouped_topk_kernel_semantics(scores, k, True, n_group, topk_group, "none", 2.5, b)
        assert torch.equal(ids.cpu(), rids)
        assert torch.isfinite(w).all()
        assert torch.allclose(w.cpu(), rw, atol=1e-6, rtol=1e-5)
    assert ids.cpu()[0].tolist() == [0, 1, 2, 3] and torch.equal(w.cpu()[0], torch.full((4,), 0.25))
    assert (w.cpu()[1] == 0).all()              # zero-bias pass: 0 / (0 + 1e-20), not NaN
    # rows without such inputs: the kernel semantics and the torch oracle agree
    plain = torch.rand(64, E, generator=g)
    a = O.grouped_topk_kernel_semantics(plain, k, True, n_group, topk_group, "none", 2.5, bias)
    b2 = O.grouped_topk(plain, k, True, n_group, topk_group, "none", 2.5, bias)
    assert torch.equal(a[1], b2[1]) and torch.allclose(a[0], b2[0], atol=1e-7)
