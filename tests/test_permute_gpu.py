"""moe_align_block_size, remap_hidden_states, init_expert_map, moe_gather and
moe_sum against the CPU oracle: every integer output bit-exact (the kernels are
stable, so the element order is the stable-sort order, not just the multiset)."""
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


def run_align(ops, ids, bs, E, emap=None, pad_sorted=False):
    n, nb = O.align_sizes(ids.numel(), E, bs, pad_sorted)
    s = torch.empty(n, dtype=torch.int32, device=DEV)
    e = torch.empty(nb, dtype=torch.int32, device=DEV)
    t = torch.empty(1, dtype=torch.int32, device=DEV)
    ops._moe_C.moe_align_block_size(ids.to(DEV), E, bs, s, e, t, None if emap is None else emap.to(DEV))
    return s.cpu(), e.cpu(), t.cpu()


@pytest.mark.parametrize("name", _names("align_"))
def test_align_golden(ops, name):
    g = load_golden(name)
    s, e, t = run_align(ops, g["ids"], g["bs"], g["E"])
    assert torch.equal(s, g["sorted"]) and torch.equal(e, g["experts"]) and torch.equal(t, g["total"])
    s, e, t = run_align(ops, g["ids"], g["bs"], g["E"], g["emap"])
    assert torch.equal(s, g["sorted_m"]) and torch.equal(e, g["experts_m"]) and torch.equal(t, g["total_m"])


@pytest.mark.parametrize("T,k,E,bs", [(1, 1, 8, 16), (64, 2, 8, 128), (256, 8, 256, 128), (257, 8, 256, 64),
                                      (4096, 2, 8, 128), (8192, 4, 128, 128), (16384, 8, 256, 128),
                                      (1000, 6, 60, 16), (3, 8, 1024, 4)])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_align_vs_oracle(ops, T, k, E, bs, dtype):
    g = torch.Generator().manual_seed(T + E)
    ids = torch.randint(0, E, (T, k), generator=g).to(dtype)
    rs, re, rt = O.moe_align_block_size(ids, bs, E)
    s, e, t = run_align(ops, ids, bs, E)
    assert torch.equal(t, rt) and torch.equal(e, re) and torch.equal(s, rs)
    # twice in a row: same answer (no atomics-ordered output)
    s2, _, _ = run_align(ops, ids, bs, E)
    assert torch.equal(s, s2)


@pytest.mark.parametrize("T,k,E,bs", [(3, 2, 4, 2), (500, 4, 32, 16), (5000, 8, 256, 128)])
def test_align_with_a_permuted_expert_map(ops, T, k, E, bs):
    """A map that is not monotone reorders the runs: they follow the mapped id, as in the
    reference kernel (csrc/moe/moe_align_sum_kernels.cpp:196-205)."""
    g = torch.Generator().manual_seed(E)
    ids = torch.randint(0, E, (T, k), generator=g).to(torch.int32)
    emap = torch.randperm(E, generator=g).to(torch.int32)
    emap[torch.rand(E, generator=g) < 0.3] = -1
    rs, re, rt = O.moe_align_block_size(ids, bs, E, expert_map=emap)
    s, e, t = run_align(ops, ids, bs, E, emap)
    assert torch.equal(t, rt) and torch.equal(e, re) and torch.equal(s, rs)


def test_align_skewed_and_out_of_range(ops):
    ids = torch.zeros(5000, 4, dtype=torch.int32)       # every token on expert 0
    ids[::7, 1] = 99                                     # ids >= num_experts are ignored
    rs, re, rt = O.moe_align_block_size(ids, 128, 16)
    s, e, t = run_align(ops, ids, 128, 16)
    assert torch.equal(t, rt) and torch.equal(e, re) and torch.equal(s, rs)


@pytest.mark.parametrize("name", _names("remap_"))
def test_remap_golden(ops, name):
    g = load_golden(name)
    hs = as_bf16(g["hs"])
    T, k = g["ids"].shape
    E_loc = g["E_loc"]
    emap = g.get("emap")
    out = torch.zeros(T * k, hs.shape[1], dtype=torch.bfloat16, device=DEV)
    rows = torch.zeros(E_loc, dtype=torch.int32, device=DEV)
    rmap = torch.empty(T, k, dtype=torch.int32, device=DEV)
    ops._moe_C.remap_hidden_states(hs.to(DEV), None, out, None, None if emap is None else emap.to(DEV),
                                   rows, rmap, g["ids"].to(DEV), 32 if emap is not None else E_loc, E_loc)
    n = int(g["rows"].sum())
    assert torch.equal(rows.cpu(), g["rows"]) and torch.equal(rmap.cpu(), g["rmap"])
    assert torch.equal(out.cpu()[:n].view(torch.int16), g["out"][:n])
    gout = torch.empty(T, hs.shape[1], dtype=torch.bfloat16, device=DEV)
    ops._moe_C.moe_gather(gout, as_bf16(g["y"]).to(DEV), g["w"].to(DEV), rmap, E_loc)
    assert torch.allclose(gout.cpu().float(), as_bf16(g["gout"]).float(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("T,H,E,k,ep", [(1, 128, 8, 2, 1), (64, 1024, 8, 2, 1), (300, 512, 64, 4, 4),
                                        (2048, 256, 256, 8, 8), (4096, 128, 128, 4, 1)])
@pytest.mark.parametrize("fmt", ["bf16", "fp8"])
def test_remap_vs_oracle(ops, T, H, E, k, ep, fmt):
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    scales = None
    if fmt == "fp8":
        x, scales = O.per_token_group_fp8_quant(x, 128)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int64)
    E_loc = E // ep
    emap = O.init_expert_map(E_loc, ep - 1, ep) if ep > 1 else None
    if ep > 1:
        dm = torch.empty(E, dtype=torch.int32, device=DEV)
        ops._moe_C.init_expert_map(dm, E_loc, ep - 1, ep)
        assert torch.equal(dm.cpu(), emap)
    ro, rs, rrows, rmap = O.remap_hidden_states(x, scales, ids, emap, E_loc)
    out = torch.zeros(T * k, H, dtype=x.dtype, device=DEV)
    so = None if scales is None else torch.zeros(T * k, scales.shape[1], dtype=torch.float32, device=DEV)
    rows = torch.zeros(E_loc, dtype=torch.int32, device=DEV)
    m = torch.empty(T, k, dtype=torch.int32, device=DEV)
    ops._moe_C.remap_hidden_states(x.to(DEV), None if scales is None else scales.to(DEV), out, so,
                                   None if emap is None else emap.to(DEV), rows, m, ids.to(DEV), E, E_loc)
    n = int(rrows.sum())
    assert torch.equal(rows.cpu(), rrows) and torch.equal(m.cpu(), rmap)
    assert torch.equal(out.cpu()[:n].view(torch.uint8), ro[:n].view(torch.uint8))
    if scales is not None:
        assert torch.equal(so.cpu()[:n], rs[:n])


@pytest.mark.parametrize("T,k,H", [(1, 8, 7168), (37, 2, 1024), (512, 4, 2880), (100, 6, 136)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_gather_and_sum_vs_oracle(ops, T, k, H, dtype):
    g = torch.Generator().manual_seed(1)
    y = torch.randn(T * k, H, generator=g).to(dtype)
    w = torch.rand(T, k, generator=g)
    rmap = torch.randperm(T * k, generator=g).view(T, k).to(torch.int32)
    rmap[torch.rand(T, k, generator=g) < 0.2] = -1
    ref = O.moe_gather(y, w, rmap)
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    ops._moe_C.moe_gather(out, y.to(DEV), w.to(DEV), rmap.to(DEV), 8)
    assert torch.allclose(out.cpu().float(), ref.float(), atol=1e-2, rtol=1e-2)

    x3 = y.view(T, k, H)
    ids = torch.randint(-1, 8, (T, k), generator=g).to(torch.int32)
    emap = torch.tensor([0, -1, 1, 2, -1, 3, 4, 5], dtype=torch.int32)
    for args, ref in (((None, None), O.moe_sum(x3)), ((ids, None), O.moe_sum(x3, ids)),
                      ((ids, emap), O.moe_sum(x3, ids, emap))):
        out = torch.empty(T, H, dtype=dtype, device=DEV)
        ops._moe_C.moe_sum(x3.to(DEV), out, *[None if a is None else a.to(DEV) for a in args])
        assert torch.allclose(out.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_moe_sum_input_validation(ops):
    m, topk, k = 32, 4, 128
    inp = torch.randn((m, topk, k), device=DEV)
    out = torch.empty((m, k), device=DEV)
    ids = torch.zeros((m, topk), device=DEV, dtype=torch.int32)
    emap = torch.arange(8, device=DEV, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="expert_map requires topk_ids"):
        ops._moe_C.moe_sum(inp, out, None, emap)
    with pytest.raises(RuntimeError, match="same dtype"):
        ops._moe_C.moe_sum(inp, out.half(), None, None)
    with pytest.raises(RuntimeError, match="contiguous"):
        ops._moe_C.moe_sum(torch.randn((m, topk, 2 * k), device=DEV)[:, :, ::2], out, None, None)
    with pytest.raises(RuntimeError, match="num_tokens, topk"):
        ops._moe_C.moe_sum(inp, out, ids[:, :topk - 1].contiguous(), None)
    with pytest.raises(RuntimeError, match="expert_map must be int32"):
        ops._moe_C.moe_sum(inp, out, ids, emap.to(torch.int64))
