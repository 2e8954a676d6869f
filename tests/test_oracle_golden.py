"""The CPU oracle against outputs of the reference project's own torch oracles
(tests/golden/*.npz, written by tests/golden/make_golden.py) and against the
known answers the reference documents."""
import glob
import os

import pytest
import torch

from conftest import GOLDEN, as_bf16, load_golden
from oracle import moe_oracle as O


def _names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


@pytest.mark.parametrize("name", _names("topk_"))
def test_topk_matches_reference(name):
    g = load_golden(name)
    k = g["k"]
    if name == "topk_ties":
        w, i = O.topk_softmax(g["logits"], k, True)
        assert torch.equal(i, g["i"]) and torch.equal(w, g["w"])
        return
    renorm = bool(g["renorm"])
    w, i = O.topk_softmax(g["logits"], k, renorm)
    assert torch.equal(i, g["i"]) and torch.equal(w, g["w"])
    w, i = O.topk_softmax(g["logits"], k, renorm, bias=g["bias"], is_padding=g["pad"])
    assert torch.equal(i, g["ib"]) and torch.equal(w, g["wb"])
    w, i = O.topk_sigmoid(g["logits"], k, renorm, bias=g["bias"], routed_scaling_factor=2.5)
    assert torch.equal(i, g["is_"]) and torch.equal(w, g["ws"])


@pytest.mark.parametrize("name", _names("grouped_"))
def test_grouped_topk_matches_reference(name):
    g = load_golden(name)
    logits = as_bf16(g["logits"]) if name == "grouped_bf16" else g["logits"]
    renorm = bool(g.get("renorm", True))
    w, i = O.grouped_topk(logits, g["k"], renorm, g["ng"], g["tg"], "sigmoid", 2.5, g["bias"])
    assert torch.equal(i, g["i"]) and torch.equal(w, g["w"])
    if "i_softmax" in g:
        w, i = O.grouped_topk(logits, g["k"], renorm, g["ng"], g["tg"], "softmax", 1.0, g["bias"])
        assert torch.equal(i, g["i_softmax"]) and torch.equal(w, g["w_softmax"])


@pytest.mark.parametrize("name", _names("align_"))
def test_align_matches_reference(name):
    g = load_golden(name)
    s, e, n = O.moe_align_block_size(g["ids"], g["bs"], g["E"])
    assert torch.equal(s, g["sorted"]) and torch.equal(e, g["experts"]) and torch.equal(n, g["total"])
    s, e, n = O.moe_align_block_size(g["ids"], g["bs"], g["E"], expert_map=g["emap"])
    assert torch.equal(s, g["sorted_m"]) and torch.equal(e, g["experts_m"]) and torch.equal(n, g["total_m"])


def test_align_documented_example():
    # tests/ops/moe_align_block_size_ops.py:56-69 of the reference, shifted to
    # zero-based expert ids (its 1..4 are experts 0..3 of 4 here).
    ids = torch.tensor([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], dtype=torch.int32) - 1
    s, e, n = O.moe_align_block_size(ids, 4, 4)
    assert s[:16].tolist() == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]
    assert e[:4].tolist() == [0, 1, 2, 3] and n.item() == 16


def test_align_with_a_permuted_expert_map_follows_the_reference_kernel():
    # expert_id = expert_map[expert_id] happens BEFORE counting in the reference kernel
    # (csrc/moe/moe_align_sum_kernels.cpp:196-205): runs are ordered by the mapped id.
    ids = torch.tensor([[0, 1], [2, 3], [0, 3]], dtype=torch.int32)
    emap = torch.tensor([2, -1, 0, 1], dtype=torch.int32)
    s, e, n = O.moe_align_block_size(ids, 2, 4, expert_map=emap)
    # key 0 <- id 2 (flat 2); key 1 <- id 3 (flat 3, 5); key 2 <- id 0 (flat 0, 4); id 1 dropped
    assert s[:6].tolist() == [2, 6, 3, 5, 0, 4] and e[:3].tolist() == [0, 1, 2] and n.item() == 6


@pytest.mark.parametrize("name", _names("remap_"))
def test_remap_and_gather_match_reference(name):
    g = load_golden(name)
    hs = as_bf16(g["hs"])
    emap = g.get("emap")
    out, _, rows, rmap = O.remap_hidden_states(hs, None, g["ids"], emap, g["E_loc"])
    n = int(rows.sum())
    assert torch.equal(rows, g["rows"]) and torch.equal(rmap, g["rmap"])
    assert torch.equal(out[:n].view(torch.int16), g["out"][:n])
    gout = O.moe_gather(as_bf16(g["y"]), g["w"], g["rmap"])
    assert torch.equal(gout.view(torch.int16), g["gout"])


def test_activations_match_reference():
    g = load_golden("act")
    x = as_bf16(g["x"])
    assert torch.equal(O.silu_and_mul(x).view(torch.int16), g["silu"])
    assert torch.equal(O.swigluoai_and_mul(x).view(torch.int16), g["oai"])


def test_other_activations_match_reference():
    """gelu / gelu_tanh / relu2 / swiglustep / situ restatements against the reference's
    torch oracles in all three dtypes."""
    g = load_golden("act_more")
    for tag, view in (("bf16", as_bf16), ("f16", lambda t: t), ("f32", lambda t: t)):
        x = view(g["x_" + tag])
        get = lambda k: view(g[k + "_" + tag])
        assert torch.equal(O.gelu_and_mul(x), get("gelu"))
        assert torch.equal(O.gelu_and_mul(x, "tanh"), get("gelu_tanh"))
        assert torch.equal(O.relu2_no_mul(x), get("relu2"))
        assert torch.equal(O.situ_and_mul(x, 1.7, -1.0), get("situ_raw"))
        assert torch.equal(O.situ_and_mul(x, 1.7, 2.0), get("situ_lin"))
        # the reference's python oracle rounds silu(gate) to the input dtype before the
        # product; its kernel (and this restatement) keep fp32: a few ulps apart
        atol, rtol = {"bf16": (1e-3, 1.6e-2), "f16": (1e-3, 1e-3), "f32": (1e-5, 1.3e-6)}[tag]
        torch.testing.assert_close(O.swiglustep_and_mul(x), get("swiglustep"), atol=atol, rtol=rtol)


def test_weight_recipe_restatements_round_trip():
    """MXFP8 and INT4 quantise -> dequantise stays within half a quantisation step."""
    g = torch.Generator().manual_seed(4)
    w = torch.randn(128, 96, generator=g)
    q, s = O.quant_mxfp8_weight(w)
    d = O.dequant_expert_weight("mxfp8", q, s)
    assert ((d - w).abs() <= 2.0 ** -3 * w.abs() + 1e-6).all()
    q4, s4 = O.quant_int4_weight(w.t().contiguous(), group=32, scale_dtype=torch.float32)
    d4 = O.dequant_expert_weight("int4", q4, s4)
    step = s4.repeat_interleave(32, dim=1).t()
    assert ((d4 - w).abs() <= 0.5 * step + 1e-6).all()
    assert torch.equal(O.dequant_expert_weight("fp8", w.to(torch.float8_e4m3fn), torch.tensor(0.5)),
                       w.to(torch.float8_e4m3fn).float() * 0.5)


def test_lora_align_restatement_has_the_reference_test_property():
    """Every block of every enabled slot holds entries of one expert and of that slot's
    tokens; a disabled slot keeps the caller's pre-fill."""
    g = torch.Generator().manual_seed(8)
    T, k, E, bs, L = 100, 6, 64, 16, 3
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    slot = torch.randint(0, L, (T,), generator=g, dtype=torch.int32)
    n = (T * k + E * (bs - 1) + bs - 1) // bs * bs
    nb = n // bs
    srt = torch.full((L * n,), -7, dtype=torch.int32)
    eid = torch.full((L * nb,), -2, dtype=torch.int32)
    npad = torch.full((L,), -13, dtype=torch.int32)
    enabled = torch.tensor([1, 0, 1, 1], dtype=torch.int32)
    srt, eid, npad = O.moe_lora_align_block_size(ids, slot, E, bs, L, n, nb, srt, eid, npad, enabled,
                                                 torch.tensor([0, 1, 2, -1], dtype=torch.int32))
    srt, eid = srt.view(L, nb, bs), eid.view(L, nb)
    assert int(npad[1]) == -13 and (srt[1] == -7).all() and (eid[1] == -2).all()
    for s in (0, 2):
        real = srt[s] != T * k
        assert int(real.sum()) == int((slot == s).sum()) * k
        for b in real.any(1).nonzero().flatten().tolist():
            idx = srt[s, b][real[b]].long()
            assert (ids.flatten()[idx] == eid[s, b]).all() and (slot[idx // k] == s).all()
        assert (eid[s, int(npad[s]) // bs:] == -1).all()


def test_fp8_group_quant_matches_reference():
    g = load_golden("fp8_group")
    # the reference test oracle divides by the scale and has no lower clamp on
    # the scale beyond eps; same formula otherwise
    q, s = O.per_token_group_fp8_quant(g["x"], 128, divide=True)
    assert torch.allclose(s, g["s"], rtol=0, atol=0)
    assert torch.equal(q.view(torch.uint8), g["q"])
    # the operator multiplies by the reciprocal: same scales, values within one code
    q2, s2 = O.per_token_group_fp8_quant(g["x"], 128)
    assert torch.equal(s2, s)
    assert (q2.float() - q.float()).abs().max() <= 32.0
    assert (q2.view(torch.uint8) != g["q"]).float().mean() < 0.01


def test_mxfp4_matches_reference():
    g = load_golden("mxfp4_ref")
    x = as_bf16(g["x"])
    packed, s = O.per_token_group_quant_mxfp4(x)
    # scales: the reference's e8m0 byte b means 2^(b-127)
    assert torch.equal(s, torch.exp2(g["s"].float() - 127.0))
    # codes differ from round-to-nearest-even only at exact midpoints
    deq = O.unpack_e2m1(packed).view(16, -1, 32) * s.unsqueeze(-1)
    assert (deq.view(16, -1) - g["deq"]).abs().max() <= 0.5 * s.max()
    assert (packed != g["q"]).float().mean() < 0.05
    # the weight quantiser used for synthetic data is round-to-nearest-even like the reference
    wq, ws = O.quant_mxfp4_weight(x.float())
    assert torch.equal(ws, g["s"]) and torch.equal(wq, g["q"])
    assert torch.equal(O.dequant_mxfp4(wq, ws), g["deq"])


def test_e2m1_code_points():
    # tests/test_mxfp4_quant.py:113-142 of the reference: every representable value maps to itself
    vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    assert O.e2m1_code(vals).tolist() == list(range(8))
    assert O.e2m1_code(-vals[1:]).tolist() == [c + 8 for c in range(1, 8)]
    assert torch.equal(O.unpack_e2m1(torch.tensor([[0x21]], dtype=torch.uint8)), torch.tensor([[0.5, 1.0]]))


def test_fp8_block_weight_dequant_matches_reference():
    g = load_golden("fp8_block_w")
    w = g["w"].view(torch.float8_e4m3fn)
    assert torch.equal(O.dequant_fp8_block(w, g["s"]), g["deq"])


def test_layer_matches_reference():
    g = load_golden("layer_bf16")
    x, w13, w2 = as_bf16(g["x"]), as_bf16(g["w13"]), as_bf16(g["w2"])
    out = O.fused_moe("bf16", x, w13.transpose(1, 2).contiguous(), None, None,
                      w2.transpose(1, 2).contiguous(), None, None, g["tw"], g["ti"], "silu")
    ref = as_bf16(g["out"]).float()
    # the reference rounds each expert's output and the weights to bf16 before summing
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)


def test_token_expert_indices():
    assert O.token_expert_indices(3, 2).tolist() == [[0, 3], [1, 4], [2, 5]]


def test_init_expert_map():
    assert O.init_expert_map(2, 1, 3).tolist() == [-1, -1, 0, 1, -1, -1]


def test_softplus_sqrt_matches_reference():
    g = load_golden("softplus_sqrt")
    w, i = O.topk_softplus_sqrt(g["logits"], 6, True, 2.5, g["bias"], None, None, g["pad"])
    assert torch.equal(i, g["i1"]) and torch.equal(w, g["w1"])
    w, i = O.topk_softplus_sqrt(g["logits"], 6, False, 1.0, None, g["iid"], g["table"], None)
    assert torch.equal(i, g["i2"]) and torch.equal(w, g["w2"])


def test_reorder_scales_matches_reference():
    g = load_golden("reorder_scales")
    out = O.reorder_mxfp_scales(g["scales"], g["rows"], g["total"])
    assert torch.equal(out, g["out"])


def test_batched_align_known_answer():
    # 3 batches of up to 5 tokens, block 4: runs [0,1,2 | pad] [10..14 | pad pad pad] [] 
    s, b, n = O.batched_moe_align_block_size(5, 4, torch.tensor([3, 5, 0], dtype=torch.int32))
    assert s.tolist() == [0, 1, 2, 15, 5, 6, 7, 8, 9, 15, 15, 15] + [15] * 12
    assert b.tolist() == [0, 1, 1, -1, -1, -1] and n.item() == 12
