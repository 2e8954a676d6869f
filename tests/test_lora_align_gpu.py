"""moe_lora_align_block_size: one alignment per adapter slot.  Bit-exact against the CPU
restatement, plus the property the reference's own test checks (every block holds entries of
one expert, tests/test_moe_lora_align_sum.py:96-107 there) and its three slot-guard
regressions (:240-320), with the same sentinel pre-fills."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
S_EXPERT, S_TOKEN, S_NPAD = -2, -7, -13


def sizes(numel, E, bs):
    n = numel + E * (bs - 1)
    n = (n + bs - 1) // bs * bs
    if numel < E:
        n = numel * bs
    return n, (n + bs - 1) // bs


def sample(T, k, E, max_loras, seed, base_fraction=0.0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    slot = torch.randint(0, max_loras, (T,), generator=g, dtype=torch.int32)
    if base_fraction:
        slot[torch.rand(T, generator=g) < base_fraction] = -1
    return ids, slot


def run(ops, ids, slot, E, bs, max_loras, lora_ids, enabled, emap=None, fills=None):
    max_padded, max_blocks = sizes(ids.numel(), E, bs)
    f_tok, f_exp, f_pad = fills or (ids.numel(), E, 0)
    srt = torch.full((max_loras * max_padded,), f_tok, dtype=torch.int32)
    eid = torch.full((max_loras * max_blocks,), f_exp, dtype=torch.int32)
    npad = torch.full((max_loras,), f_pad, dtype=torch.int32)
    ref = O.moe_lora_align_block_size(ids, slot, E, bs, max_loras, max_padded, max_blocks, srt, eid,
                                      npad, enabled, lora_ids, emap)
    d = [t.to(DEV) for t in (srt, eid, npad)]
    ops._moe_C.moe_lora_align_block_size(ids.to(DEV), slot.to(DEV), E, bs, max_loras, max_padded,
                                         max_blocks, d[0], d[1], d[2], enabled.to(DEV),
                                         lora_ids.to(DEV), None if emap is None else emap.to(DEV))
    return [t.cpu() for t in d], ref, (max_padded, max_blocks)


@pytest.mark.parametrize("T", [1, 100, 1024, 4096])
@pytest.mark.parametrize("E", [64, 128, 512])
@pytest.mark.parametrize("max_loras", [2, 32])
def test_vs_oracle_and_block_property(ops, T, E, max_loras):
    k, bs = 6, 16
    ids, slot = sample(T, k, E, max_loras, seed=T + E)
    lora_ids = torch.arange(max_loras + 2, dtype=torch.int32)   # as the reference's test passes it
    enabled = torch.ones(max_loras + 1, dtype=torch.int32)
    (srt, eid, npad), ref, (max_padded, _) = run(ops, ids, slot, E, bs, max_loras, lora_ids, enabled)
    assert torch.equal(srt, ref[0]) and torch.equal(eid, ref[1]) and torch.equal(npad, ref[2])
    flat = ids.flatten()
    srt, eid = srt.view(max_loras, -1, bs), eid.view(max_loras, -1)
    seen = 0
    for s in range(max_loras):
        real = srt[s] != ids.numel()
        seen += int(real.sum())
        blocks = real.any(1).nonzero().flatten()
        for b in blocks.tolist():
            idx = srt[s, b][real[b]].long()
            assert (flat[idx] == eid[s, b]).all()
            assert (slot[idx // k] == s).all()
        assert int(npad[s]) % bs == 0 and int(npad[s]) <= max_padded
    assert seen == ids.numel()          # every (token, slot) entry lands in exactly one row


def test_int64_ids_and_expert_map(ops):
    E, bs, max_loras = 64, 16, 4
    ids, slot = sample(300, 6, E, max_loras, seed=5, base_fraction=0.2)
    emap = torch.full((E,), -1, dtype=torch.int32)
    emap[16:48] = torch.arange(32, dtype=torch.int32)
    lora_ids = torch.tensor([-1, 0, 1, 2, 3], dtype=torch.int32)
    enabled = torch.ones(max_loras + 1, dtype=torch.int32)
    out, ref, _ = run(ops, ids.to(torch.int64), slot, E, bs, max_loras, lora_ids, enabled, emap)
    for a, b in zip(out, ref):
        assert torch.equal(a, b)
    assert int(out[1].max()) < 32       # block labels are the mapped ids


@pytest.mark.parametrize("max_loras", [1, 2])
def test_real_slot_not_skipped_behind_a_minus_one(ops, max_loras):
    E, bs = 64, 16
    ids, _ = sample(16, 6, E, 1, seed=1)
    slot = torch.tensor([0] * 8 + [-1] * 8, dtype=torch.int32)
    lora_ids = torch.full((max_loras + 1,), -1, dtype=torch.int32)
    u = torch.unique(slot, sorted=True)
    lora_ids[: u.numel()] = u
    assert int(lora_ids[0]) == -1
    enabled = torch.ones(max_loras + 1, dtype=torch.int32)
    (srt, eid, npad), ref, (max_padded, _) = run(ops, ids, slot, E, bs, max_loras, lora_ids, enabled,
                                                 fills=(S_TOKEN, S_EXPERT, S_NPAD))
    assert 0 < int(npad[0]) <= max_padded and int(npad[0]) % bs == 0
    assert (eid.view(max_loras, -1)[0] != S_EXPERT).all()
    assert (srt.view(max_loras, -1)[0] != S_TOKEN).all()
    for a, b in zip((srt, eid, npad), ref):
        assert torch.equal(a, b)


def test_disabled_slot_is_untouched(ops):
    E, bs, max_loras = 64, 16, 1
    ids, _ = sample(16, 6, E, 1, seed=1)
    slot = torch.zeros(16, dtype=torch.int32)
    lora_ids = torch.tensor([0, -1], dtype=torch.int32)
    enabled = torch.tensor([0, 1], dtype=torch.int32)
    (srt, eid, npad), _, _ = run(ops, ids, slot, E, bs, max_loras, lora_ids, enabled,
                                 fills=(S_TOKEN, S_EXPERT, S_NPAD))
    assert int(npad[0]) == S_NPAD and (eid == S_EXPERT).all() and (srt == S_TOKEN).all()


def test_out_of_range_slot_id_is_ignored(ops):
    E, bs, max_loras = 64, 16, 1
    ids, _ = sample(16, 6, E, 1, seed=1)
    slot = torch.zeros(16, dtype=torch.int32)
    lora_ids = torch.tensor([0, 5], dtype=torch.int32)
    enabled = torch.ones(2, dtype=torch.int32)
    (srt, eid, npad), ref, _ = run(ops, ids, slot, E, bs, max_loras, lora_ids, enabled,
                                   fills=(S_TOKEN, S_EXPERT, S_NPAD))
    assert int(npad[0]) != S_NPAD
    for a, b in zip((srt, eid, npad), ref):
        assert torch.equal(a, b)
