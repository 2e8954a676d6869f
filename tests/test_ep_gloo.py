"""Expert-parallel dispatch / combine on two CPU ranks (gloo): the exchange logic of
vllm_xpu_kernels/ep.py with torch stand-ins for the three CUDA steps, against the
single-process layer oracle.  Also a rank that never joins: the others must get an
error from the process-group timeout, not hang."""
import datetime
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_DIR, ROOT
from oracle import moe_oracle as O

CFG = dict(T=40, H=64, I=96, E=8, k=2, recipe="bf16", routing="softmax", activation="silu", bias=False)


def _cpu_plan(hidden, scales, topk_ids, experts_per_rank, world):
    from vllm_xpu_kernels.ep import Plan
    E_total = experts_per_rank * world
    rank_of = torch.arange(E_total, dtype=torch.int32) // experts_per_rank
    rows, rs, counts, row_map = O.remap_hidden_states(hidden, scales, topk_ids, rank_of, world)
    send_expert = torch.empty(topk_ids.numel(), dtype=torch.int32)
    send_expert[row_map.flatten().long()] = (topk_ids.flatten() % experts_per_rank).to(torch.int32)
    return Plan(rows, rs, send_expert, counts, row_map)


def _cpu_combine(output, returned, topk_weights, row_map):
    output.copy_(O.moe_gather(returned, topk_weights, row_map, output.dtype))


def _worker(rank, world, port, result):
    for p in (ROOT, PKG_DIR):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vllm_xpu_kernels.ep import ExpertParallel
    layer = O.make_layer(CFG, seed=0)                      # same weights on every rank
    per = CFG["E"] // world
    lo = rank * per
    tokens = O.make_layer(CFG, seed=100 + rank)            # this rank's tokens
    x, logits = tokens["x"], tokens["logits"]
    w, ids = O.topk_softmax(logits, CFG["k"], True)

    def local_fn(rows, scales, experts):
        n = rows.shape[0]
        return O.fused_moe("bf16", rows, layer["w13"][lo:lo + per], None, None, layer["w2"][lo:lo + per],
                           None, None, torch.ones(n, 1), experts.view(n, 1).long(), "silu",
                           out_dtype=torch.bfloat16)

    ep = ExpertParallel(dist.group.WORLD, per, local_fn, _cpu_plan, _cpu_combine)
    out = torch.empty(CFG["T"], CFG["H"], dtype=torch.bfloat16)
    ep.apply(out, x, w, ids)
    ref = O.fused_moe("bf16", x, layer["w13"], None, None, layer["w2"], None, None, w, ids, "silu",
                      out_dtype=torch.float32)
    err = (out.float() - ref).abs().max().item()
    recv = torch.tensor([ep.last_recv_rows])
    dist.all_reduce(recv)
    result[rank] = (err, int(recv.item()))
    dist.destroy_process_group()


def test_dispatch_combine_two_ranks():
    world = 2
    with mp.Manager() as m:
        result = m.dict()
        mp.spawn(_worker, args=(world, 29611, result), nprocs=world, join=True)
        assert len(result) == world
        for rank in range(world):
            err, total_rows = result[rank]
            assert err < 3e-2, f"rank {rank}: max err {err}"
            assert total_rows == world * CFG["T"] * CFG["k"]     # every routed row arrived somewhere


def _late_worker(rank, world, port, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if rank == 1:
        result[rank] = "never joined"
        return                                                    # this rank does not show up
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=3))
        result[rank] = "joined"
    except Exception as e:                                        # noqa: BLE001
        result[rank] = "error: " + type(e).__name__


def test_missing_rank_is_an_error_not_a_hang():
    with mp.Manager() as m:
        result = m.dict()
        mp.spawn(_late_worker, args=(2, 29613, result), nprocs=2, join=True)
        assert result[1] == "never joined"
        assert result[0].startswith("error")


def test_peer_exchange_refuses_calls_beyond_its_buffers():
    """PeerExpertParallel sizes its exchange buffers and address tables at construction; a call
    with more tokens, another top-k, another row width or missing scales must be refused before
    any kernel is enqueued (no device needed for the check itself)."""
    from vllm_xpu_kernels.ep import PeerExpertParallel
    ep = object.__new__(PeerExpertParallel)
    ep.T, ep.k, ep.H, ep.row_bytes, ep.scale_row_bytes = 16, 2, 64, 64, 0
    x = torch.zeros(16, 64, dtype=torch.float8_e4m3fn)
    ids = torch.zeros(16, 2, dtype=torch.int32)
    ep.check_call(x, ids, None)                                        # fits
    ep.check_call(x[:8], ids[:8], None)                                # fewer tokens fit too
    with pytest.raises(ValueError, match="at most 16 tokens"):
        ep.check_call(torch.zeros(17, 64, dtype=torch.float8_e4m3fn), torch.zeros(17, 2, dtype=torch.int32), None)
    with pytest.raises(ValueError, match="top-2"):
        ep.check_call(x, torch.zeros(16, 4, dtype=torch.int32), None)
    with pytest.raises(ValueError, match="rows of 64 bytes"):
        ep.check_call(torch.zeros(16, 64, dtype=torch.bfloat16), ids, None)
    with pytest.raises(ValueError, match="activation scales"):
        ep.check_call(x, ids, torch.zeros(16, 1))
