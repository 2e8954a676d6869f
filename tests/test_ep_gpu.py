"""Expert-parallel layer on two GPUs (NCCL): tokens data-parallel, experts sharded,
all-to-all dispatch/combine around the local CUDA layer; result = single-GPU oracle."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

from conftest import PKG_DIR, ROOT
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, recipe, backend, result):
    for p in (ROOT, PKG_DIR):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import vllm_xpu_kernels._C  # noqa: F401
    import vllm_xpu_kernels._moe_C  # noqa: F401
    import vllm_xpu_kernels._xpu_C  # noqa: F401
    from vllm_xpu_kernels.ep import ExpertParallel, make_local_fn
    from vllm_xpu_kernels.fused_moe_interface import XpuFusedMoe
    from vllm_xpu_kernels.moe_utils import quant_fp8_block_act
    cfg = dict(O.CONFIGS["c0" if recipe == "bf16" else "c1"], T=96, H=256, I=512)
    layer = O.make_layer(cfg, seed=0)
    per = cfg["E"] // world
    sl = slice(rank * per, (rank + 1) * per)
    d = lambda t: None if t is None else t[sl].to(dev)  # noqa: E731
    moe = XpuFusedMoe(d(layer["w13"]), d(layer["w13_scale"]), None, d(layer["w2"]), d(layer["w2_scale"]),
                      None, cfg["k"], "silu", per)
    if backend in ("token", "wave"):
        from vllm_xpu_kernels.ep import TokenExpertParallel, WaveExpertParallel
        fp8 = recipe == "fp8block"
        cls = TokenExpertParallel if backend == "token" else WaveExpertParallel
        ep = cls(dist.group.WORLD, moe, cfg["T"], cfg["k"], cfg["H"],
                 cfg["H"] * (1 if fp8 else 2), (cfg["H"] // 128) * 4 if fp8 else 0, per, dev)
    elif backend.startswith("peer"):
        from vllm_xpu_kernels.ep import PeerExpertParallel
        fp8 = recipe == "fp8block"
        ep = PeerExpertParallel(dist.group.WORLD, moe, cfg["T"], cfg["k"], cfg["H"],
                                cfg["H"] * (1 if fp8 else 2), (cfg["H"] // 128) * 4 if fp8 else 0, per, dev,
                                combine=backend.split("-")[1])
    else:
        ep = ExpertParallel(dist.group.WORLD, per, make_local_fn(moe))
    ok = True
    for call in range(2):   # twice: the exchange buffers are reused from call to call
        tok = O.make_layer(dict(cfg, E=cfg["E"]), seed=50 + rank + 10 * call, E_limit=1)
        x, logits = tok["x"], tok["logits"]
        w, ids = O.topk_softmax(logits, cfg["k"], True)
        out = torch.empty(cfg["T"], cfg["H"], dtype=torch.bfloat16, device=dev)
        xd, scales = x.to(dev), None
        if recipe == "fp8block":
            xd, scales = quant_fp8_block_act(xd)
        ep.apply(out, xd, w.to(dev), ids.to(dev), scales=scales)
        torch.cuda.synchronize()
        ref = O.fused_moe(recipe, x, layer["w13"], layer["w13_scale"], None, layer["w2"], layer["w2_scale"],
                          None, w, ids, "silu", out_dtype=torch.float32)
        err = (out.float().cpu() - ref).abs()
        tol = 2e-2
        ok = ok and bool((err <= tol + tol * ref.abs()).all())
    ok = ok and torch.ops._xpu_C.b200_device_status() == 0
    result[rank] = ok
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("backend", ["nccl", "peer-pull", "peer-push", "token", "wave"])
@pytest.mark.parametrize("recipe", ["bf16", "fp8block"])
def test_expert_parallel_two_gpus(recipe, backend):
    """backend 'nccl': all-to-all-v through torch.distributed; 'peer-*': this library's kernels
    storing into the other GPU's memory for the dispatch, and for the combine either the
    token's owner reading the result rows from the peers ('pull') or the second GEMM's
    epilogue storing them into the sender's memory ('push'); 'token': one row per (token, rank)
    out, the receiving rank's ordinary local layer, one partial sum per (token, rank) back;
    'wave': the same in two waves of tokens on two streams."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29621 + 5 * (recipe != "bf16") + ["nccl", "peer-pull", "peer-push", "token", "wave"].index(backend)
    with mp.Manager() as m:
        result = m.dict()
        mp.spawn(_worker, args=(2, port, recipe, backend, result), nprocs=2, join=True)
        assert result[0] and result[1]


def _barrier_worker(rank, world, port, result):
    for p in (ROOT, PKG_DIR):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import ctypes

    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from vllm_xpu_kernels import capi
    lib = capi.lib()
    n = 1 << 20
    buf = symm_mem.empty(4096 + n * 4, dtype=torch.uint8, device=dev)
    hdl = symm_mem.rendezvous(buf, dist.group.WORLD.group_name)
    buf.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    bases = (ctypes.c_int64 * world)(*[int(p) for p in hdl.buffer_ptrs])
    epochs = torch.zeros(capi.EP_BARRIER_CHANNELS, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream

    def barrier(ch, budget=0):
        assert lib.b200moe_ep_barrier(bases, 0, rank, world, ch, epochs.data_ptr(), budget, st) == capi.OK

    def status():
        s = ctypes.c_int(0)
        assert lib.b200moe_device_status(st, ctypes.byref(s)) == capi.OK
        return s.value

    ok = True
    # (1) ordering: write into the peer's memory, barrier, read what the peer wrote into mine
    mine = buf[4096:].view(torch.int32)
    peer = hdl.get_buffer((rank + 1) % world, (n,), torch.int32, 1024)
    for it in range(3):
        peer.copy_(torch.arange(n, dtype=torch.int32, device=dev) + (rank + 1) * 1000 + it)
        barrier(0)
        src = (rank - 1) % world
        ok = ok and bool((mine == torch.arange(n, dtype=torch.int32, device=dev) + (src + 1) * 1000 + it).all())
        barrier(0)   # nobody overwrites a buffer that is still being checked
    ok = ok and status() == 0
    # (2) a rank that skips a barrier: the other one gives up after its budget and says so
    dist.barrier()
    if rank == 0:
        barrier(1, 50_000_000)
        ok = ok and status() == capi.TIMEOUT
    torch.cuda.synchronize()
    dist.barrier()          # the skipped barrier is over on rank 0 before rank 1 goes on
    if rank != 0:
        barrier(1, 50_000_000)      # late: the flag of rank 0 is already there
        ok = ok and status() == 0
    barrier(1, 5_000_000_000)
    ok = ok and status() == 0 and epochs.cpu().tolist()[:2] == [6, 2]
    result[rank] = ok
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def test_bounded_barrier_two_gpus():
    """The library's cross-rank barrier between two processes with a GPU each: it orders peer
    writes, and when one rank does not call it the other returns after its budget with
    B200MOE_TIMEOUT in the status word.  No rank exits or faults; the failure is played by
    the host skipping a call between steps."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with mp.Manager() as m:
        result = m.dict()
        mp.spawn(_barrier_worker, args=(2, 29641, result), nprocs=2, join=True)
        assert result[0] and result[1]
