"""b200moe_moe_align_block_size_static: the variant of moe_align_block_size for hosts
that may not allocate device memory around the call (a server that gave all of HBM to
its own pools, a plug-in contract that bans cudaMalloc on the request path).  Its
scratch is an array built into the library, so this checks, through the C ABI, that it
gives exactly what the workspace-taking entry point gives — twice in a row, the second
call on a smaller problem so stale scratch contents would show."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(lib, capi, fn_static, ids, E, bs):
    numel = ids.numel()
    n, nb = O.align_sizes(numel, E, bs)
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for static in (False, True):
        s = torch.full((n,), -7, dtype=torch.int32, device=DEV)
        e = torch.full((nb,), -7, dtype=torch.int32, device=DEV)
        t = torch.full((1,), -7, dtype=torch.int32, device=DEV)
        if static:
            rc = fn_static(ids.data_ptr(), capi.I32, numel, E, bs, None, s.data_ptr(), n,
                           e.data_ptr(), nb, t.data_ptr(), stream)
        else:
            ws_bytes = lib.b200moe_moe_align_block_size_workspace_bytes(numel, E)
            ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=DEV)
            rc = lib.b200moe_moe_align_block_size(ids.data_ptr(), capi.I32, numel, E, bs, None,
                                                  s.data_ptr(), n, e.data_ptr(), nb, t.data_ptr(),
                                                  ws.data_ptr(), ws_bytes, stream)
        assert rc == capi.OK, (rc, lib.b200moe_last_error())
        torch.cuda.synchronize()
        outs.append((s.cpu(), e.cpu(), t.cpu()))
    return outs


def test_static_scratch_variant_matches_workspace_variant():
    from vllm_xpu_kernels import capi
    lib = capi.lib()
    fn = lib.b200moe_moe_align_block_size_static
    g = torch.Generator().manual_seed(3)
    for T, k, E, bs in ((4096, 8, 256, 128), (1500, 4, 64, 16)):   # 16 and 3 chunks of scratch
        ids = torch.randint(0, E, (T, k), generator=g).to(torch.int32).to(DEV)
        (s0, e0, t0), (s1, e1, t1) = _run(lib, capi, fn, ids, E, bs)
        assert torch.equal(t0, t1) and torch.equal(e0, e1) and torch.equal(s0, s1)
        rs, re, rt = O.moe_align_block_size(ids.cpu(), bs, E)
        assert torch.equal(s1, rs) and torch.equal(e1, re) and torch.equal(t1, rt)


def test_static_scratch_variant_rejects_oversized_problems():
    from vllm_xpu_kernels import capi
    lib = capi.lib()
    # ceil(numel/2048) * E = 300 * 1024 ints > 65536: refused before anything is launched
    rc = lib.b200moe_moe_align_block_size_static(None, capi.I32, 2048 * 300, 1024, 128, None, None, 0,
                                                 None, 0, None, None)
    assert rc == capi.WORKSPACE_TOO_SMALL
    assert b"exceeds the built-in scratch" in lib.b200moe_last_error()
