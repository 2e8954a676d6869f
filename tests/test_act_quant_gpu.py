"""Gated activations and activation quantisation against the CPU oracle."""
import pytest
import torch

from conftest import as_bf16, load_golden
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("R,d", [(1, 64), (24, 256), (333, 2880), (128, 14336), (7, 13)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_silu_and_mul(ops, R, d, dtype):
    x = (torch.randn(R, 2 * d, generator=torch.Generator().manual_seed(d)) * 2).to(dtype)
    out = torch.empty(R, d, dtype=dtype, device=DEV)
    ops._C.silu_and_mul(out, x.to(DEV))
    tol = 1e-3 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.cpu().float(), O.silu_and_mul(x).float(), atol=tol, rtol=tol)


def test_activations_golden(ops):
    g = load_golden("act")
    x = as_bf16(g["x"])
    out = torch.empty(x.shape[0], x.shape[1] // 2, dtype=torch.bfloat16, device=DEV)
    ops._C.silu_and_mul(out, x.to(DEV))
    assert torch.allclose(out.cpu().float(), as_bf16(g["silu"]).float(), atol=2e-2, rtol=2e-2)
    ops._C.swigluoai_and_mul(out, x.to(DEV), 1.702, 7.0)
    assert torch.allclose(out.cpu().float(), as_bf16(g["oai"]).float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("R,d", [(1, 32), (100, 2880), (4096, 512)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swigluoai_and_mul(ops, R, d, dtype):
    x = (torch.randn(R, 2 * d, generator=torch.Generator().manual_seed(d)) * 4).to(dtype)
    out = torch.empty(R, d, dtype=dtype, device=DEV)
    ops._C.swigluoai_and_mul(out, x.to(DEV), 1.702, 7.0)
    ref = O.swigluoai_and_mul(x.float())
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.cpu().float(), ref, atol=tol, rtol=tol)


@pytest.mark.parametrize("R,N,gs", [(1, 128, 128), (16, 512, 128), (4096, 4096, 128), (333, 7168, 128),
                                    (64, 2880, 32), (50, 256, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("ue8m0", [False, True])
def test_per_token_group_fp8_quant(ops, R, N, gs, dtype, ue8m0):
    x = (torch.randn(R, N, generator=torch.Generator().manual_seed(N)) * 3).to(dtype)
    x[0, :gs] = 0          # an all-zero group exercises the scale floor
    rq, rs = O.per_token_group_fp8_quant(x, gs, 1e-10, ue8m0)
    q = torch.empty(R, N, dtype=torch.float8_e4m3fn, device=DEV)
    s = torch.empty(R, N // gs, dtype=torch.float32, device=DEV)
    ops._C.per_token_group_fp8_quant(x.to(DEV), q, s, gs, 1e-10, -448.0, 448.0, ue8m0, False, False)
    assert torch.equal(s.cpu(), rs)
    assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
    # column-major scales (what a TMA-aligned caller passes)
    st = torch.empty(N // gs, R, dtype=torch.float32, device=DEV).t()
    ops._C.per_token_group_fp8_quant(x.to(DEV), q, st, gs, 1e-10, -448.0, 448.0, ue8m0, False, False)
    assert torch.equal(st.cpu(), rs)


def test_fp8_group_quant_golden(ops):
    g = load_golden("fp8_group")
    q = torch.empty(16, 512, dtype=torch.float8_e4m3fn, device=DEV)
    s = torch.empty(16, 4, dtype=torch.float32, device=DEV)
    ops._C.per_token_group_fp8_quant(g["x"].to(DEV), q, s, 128, 1e-10, -448.0, 448.0, False, False, False)
    assert torch.allclose(s.cpu(), g["s"], atol=1e-2 * g["s"].max().item())
    deq = q.cpu().float().view(16, 4, 128) * s.cpu().unsqueeze(-1)
    ref = g["q"].view(torch.float8_e4m3fn).float().view(16, 4, 128) * g["s"].unsqueeze(-1)
    assert torch.allclose(deq, ref, atol=0.15, rtol=0.15)


@pytest.mark.parametrize("R,N", [(1, 32), (16, 256), (777, 2880)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_per_token_group_quant_mxfp4(ops, R, N, dtype):
    x = (torch.randn(R, N, generator=torch.Generator().manual_seed(N)) * 2).to(dtype)
    rq, rs = O.per_token_group_quant_mxfp4(x)
    q = torch.empty(R, N // 2, dtype=torch.uint8, device=DEV)
    s = torch.empty(R, N // 32, dtype=torch.float32, device=DEV)
    ops._C.per_token_group_quant_mxfp4(x.to(DEV), q, s, 32, 1e-10)
    assert torch.allclose(s.cpu(), rs, atol=0, rtol=1e-5)
    assert torch.equal(q.cpu(), rq)


def test_mxfp4_golden(ops):
    g = load_golden("mxfp4_ref")
    x = as_bf16(g["x"])
    q = torch.empty(16, 128, dtype=torch.uint8, device=DEV)
    s = torch.empty(16, 8, dtype=torch.float32, device=DEV)
    ops._C.per_token_group_quant_mxfp4(x.to(DEV), q, s, 32, 1e-10)
    assert torch.equal(s.cpu(), torch.exp2(g["s"].float() - 127.0))
    deq = (O.unpack_e2m1(q.cpu()).view(16, 8, 32) * s.cpu().unsqueeze(-1)).view(16, 256)
    # the reference oracle rounds exact midpoints to even, the operator towards zero:
    # at most one code step (<= 1.0 x scale) apart, and only at midpoints
    assert (deq - g["deq"]).abs().max() <= s.cpu().max()
    assert ((deq - g["deq"]).abs() > 0).float().mean() < 0.05


@pytest.mark.parametrize("R,d", [(1, 128), (64, 2048), (300, 14336)])
@pytest.mark.parametrize("ue8m0", [False, True])
def test_silu_and_mul_per_block_quant(ops, R, d, ue8m0):
    x = (torch.randn(R, 2 * d, generator=torch.Generator().manual_seed(d)) * 2).to(torch.bfloat16)
    rq, rs = O.silu_and_mul_per_block_quant(x, 128, ue8m0)
    q = torch.empty(R, d, dtype=torch.float8_e4m3fn, device=DEV)
    s = torch.empty(R, d // 128, dtype=torch.float32, device=DEV)
    ops._C.silu_and_mul_per_block_quant(q, x.to(DEV), s, 128, None, False, ue8m0)
    assert torch.allclose(s.cpu(), rs, rtol=1e-5, atol=0)
    # expf on the device and torch.exp on the host differ in the last bit now and then,
    # which can move a value across an e4m3 rounding boundary: rare, and never by more
    # than one code step (2^-3 relative)
    deq = q.cpu().float().view(R, -1, 128) * s.cpu().unsqueeze(-1)
    ref = rq.float().view(R, -1, 128) * rs.unsqueeze(-1)
    assert ((deq - ref).abs() <= 0.13 * ref.abs() + 2e-3 * rs.unsqueeze(-1)).all()
    assert (q.cpu().view(torch.uint8) != rq.view(torch.uint8)).float().mean() < 0.01


@pytest.mark.parametrize("R,d", [(8, 64), (100, 2880)])
def test_silu_and_mul_mxfp4_quant(ops, R, d):
    x = (torch.randn(R, 2 * d, generator=torch.Generator().manual_seed(d)) * 2).to(torch.bfloat16)
    rq, rs = O.silu_and_mul_mxfp4_quant(x)
    q = torch.empty(R, d // 2, dtype=torch.uint8, device=DEV)
    s = torch.empty(R, d // 32, dtype=torch.float32, device=DEV)
    ops._C.silu_and_mul_mxfp4_quant(q, x.to(DEV), s, 32, 1e-10)
    assert torch.allclose(s.cpu(), rs, rtol=1e-5, atol=0)
    deq = O.unpack_e2m1(q.cpu()).view(R, -1, 32) * s.cpu().unsqueeze(-1)
    ref = O.unpack_e2m1(rq).view(R, -1, 32) * rs.unsqueeze(-1)
    assert torch.allclose(deq, ref, atol=0.5, rtol=0)
    assert (q.cpu() != rq).float().mean() < 0.01
