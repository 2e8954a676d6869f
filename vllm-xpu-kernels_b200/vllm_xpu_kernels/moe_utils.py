"""Quantisation helpers of the fused-MoE path.

Same names and argument meaning as vllm_xpu_kernels/moe_utils.py of the
reference project; the quantising functions call the CUDA operators, the
de-quantising ones are plain tensor arithmetic on whatever device the input
lives on.
"""
import torch

from . import _C  # noqa: F401
from . import _moe_C  # noqa: F401
from . import _xpu_C  # noqa: F401

finfo = torch.finfo(torch.float8_e4m3fn)
FP8_E4M3_MIN = finfo.min
FP8_E4M3_MAX = finfo.max

_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def _as_e8m0(s):
    return s.view(torch.float8_e8m0fnu) if s.dtype == torch.uint8 else s


def dequant_mxfp4(x_lp, x_scale):
    """[..., n] packed e2m1 pairs with one scale per 32 values -> fp32 [..., 2n]."""
    u8 = x_lp.view(torch.uint8)
    lut = torch.tensor(_E2M1, dtype=torch.float32, device=u8.device)
    vals = torch.stack((lut[(u8 & 0xF).long()], lut[(u8 >> 4).long()]), dim=-1).flatten(-2)
    out = vals.reshape(-1, 32) * x_scale.reshape(-1, 1).to(torch.float32)
    return out.reshape(u8.shape[:-1] + (u8.shape[-1] * 2,))


def dequant_mxfp8(x_lp, x_scale):
    out = x_lp.to(torch.float32).reshape(-1, 32) * x_scale.reshape(-1, 1).to(torch.float32)
    return out.reshape(x_lp.shape)


def dequant_fp8_block_wei(x_lp, x_scale):
    K, N = x_lp.shape
    x = x_lp.to(torch.float32).view(K // 128, 128, N // 128, 128)
    return (x * x_scale.unsqueeze(1).unsqueeze(-1)).reshape(K, N)


def dequant_fp8_block_act(x_lp, x_scale):
    shape = x_lp.shape
    x = x_lp.reshape(shape[0], shape[-1] // 128, 128).to(torch.float32)
    return (x * x_scale.unsqueeze(-1)).reshape(shape)


def quant_fp8_block_act(x: torch.Tensor, pow2_scales: bool = False):
    """Per-token-group-128 FP8 quantisation -> (e4m3 [M, K], f32 [M, K/128]).  With
    ``pow2_scales`` every scale is rounded up to a power of two (the operator's scale_ue8m0
    flag), which is what a layer whose weight scales are powers of two wants
    (``XpuFusedMoe.act_scales_pow2``)."""
    x_q = torch.empty(x.shape, device=x.device, dtype=torch.float8_e4m3fn)
    x_s = torch.empty(x.shape[:-1] + (x.shape[-1] // 128,), device=x.device, dtype=torch.float32)
    torch.ops._C.per_token_group_fp8_quant(x, x_q, x_s, 128, 1e-10, FP8_E4M3_MIN, FP8_E4M3_MAX,
                                           bool(pow2_scales), False, False)
    return x_q, x_s


def requant_fp8_block_weights_pow2_(w: torch.Tensor, scales: torch.Tensor) -> None:
    """In place: block-FP8 weights [E, K, N] (e4m3) with 128x128 fp32 scales [E, K/128, N/128] are
    re-expressed with every scale rounded UP to a power of two, the elements re-rounded to e4m3
    against the new scale (value * old / new, at most a factor two smaller, so nothing
    saturates).  A load-time step for checkpoints whose scales are arbitrary fp32 numbers: the
    layer can then let the tensor core apply the scales.  Not exact -- each element is rounded
    to e4m3 a second time -- which is why it is opt-in (B200MOE_FP8_REQUANT_POW2=1)."""
    E, K, N = w.shape
    assert K % 128 == 0 and N % 128 == 0 and scales.shape == (E, K // 128, N // 128)
    for e in range(E):  # one expert at a time: the fp32 copy of one expert is all that is held
        old = scales[e].float()
        m, ex = torch.frexp(old)                      # old = m * 2^ex, m in [0.5, 1)
        new = torch.ldexp(torch.ones_like(old), torch.where(m == 0.5, ex - 1, ex))
        ratio = (old / new).view(K // 128, 1, N // 128, 1)
        blk = w[e].float().view(K // 128, 128, N // 128, 128) * ratio
        w[e].copy_(blk.view(K, N).to(torch.float8_e4m3fn))
        scales[e].copy_(new)


def _quant_mxfp8_act_xpu(x):
    assert x.shape[-1] % 32 == 0
    x_q = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    x_s = torch.empty(x.shape[:-1] + (x.shape[-1] // 32,), device=x.device, dtype=torch.float32)
    torch.ops._C.per_token_group_fp8_quant(x, x_q, x_s, 32, 1e-10, FP8_E4M3_MIN, FP8_E4M3_MAX,
                                           True, False, False)
    return x_q, x_s.to(torch.float8_e8m0fnu)


def _quant_mxfp4_act_xpu(x):
    M, N = x.shape
    x_q = torch.empty(M, N // 2, device=x.device, dtype=torch.uint8)
    x_s = torch.empty(M, N // 32, device=x.device, dtype=torch.float32)
    torch.ops._C.per_token_group_quant_mxfp4(x, x_q, x_s, 32, 1e-10)
    return x_q.view(torch.float4_e2m1fn_x2), x_s.to(torch.float8_e8m0fnu)


def quant_mxfp_act_xpu(x, recipe):
    assert recipe in ("mxfp8", "mxfp4")
    return _quant_mxfp8_act_xpu(x) if recipe == "mxfp8" else _quant_mxfp4_act_xpu(x)


def quant_act_xpu(x, recipe):
    if recipe in ("mxfp4", "mxfp8"):
        return quant_mxfp_act_xpu(x, recipe)
    if recipe == "fp8block":
        return quant_fp8_block_act(x)
    raise NotImplementedError(f"Unsupported recipe for quant_act_xpu: {recipe}")


def dequant_act(x, x_scale, recipe):
    if recipe == "fp8block":
        return dequant_fp8_block_act(x, x_scale)
    if recipe == "mxfp4":
        return dequant_mxfp4(x, _as_e8m0(x_scale))
    if recipe == "mxfp8":
        return dequant_mxfp8(x, _as_e8m0(x_scale))
    return x


def dequant_wei(wei, wei_scale, recipe):
    if recipe in ("mxfp4", "mxfp4_fp8"):
        return dequant_mxfp4(wei, _as_e8m0(wei_scale))
    if recipe == "fp8block":
        return dequant_fp8_block_wei(wei, wei_scale)
    if recipe == "fp8":
        return wei.float() * wei_scale.float()
    return wei
