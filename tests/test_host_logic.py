"""Host-side pieces of the layer that need no GPU."""
import torch

from oracle import moe_oracle as O


def _blocks(E, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    q, s = zip(*[O.quant_fp8_block_weight(torch.randn(K, N, generator=g) / K ** 0.5) for _ in range(E)])
    return torch.stack(q), torch.stack(s)


def test_requantisation_to_power_of_two_block_scales():
    """moe_utils.requant_fp8_block_weights_pow2_: new scales are the old ones rounded up to a
    power of two, the weights move by at most one e4m3 rounding, nothing saturates, and a second
    application changes nothing (power-of-two scales are a fixed point)."""
    from vllm_xpu_kernels.moe_utils import requant_fp8_block_weights_pow2_
    E, K, N = 3, 384, 256
    q, s = _blocks(E, K, N, 5)
    s[0, 0, 0] = 2.0 ** -7           # an exact power of two stays as it is, with its weights
    q0, s0 = q.clone(), s.clone()
    requant_fp8_block_weights_pow2_(q, s)
    m, _ = torch.frexp(s)
    assert bool((m == 0.5).all())
    assert bool((s >= s0).all()) and bool((s < 2 * s0).all())
    assert torch.equal(q[0, :128, :128].view(torch.uint8), q0[0, :128, :128].view(torch.uint8))
    assert bool(torch.isfinite(q.float()).all()) and float(q.float().abs().max()) <= 448.0
    for e in range(E):
        w_old = O.dequant_expert_weight("fp8block", q0[e], s0[e])
        w_new = O.dequant_expert_weight("fp8block", q[e], s[e])
        # half a step of three mantissa bits, or half a subnormal step (2^-10 of the block's scale)
        step = 2.0 ** -10 * s[e].repeat_interleave(128, 0).repeat_interleave(128, 1)
        assert bool(((w_new - w_old).abs() <= 0.0625 * w_old.abs() + step).all())
    q1, s1 = q.clone(), s.clone()
    requant_fp8_block_weights_pow2_(q1, s1)
    assert torch.equal(s1, s) and torch.equal(q1.view(torch.uint8), q.view(torch.uint8))


def test_power_of_two_activation_format_of_the_oracle():
    """The oracle's "fp8_pow2" activation format (what a layer with power-of-two weight scales
    is compared against): scales are the fp32 ones rounded up to a power of two."""
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 256, generator=g)
    plain = O.qdq_act("fp8block", x)
    pow2 = O.qdq_act("fp8block", x, act_format="fp8_pow2")
    _, s_plain = O.per_token_group_fp8_quant(x, 128)
    _, s_pow2 = O.per_token_group_fp8_quant(x, 128, scale_ue8m0=True)
    m, _ = torch.frexp(s_pow2)
    assert bool((m == 0.5).all()) and bool((s_pow2 >= s_plain).all()) and bool((s_pow2 < 2 * s_plain).all())
    assert plain.shape == pow2.shape == x.shape
    # both are e4m3 roundings of x against a per-128 scale: within 2^-4 relative + a subnormal step
    for y in (plain, pow2):
        assert bool(((y - x).abs() <= 0.0625 * x.abs() + 2.0 ** -9 * x.abs().max()).all())
