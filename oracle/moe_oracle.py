"""CPU oracle for the fused Mixture-of-Experts path.  TEST INFRASTRUCTURE ONLY.

Every function here restates, with plain torch CPU ops, what the reference
project's own tests take as ground truth for one operator of the fused-MoE
path.  Nothing in the shipped package may import this module: it exists so
that the parity tests, the smoke check and the benchmark's CPU-baseline leg
have something independent to compare the CUDA kernels against.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the
reference's torch oracles (with its three native extension modules stubbed)
and stores their outputs on seeded inputs under ``tests/golden/*.npz``;
``tests/test_oracle_golden.py`` checks every function below against those
files, plus the worked example in the reference's align docstring
(tests/ops/moe_align_block_size_ops.py:56-69) and the FP4 code points of
tests/test_mxfp4_quant.py:113-142.

Citations are paths inside the reference project.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

FP8_MAX = 448.0
FP8_MIN_SCALE = 1.0 / (448.0 * 512.0)
E2M1_VALUES = torch.tensor(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
     -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=torch.float32)


# --------------------------------------------------------------------------
# routing
# --------------------------------------------------------------------------
def stable_topk(x: torch.Tensor, k: int):
    """Top-k by a stable descending sort: equal keys keep the lower index first
    (tests/ops/topk_op.py:11-13)."""
    v, i = torch.sort(x, dim=-1, descending=True, stable=True)
    return v[..., :k], i[..., :k]


def _finish_topk(scores, k, renormalize, bias, scale, is_padding):
    if bias is not None:
        _, ids = stable_topk(scores + bias.unsqueeze(0), k)
        w = scores.gather(1, ids)
    else:
        w, ids = stable_topk(scores, k)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    if scale is not None:
        w = w * scale
    if is_padding is not None:
        w = w.clone()
        ids = ids.clone()
        w[is_padding] = 0
        ids[is_padding] = -1
    return w.to(torch.float32), ids.to(torch.int32)


def topk_softmax(gating_output, topk, renormalize, bias=None, is_padding=None):
    """fp32 softmax, selection on score(+bias), weights without the bias
    (tests/ops/topk_op.py:16-41)."""
    scores = torch.softmax(gating_output, dim=-1, dtype=torch.float32)
    return _finish_topk(scores, topk, renormalize, bias, None, is_padding)


def topk_sigmoid(gating_output, topk, renormalize, bias=None,
                 routed_scaling_factor=1.0, is_padding=None):
    """Sigmoid in the input dtype, then as topk_softmax, then a final scale
    (tests/ops/topk_op.py:44-71)."""
    scores = torch.sigmoid(gating_output).to(torch.float32)
    return _finish_topk(scores, topk, renormalize, bias,
                        routed_scaling_factor, is_padding)


def topk_softplus_sqrt(gating_output, topk, renormalize, routed_scaling_factor=1.0, bias=None,
                       input_ids=None, hash_indices_table=None, is_padding=None):
    """sqrt(softplus(x)) scores in fp32; experts by stable top-k of score(+bias) or, with a
    hash table, looked up by the token's input id (tests/test_topk_softplus_sqrt.py:20-55)."""
    scores = torch.nn.functional.softplus(gating_output.float()).sqrt()
    if hash_indices_table is not None:
        ids = hash_indices_table[input_ids.long()]
    else:
        _, ids = stable_topk(scores + bias.unsqueeze(0) if bias is not None else scores, topk)
    w = scores.gather(1, ids.long())
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    if routed_scaling_factor != 1.0:
        w = w * routed_scaling_factor
    if is_padding is not None:
        w, ids = w.clone(), ids.clone()
        w[is_padding] = 0
        ids[is_padding] = -1
    return w.to(torch.float32), ids.to(torch.int32)


def token_expert_indices(num_tokens: int, topk: int) -> torch.Tensor:
    """Third output of topk_softmax/sigmoid: entry (t, j) = j*T + t
    (csrc/moe/topk.cpp:578)."""
    t = torch.arange(num_tokens, dtype=torch.int32).unsqueeze(1)
    j = torch.arange(topk, dtype=torch.int32).unsqueeze(0)
    return j * num_tokens + t


def grouped_topk(gating_output, topk, renormalize, num_expert_group,
                 topk_group, scoring_func="softmax", routed_scaling_factor=1.0,
                 e_score_correction_bias=None):
    """DeepSeek grouped routing (tests/ops/grouped_topk_op.py:16-68).

    Scores are taken in the input dtype; with a bias, a group's score is the
    sum of its two best biased scores, otherwise its maximum.  The best
    ``topk_group`` groups stay, everything else is masked to -inf, and the
    final top-k runs over the biased scores while the returned weights are the
    unbiased ones.
    """
    if scoring_func == "softmax":
        scores = torch.softmax(gating_output, dim=-1)
    elif scoring_func == "sigmoid":
        scores = torch.sigmoid(gating_output)
    elif scoring_func == "none":
        scores = gating_output
    else:
        raise ValueError(scoring_func)
    T, E = scores.shape
    per = E // num_expert_group
    original = scores
    if e_score_correction_bias is not None:
        scores = scores + e_score_correction_bias.unsqueeze(0)
        group_scores = stable_topk(scores.view(T, num_expert_group, per), 2)[0].sum(-1)
    else:
        group_scores = scores.view(T, num_expert_group, per).max(dim=-1).values
    _, gidx = stable_topk(group_scores, topk_group)
    gmask = torch.zeros_like(group_scores)
    gmask.scatter_(1, gidx, 1)
    smask = gmask.unsqueeze(-1).expand(T, num_expert_group, per).reshape(T, E)
    masked = scores.masked_fill(~smask.bool(), float("-inf"))
    if e_score_correction_bias is not None:
        _, ids = stable_topk(masked, topk)
        w = original.gather(1, ids)
    else:
        w, ids = stable_topk(masked, topk)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    w = w * routed_scaling_factor
    return w.to(torch.float32), ids.to(torch.int32)


def grouped_topk_kernel_semantics(gating_output, topk, renormalize, num_expert_group, topk_group,
                                  scoring_func, routed_scaling_factor, e_score_correction_bias):
    """grouped_topk with the three behaviours the reference's device kernel adds to its torch
    oracle (csrc/moe/grouped_topk.cpp): a row whose ``topk_group``-th best group score is -inf
    returns experts 0..k-1 with weight 1/k each (:608-624); experts whose raw score is +-inf
    are never selected although they count for their group's score (:659-662); the
    renormalising denominator is the sum + 1e-20 (:678-687).  On rows without such inputs it
    equals ``grouped_topk``."""
    if scoring_func == "sigmoid":
        scores = torch.sigmoid(gating_output)
    elif scoring_func == "none":
        scores = gating_output.clone()
    else:
        raise ValueError(scoring_func)
    T, E = scores.shape
    per = E // num_expert_group
    biased = scores + e_score_correction_bias.unsqueeze(0)
    group_scores = stable_topk(biased.view(T, num_expert_group, per), 2)[0].sum(-1)
    gval, gidx = stable_topk(group_scores, topk_group)
    degenerate = gval[:, -1] == float("-inf")
    gmask = torch.zeros_like(group_scores)
    gmask.scatter_(1, gidx, 1)
    smask = gmask.unsqueeze(-1).expand(T, num_expert_group, per).reshape(T, E).bool()
    masked = biased.masked_fill(~smask | torch.isinf(gating_output), float("-inf"))
    _, ids = stable_topk(masked, topk)
    w = scores.gather(1, ids)
    if renormalize:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    w = w * routed_scaling_factor
    ids = torch.where(degenerate.unsqueeze(1), torch.arange(topk).expand(T, topk), ids)
    w = torch.where(degenerate.unsqueeze(1), torch.full_like(w, 1.0 / topk), w)
    return w.to(torch.float32), ids.to(torch.int32)


def routing_margin(keys: torch.Tensor, k: int) -> torch.Tensor:
    """Per row: gap between the k-th and (k+1)-th largest selection key.  Rows
    whose gap is a few ulps are the only ones where two correct fp32
    implementations of the score may legitimately pick different experts."""
    v, _ = torch.sort(keys.float(), dim=-1, descending=True, stable=True)
    if v.shape[-1] <= k:
        return torch.full((v.shape[0],), float("inf"))
    return v[:, k - 1] - v[:, k]


# --------------------------------------------------------------------------
# permutation
# --------------------------------------------------------------------------
def align_sizes(numel: int, num_experts: int, block_size: int, pad_sorted_ids=False):
    """Buffer sizes the caller allocates (tests/ops/moe_align_block_size_ops.py:71-86)."""
    n = numel + num_experts * (block_size - 1)
    if pad_sorted_ids:
        n = (n + block_size - 1) // block_size * block_size
    if numel < num_experts:
        n = numel * block_size
    return n, (n + block_size - 1) // block_size


def moe_align_block_size(topk_ids, block_size, num_experts, expert_map=None,
                         pad_sorted_ids=False):
    """Stable grouping of flat (token, slot) indices by expert, each expert's
    run padded to ``block_size`` with the sentinel ``numel``
    (tests/test_moe_align_block_size.py:97-183).  ``expert_ids`` holds one
    (local) expert per block, 0 in the unused tail.  Experts mapped to -1 are
    dropped; ids >= num_experts are ignored.  With an ``expert_map`` the runs are
    keyed and ordered by the MAPPED id, which is what the reference kernel does
    (csrc/moe/moe_align_sum_kernels.cpp:196-205: ``expert_id =
    expert_map[expert_id]`` before counting).  The reference's torch golden walks
    the global ids instead (tests/test_moe_align_block_size.py:156-176); the two
    agree for every map whose kept entries are increasing - all its tests use -
    and differ only for a permuted map, where this follows the kernel."""
    numel = topk_ids.numel()
    max_padded, max_blocks = align_sizes(numel, num_experts, block_size, pad_sorted_ids)
    flat = topk_ids.flatten().to(torch.int64)
    valid = (flat >= 0) & (flat < num_experts)
    if expert_map is not None:
        mapped = expert_map.to(torch.int64)[flat.clamp(0, num_experts - 1)]
        valid &= (mapped >= 0) & (mapped < num_experts)
        flat = torch.where(valid, mapped, flat)     # the key is the mapped id
    counts = torch.bincount(flat[valid], minlength=num_experts)
    padded = (counts + block_size - 1) // block_size * block_size
    starts = torch.cumsum(padded, 0) - padded
    sorted_ids = torch.full((max_padded,), numel, dtype=torch.int32)
    expert_ids = torch.zeros(max_blocks, dtype=torch.int32)
    order = torch.sort(torch.where(valid, flat, torch.full_like(flat, num_experts)),
                       stable=True).indices
    order = order[: int(valid.sum())]
    e_sorted = flat[order]
    rank = torch.arange(order.numel()) - (torch.cumsum(counts, 0) - counts)[e_sorted]
    sorted_ids[(starts[e_sorted] + rank)] = order.to(torch.int32)
    blocks = padded // block_size
    owner = torch.repeat_interleave(torch.arange(num_experts), blocks)
    expert_ids[: owner.numel()] = owner.to(torch.int32)
    total = torch.tensor([int(padded.sum())], dtype=torch.int32)
    return sorted_ids, expert_ids, total


def moe_lora_align_block_size(topk_ids, token_lora_mapping, num_experts, block_size, max_loras,
                              max_num_tokens_padded, max_num_m_blocks, sorted_token_ids,
                              expert_ids, num_tokens_post_pad, adapter_enabled, lora_ids,
                              expert_map=None):
    """One alignment per enabled adapter slot, written into that slot's rows of the
    caller's (pre-filled) flat outputs; other rows stay as they are
    (csrc/moe/moe_align_sum_kernels.cpp:803-848 for the slot guards and the token mask,
    :136-277 for the alignment with inactive blocks labelled -1).  With an expert_map the
    entries are grouped by the mapped id.  Inside an expert the order is ascending flat
    index (the reference's is whatever its atomics give; its test checks membership only)."""
    numel = topk_ids.numel()
    k = topk_ids.shape[1]
    sorted_token_ids = sorted_token_ids.clone().view(max_loras, -1)
    expert_ids = expert_ids.clone().view(max_loras, -1)
    num_tokens_post_pad = num_tokens_post_pad.clone()
    for s in lora_ids[: max_loras + 1].tolist():
        if s < 0 or s >= max_loras or int(adapter_enabled[s]) == 0:
            continue
        ids = topk_ids.to(torch.int64).clone()
        if expert_map is not None:
            ok = (ids >= 0) & (ids < num_experts)
            mapped = expert_map.to(torch.int64)[ids.clamp(0, num_experts - 1)]
            ids = torch.where(ok & (mapped >= 0), mapped, torch.full_like(ids, num_experts))
        ids[token_lora_mapping != s] = num_experts          # ignored by the alignment
        srt, eid, tot = moe_align_block_size(ids, block_size, num_experts)
        n = min(srt.numel(), max_num_tokens_padded)
        row = torch.full((max_num_tokens_padded,), numel, dtype=torch.int32)
        row[:n] = srt[:n]
        sorted_token_ids[s, :max_num_tokens_padded] = row
        used = int(tot) // block_size
        blocks = torch.full((max_num_m_blocks,), -1, dtype=torch.int32)
        blocks[:used] = eid[:used]
        expert_ids[s, :max_num_m_blocks] = blocks
        num_tokens_post_pad[s] = int(tot)
    return sorted_token_ids.flatten(), expert_ids.flatten(), num_tokens_post_pad


def batched_moe_align_block_size(max_tokens_per_batch, block_size, expert_num_tokens):
    """Batch b owns token slots [b*max, b*max + n_b); runs padded to the block size, sentinel
    B*max, unused blocks -1 (tests/test_moe_align_block_size.py:346-392)."""
    B = expert_num_tokens.numel()
    per = (max_tokens_per_batch + block_size - 1) // block_size * block_size
    sorted_ids = torch.full((per * B,), B * max_tokens_per_batch, dtype=torch.int32)
    block_ids = torch.full((per * B // block_size,), -1, dtype=torch.int32)
    pos = 0
    for b, n in enumerate(expert_num_tokens.tolist()):
        sorted_ids[pos: pos + n] = torch.arange(n, dtype=torch.int32) + b * max_tokens_per_batch
        nb = (n + block_size - 1) // block_size
        block_ids[pos // block_size: pos // block_size + nb] = b
        pos += nb * block_size
    return sorted_ids, block_ids, torch.tensor([pos], dtype=torch.int32)


def reorder_mxfp_scales(scales_u8, rows_per_expert, total_padded_rows):
    """Per expert: [rows, scale_k] -> [scale_k, rows padded to 4], blocks back to back, zero
    tail (tests/fused_moe/test_reorder_mxfp_scales.py:26-43)."""
    scale_k = scales_u8.shape[1]
    out = torch.zeros((total_padded_rows, scale_k), dtype=torch.uint8)
    src = dst = 0
    for r in rows_per_expert.tolist():
        pr = (r + 3) & ~3
        if r:
            out[dst: dst + pr].view(scale_k, pr)[:, :r] = scales_u8[src: src + r].t()
        src += r
        dst += pr
    return out


def init_expert_map(num_local_experts: int, ep_rank: int, ep_size: int):
    """Global id -> local id inside this rank's window, -1 outside
    (csrc/moe/init_expert_map.cpp:45-52)."""
    m = torch.full((num_local_experts * ep_size,), -1, dtype=torch.int32)
    lo = ep_rank * num_local_experts
    m[lo: lo + num_local_experts] = torch.arange(num_local_experts, dtype=torch.int32)
    return m


def remap_hidden_states(hidden_states, scales, topk_ids, expert_map,
                        local_experts_num):
    """Stable permutation of token rows into expert-contiguous order
    (tests/fused_moe/test_remap_hidden_states.py:39-84): row of (t, j) =
    prefix[e] + number of earlier (t', j') in row-major order with the same
    local expert; non-local pairs get -1.

    Returns (remapped, remapped_scales, rows_per_expert, row_map)."""
    T, k = topk_ids.shape
    ids = topk_ids.to(torch.int64)
    local = expert_map.to(torch.int64)[ids] if expert_map is not None else ids
    flat = local.flatten()
    valid = flat >= 0
    counts = torch.bincount(flat[valid], minlength=local_experts_num)
    prefix = torch.cumsum(counts, 0) - counts
    order = torch.sort(torch.where(valid, flat, torch.full_like(flat, local_experts_num)),
                       stable=True).indices[: int(valid.sum())]
    row_map = torch.full((T * k,), -1, dtype=torch.int32)
    row_map[order] = torch.arange(order.numel(), dtype=torch.int32)
    src_token = order // k
    remapped = torch.zeros((T * k, hidden_states.shape[1]), dtype=hidden_states.dtype)
    view = remapped.view(torch.uint8) if remapped.dtype.itemsize == 1 else remapped
    src = hidden_states.view(torch.uint8) if hidden_states.dtype.itemsize == 1 else hidden_states
    view[: order.numel()] = src[src_token]
    rs = None
    if scales is not None:
        s = scales.view(torch.uint8) if scales.dtype.itemsize == 1 else scales
        rs_ = torch.zeros((T * k, scales.shape[1]), dtype=s.dtype)
        rs_[: order.numel()] = s[src_token]
        rs = rs_.view(scales.dtype)
    return remapped, rs, counts.to(torch.int32), row_map.view(T, k)


def moe_gather(moe_output, topk_weights, row_map, out_dtype=None):
    """out[t] = sum_j w[t,j] * y[row_map[t,j]] in fp32, skipping -1 rows
    (tests/test_moe_gather.py:27-42)."""
    T, k = topk_weights.shape
    acc = torch.zeros((T, moe_output.shape[1]), dtype=torch.float32)
    for j in range(k):
        idx = row_map[:, j].to(torch.int64)
        w = topk_weights[:, j] * (idx >= 0)
        acc += moe_output[idx.clamp_min(0)].float() * w[:, None]
    return acc.to(out_dtype or moe_output.dtype)


def moe_sum(inp, topk_ids=None, expert_map=None):
    """out[t] = sum_k in[t,k] in fp32; with ids, slots whose id is negative or
    maps to -1 are left out (tests/test_moe_sum.py:24-101)."""
    x = inp.float()
    if topk_ids is not None:
        ids = topk_ids.to(torch.int64)
        keep = ids >= 0
        if expert_map is not None:
            keep &= expert_map.to(torch.int64)[ids.clamp_min(0)] >= 0
        x = x * keep.unsqueeze(-1)
    return x.sum(1).to(inp.dtype)


# --------------------------------------------------------------------------
# gated activations and activation quantisation
# --------------------------------------------------------------------------
def silu_and_mul(x):
    """silu(first half) * second half (tests/ops/activation_op.py:22-25)."""
    d = x.shape[-1] // 2
    return torch.nn.functional.silu(x[..., :d]) * x[..., d:]


def swigluoai_and_mul(x, alpha=1.702, limit=7.0):
    """gpt-oss gate: even columns gate, odd columns up
    (tests/ops/swigluoai_and_mul_op.py:24-32)."""
    g = x[..., ::2].clamp(max=limit)
    u = x[..., 1::2].clamp(min=-limit, max=limit)
    return (u + 1) * (g * torch.sigmoid(g * alpha))


def gelu_and_mul(x, approximate="none"):
    """gelu(first half) * second half (tests/ops/activation_op.py:83-86)."""
    d = x.shape[-1] // 2
    return torch.nn.functional.gelu(x[..., :d], approximate=approximate) * x[..., d:]


def relu2_no_mul(x):
    """relu(x)^2 over every column (tests/ops/activation_op.py:188-190)."""
    return torch.square(torch.relu(x))


def swiglustep_and_mul(x, limit=7.0):
    """min(silu(gate), limit) * clamp(up, +-limit), fp32 inside
    (csrc/activation.cpp:297-311; tests/ops/swiglustep_and_mul_op.py)."""
    d = x.shape[-1] // 2
    g, u = x[..., :d].float(), x[..., d:].float()
    return (torch.nn.functional.silu(g).clamp(max=limit) * u.clamp(-limit, limit)).to(x.dtype)


def situ_and_mul(x, beta, linear_beta=-1.0):
    """beta*tanh(gate/beta)*sigmoid(gate) * (linear_beta*tanh(up/linear_beta) or up), fp32
    inside (tests/test_activation.py:98-103)."""
    g, u = x.float().chunk(2, dim=-1)
    g = beta * torch.tanh(g / beta) * torch.sigmoid(g)
    if linear_beta > 0:
        u = linear_beta * torch.tanh(u / linear_beta)
    return (g * u).to(x.dtype)


def layer_activation(h, activation, situ_beta=None, situ_linear_beta=None):
    """fp32 activation step of the layer oracle, by the names XpuFusedMoe takes
    (vllm_xpu_kernels/fused_moe_interface.py:133-154 and :452-464 for the situ arguments)."""
    if activation == "silu":
        return silu_mul_fp32(h)
    if "swigluoai" in str(activation).lower():
        return swigluoai_and_mul(h)
    if activation == "gelu":
        return gelu_and_mul(h)
    if activation == "gelu_tanh":
        return gelu_and_mul(h, "tanh")
    if activation == "relu2_no_mul":
        return relu2_no_mul(h)
    if activation == "swiglustep":
        return swiglustep_and_mul(h, 7.0)
    if activation == "situ":
        return situ_and_mul(h, situ_beta, -1.0 if situ_linear_beta is None else situ_linear_beta)
    raise ValueError(activation)


def per_token_group_fp8_quant(x, group_size=128, eps=1e-10, scale_ue8m0=False,
                              divide=False):
    """scale = max(max(eps, amax)/448, 1/(448*512)), optionally rounded up to a
    power of two; q = e4m3(clamp(x * (1/scale))) — or x / scale when
    ``divide`` (csrc/quantization/fp8/fp8_quant.cpp:238-252,
    quant_utils.h:61-71; the fused SiLU kernel divides,
    fused_silu_mul_block_quant.cpp:118-119)."""
    M, N = x.shape
    g = x.float().view(M, N // group_size, group_size)
    amax = g.abs().amax(-1).clamp_min(eps)
    s = torch.maximum(amax / FP8_MAX, torch.tensor(FP8_MIN_SCALE))
    if scale_ue8m0:
        s = torch.exp2(torch.ceil(torch.log2(s.abs().clamp_min(1e-10))))
    y = g / s.unsqueeze(-1) if divide else g * (1.0 / s).unsqueeze(-1)
    q = y.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(M, N)
    return q, s


def quant_mxfp8_act(x):
    """MXFP8 activations the way the reference quantises them
    (vllm_xpu_kernels/moe_utils.py:84-109: per_token_group_fp8_quant with group
    32 and scale_ue8m0, the scale then cast to e8m0): (e4m3 [M, N], e8m0 bytes
    u8 [M, N/32])."""
    q, s = per_token_group_fp8_quant(x, 32, scale_ue8m0=True)
    return q, (torch.log2(s).round().to(torch.int32) + 127).to(torch.uint8)


def dequant_mxfp8_act(q, sf_u8):
    """(vllm_xpu_kernels/moe_utils.py:71-75) fp32 = e4m3 * 2^(byte - 127) per 32 columns."""
    M, N = q.shape
    return (q.float().view(M, N // 32, 32) * e8m0_to_f32(sf_u8[:, :N // 32]).unsqueeze(-1)).view(M, N)


def e2m1_code(x: torch.Tensor) -> torch.Tensor:
    """4-bit code of the nearest e2m1 value; a value exactly between two
    code points goes to the smaller magnitude (strict '>' compares,
    csrc/quantization/fp4/mxfp4_quant.h:17-28)."""
    a = x.abs()
    code = torch.zeros_like(a, dtype=torch.uint8)
    for b in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        code += (a > b).to(torch.uint8)
    return code | ((x < 0).to(torch.uint8) << 3)


def per_token_group_quant_mxfp4(x, group_size=32, eps=1e-10):
    """scale = 2^ceil(log2(max(amax/6, eps))) as fp32; q = e2m1(clamp(x/scale,
    ±6)); byte i = code[2i+1] << 4 | code[2i]
    (csrc/quantization/fp4/mxfp4_quant.h:104-130)."""
    M, N = x.shape
    g = x.float().view(M, N // group_size, group_size)
    amax = g.abs().amax(-1).clamp_min(eps)
    s = torch.exp2(torch.ceil(torch.log2((amax / 6.0).abs().clamp_min(eps))))
    y = (g * (1.0 / s).unsqueeze(-1)).clamp(-6.0, 6.0)
    c = e2m1_code(y).view(M, N)
    packed = (c[:, 1::2] << 4) | c[:, 0::2]
    return packed, s


def silu_mul_fp32(x):
    d = x.shape[-1] // 2
    g = x[..., :d].float()
    return (g / (1.0 + torch.exp(-g))) * x[..., d:].float()


def silu_and_mul_per_block_quant(x, group_size=128, scale_ue8m0=False):
    """fp32 silu(g)*u with no intermediate rounding, then group quant dividing
    by the scale (fused_kernels/fused_silu_mul_block_quant.cpp:71-119)."""
    y = silu_mul_fp32(x)
    M, N = y.shape
    g = y.view(M, N // group_size, group_size)
    s = torch.maximum(g.abs().amax(-1) / FP8_MAX, torch.tensor(FP8_MIN_SCALE))
    if scale_ue8m0:
        s = torch.exp2(torch.ceil(torch.log2(s.abs().clamp_min(1e-10))))
    q = (g / s.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(M, N), s


def silu_and_mul_mxfp4_quant(x, group_size=32, eps=1e-10):
    """fp32 silu(g)*u then MXFP4 group quant
    (fused_kernels/fused_silu_mul_mxfp4_quant.cpp:19-131)."""
    return per_token_group_quant_mxfp4(silu_mul_fp32(x), group_size, eps)


# --------------------------------------------------------------------------
# weight formats
# --------------------------------------------------------------------------
def unpack_e2m1(packed_u8: torch.Tensor) -> torch.Tensor:
    """[..., n] bytes -> [..., 2n] fp32; low nibble is the even element
    (vllm_xpu_kernels/moe_utils.py:12-62)."""
    lo = E2M1_VALUES[(packed_u8 & 0xF).long()]
    hi = E2M1_VALUES[(packed_u8 >> 4).long()]
    return torch.stack((lo, hi), dim=-1).flatten(-2)


def e8m0_to_f32(s_u8: torch.Tensor) -> torch.Tensor:
    """2^(b-127) (csrc/xpu/grouped_gemm/xe_2/gemm_xe2.hpp:426-434)."""
    return torch.exp2(s_u8.to(torch.float32) - 127.0)


def dequant_mxfp4(w_u8, s_u8):
    """[N, K/2] bytes + [N, K/32] e8m0 -> [N, K] fp32 (moe_utils.py:65-69)."""
    v = unpack_e2m1(w_u8)
    return (v.view(*v.shape[:-1], -1, 32) * e8m0_to_f32(s_u8).unsqueeze(-1)).view(v.shape)


def dequant_fp8_block(w, s, block=128):
    """[K, N] e4m3 + [K/128, N/128] fp32 -> [K, N] fp32 (moe_utils.py:135-142)."""
    K, N = w.shape
    return (w.float().view(K // block, block, N // block, block)
            * s.view(K // block, 1, N // block, 1)).view(K, N)


def dequant_fp8_group_act(q, s, group=128):
    """[M, K] e4m3 + [M, K/128] fp32 -> fp32 (moe_utils.py:144-149)."""
    M, K = q.shape
    return (q.float().view(M, K // group, group) * s.unsqueeze(-1)).view(M, K)


def quant_fp8_block_weight(w: torch.Tensor, block=128):
    """One fp32 scale amax/448 per 128x128 block; used to make synthetic
    weights in the layout the grouped GEMM takes."""
    K, N = w.shape
    g = w.float().view(K // block, block, N // block, block)
    s = (g.abs().amax(dim=(1, 3)) / FP8_MAX).clamp_min(1e-12)
    q = (g / s.view(K // block, 1, N // block, 1)).clamp(-FP8_MAX, FP8_MAX)
    return q.view(K, N).to(torch.float8_e4m3fn), s


def quant_mxfp4_weight(w: torch.Tensor):
    """[N, K] -> bytes [N, K/2] and e8m0 [N, K/32] with the scale rounded up
    (tests/ops/mx_utils.py:277-353, RCEIL) and values rounded to nearest even
    by the bf16->e2m1 cast of that file."""
    N, K = w.shape
    g = w.float().view(N, K // 32, 32)
    amax = g.abs().amax(-1)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127) + 127
    e = torch.where(amax == 0, torch.zeros_like(e), e)
    s_u8 = e.to(torch.uint8)
    inv = torch.where(s_u8 == 0, torch.ones_like(e), torch.exp2(127 - e))
    y = (g * inv.unsqueeze(-1)).clamp(-6.0, 6.0).to(torch.bfloat16).float()
    c = e2m1_code_rne(y).view(N, K)
    return (c[:, 1::2] << 4) | c[:, 0::2], s_u8


def e2m1_code_rne(x):
    """Nearest e2m1 code with ties to the even mantissa (0.25->0, 0.75->1.0,
    1.25->1.0, 1.75->2.0, 2.5->2.0, 3.5->4.0, 5.0->4.0)."""
    a = x.abs()
    code = torch.zeros_like(a, dtype=torch.uint8)
    for b, up_on_tie in ((0.25, False), (0.75, True), (1.25, False), (1.75, True),
                         (2.5, False), (3.5, True), (5.0, False)):
        code += ((a > b) | ((a == b) & up_on_tie)).to(torch.uint8)
    return code | ((x < 0).to(torch.uint8) << 3)


# --------------------------------------------------------------------------
# grouped GEMM and the whole layer
# --------------------------------------------------------------------------
def dequant_expert_weight(recipe, w_e, s_e):
    """Weight of one expert as fp32 [K, N]."""
    if recipe == "bf16":
        return w_e.float()
    if recipe == "fp8block":
        return dequant_fp8_block(w_e, s_e)
    if recipe == "mxfp4":
        return dequant_mxfp4(w_e.view(torch.uint8), s_e.view(torch.uint8)).t()
    if recipe == "fp8":      # one scale per expert (vllm_xpu_kernels/moe_utils.py:214-215)
        return w_e.float() * s_e.float()
    if recipe == "mxfp8":    # e8m0 per 32 of K, [K/32, N] (moe_utils.py:77-80)
        return w_e.float() * e8m0_to_f32(s_e.view(torch.uint8)).repeat_interleave(32, dim=0)
    if recipe == "int4":     # [N, K/2] nibbles - 8, scale [N, K/group] (test_fused_moe.py:37-50)
        return dequant_int4(w_e, s_e).t()
    raise ValueError(recipe)


def dequant_int4(w_u8, scale):
    """[N, K/2] packed (low nibble = even k) -> fp32 [N, K], value (nibble - 8) * scale."""
    lo = (w_u8 & 0xF).to(torch.int32) - 8
    hi = (w_u8 >> 4).to(torch.int32) - 8
    q = torch.stack([lo, hi], dim=-1).reshape(w_u8.shape[0], -1).float()
    group = q.shape[1] // scale.shape[1]
    return q * scale.float().repeat_interleave(group, dim=1)


def quant_mxfp8_weight(w: torch.Tensor):
    """fp32 [K, N] -> (e4m3 [K, N], e8m0 u8 [K/32, N]); scale 2^ceil(log2(amax/448)) per 32 of K."""
    K, N = w.shape
    g = w.reshape(K // 32, 32, N)
    amax = g.abs().amax(1).clamp_min(2.0 ** -120)
    e = torch.ceil(torch.log2(amax / 448.0)).clamp(-127, 127)
    q = (g / torch.exp2(e).unsqueeze(1)).clamp(-448, 448).reshape(K, N).to(torch.float8_e4m3fn)
    return q, (e + 127).to(torch.uint8)


def quant_int4_weight(w: torch.Tensor, group=128, scale_dtype=torch.bfloat16):
    """fp32 [N, K] -> (u8 [N, K/2], scale [N, K/group]); symmetric, zero point 8."""
    N, K = w.shape
    g = w.reshape(N, K // group, group)
    scale = (g.abs().amax(-1) / 7.0).clamp_min(1e-8).to(scale_dtype)
    q = torch.round(g / scale.float().unsqueeze(-1)).clamp(-8, 7).to(torch.int32).reshape(N, K) + 8
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8)
    return packed, scale


def grouped_gemm(recipe, A, B, B_scale, bias, rows_per_expert, out_dtype=None):
    """D[rows of e] = A[rows of e] @ dequant(B_e) (+ bias_e), fp32 accumulate
    (tests/fused_moe/test_grouped_gemm.py:102-589: dequantise then fp32
    matmul per expert).  A is fp32/bf16 [R, K] (already dequantised if it was
    quantised)."""
    out = []
    off = 0
    for e, n in enumerate(rows_per_expert.tolist()):
        if n == 0:
            continue
        w = dequant_expert_weight(recipe, B[e], None if B_scale is None else B_scale[e])
        y = A[off: off + n].float() @ w
        if bias is not None:
            y = y + bias[e].float()
        out.append(y)
        off += n
    R = A.shape[0]
    N = out[0].shape[1] if out else 0
    D = torch.zeros((R, N), dtype=torch.float32)
    if out:
        D[:off] = torch.cat(out, 0)
    return D.to(out_dtype or A.dtype)


def qdq_act(recipe, x, act_format=None):
    """Quantise-dequantise an activation the way the layer's tensor-core path
    sees it: per-token-group-128 FP8 for block-FP8 weights
    (moe_utils.py:190-204), nothing for bf16 and for MXFP4 weights run W4A16.
    ``act_format="mxfp8"``: e4m3 with e8m0 scales per 32 columns
    (moe_utils.py:84-109, 198-200), what the block-scaled MXFP4 path feeds its
    tensor cores.  ``act_format="fp8_pow2"``: group 128 with power-of-two scales,
    what a block-FP8 layer whose weight scales are powers of two feeds them."""
    if act_format == "mxfp8":
        q, sf = quant_mxfp8_act(x)
        return dequant_mxfp8_act(q, sf)
    if act_format == "fp8_pow2":   # per-token-group-128 FP8 with the scale rounded up to a power of
        q, s = per_token_group_fp8_quant(x, 128, scale_ue8m0=True)   # two (the op's scale_ue8m0 flag,
        return dequant_fp8_group_act(q, s)                           # csrc/quantization/fp8/fp8_quant.cpp:238-252)
    if recipe == "fp8block":
        q, s = per_token_group_fp8_quant(x, 128)
        return dequant_fp8_group_act(q, s)
    return x.float()


def fused_moe(recipe, x, w13, w13_scale, w13_bias, w2, w2_scale, w2_bias,
              topk_weights, topk_ids, activation="silu", expert_map=None,
              num_local_experts=None, quant_act=True, out_dtype=None,
              gemm1_clamp_limit=None, situ_beta=None, situ_linear_beta=None, act_format=None):
    """Layer oracle: permute, per-expert dequantise-then-fp32 matmuls with the
    activation between them, weighted un-permute
    (tests/fused_moe/test_fused_moe.py:93-166 for the structure,
    vllm_xpu_kernels/moe_utils.py:244-411 for where activations are
    quantise-dequantised).  Intermediates stay fp32, so this is the
    'dequantise-then-fp32 matmul' the tolerance is stated against."""
    E = num_local_experts if num_local_experts is not None else w13.shape[0]
    xa = qdq_act(recipe, x, act_format) if quant_act else x.float()
    perm, _, rows, row_map = remap_hidden_states(xa, None, topk_ids, expert_map, E)
    h = grouped_gemm(recipe, perm, w13, w13_scale, w13_bias, rows, torch.float32)
    if gemm1_clamp_limit:
        d = h.shape[1] // 2
        h[:, :d].clamp_(max=gemm1_clamp_limit)
        h[:, d:].clamp_(min=-gemm1_clamp_limit, max=gemm1_clamp_limit)
    a = layer_activation(h, activation, situ_beta, situ_linear_beta)
    if quant_act:
        a = qdq_act(recipe, a, act_format)
    y = grouped_gemm(recipe, a, w2, w2_scale, w2_bias, rows, torch.float32)
    return moe_gather(y, topk_weights, row_map, out_dtype or x.dtype)


# --------------------------------------------------------------------------
# seeded synthetic workloads (shared by tests and bench)
# --------------------------------------------------------------------------
CONFIGS = {
    "c0": dict(T=64, H=1024, I=2048, E=8, k=2, recipe="bf16", routing="softmax",
               activation="silu", bias=False),
    "c1": dict(T=4096, H=4096, I=14336, E=8, k=2, recipe="fp8block", routing="softmax",
               activation="silu", bias=False),
    "c2": dict(T=8192, H=2880, I=2880, E=128, k=4, recipe="mxfp4", routing="softmax",
               activation="swigluoai", bias=True),
    "c3": dict(T=16384, H=7168, I=2048, E=256, k=8, recipe="fp8block", routing="grouped",
               activation="silu", bias=False, n_group=8, topk_group=4, scale=2.5),
}


def make_layer(cfg: dict, seed: int = 0, T: Optional[int] = None,
               E_limit: Optional[int] = None, skew: bool = False):
    """Seeded synthetic tensors for one config in the layouts the operators
    take: x bf16 N(0,1); weights N(0, 1/fan_in) quantised per recipe; router
    logits fp32 N(0,1).  ``E_limit`` builds only the first experts' weights
    (routing still runs over all E) for CPU-sized checks."""
    g = torch.Generator().manual_seed(seed)
    T = T or cfg["T"]
    H, I, E = cfg["H"], cfg["I"], cfg["E"]
    En = E_limit or E
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    out = dict(x=x, logits=logits)
    if cfg["routing"] == "grouped":
        out["score_bias"] = torch.randn(E, generator=g) * 0.01
    if skew:
        rank = torch.randperm(E, generator=g) + 1
        out["logits"] = logits + 1.5 * torch.log(1.0 / rank.float())
    w13s, w13sc, w2s, w2sc = [], [], [], []
    for _ in range(En):
        w13 = torch.randn(2 * I, H, generator=g) / math.sqrt(H)   # [N, K]
        w2 = torch.randn(H, I, generator=g) / math.sqrt(I)        # [N, K]
        if cfg["recipe"] == "bf16":
            w13s.append(w13.t().contiguous().to(torch.bfloat16))
            w2s.append(w2.t().contiguous().to(torch.bfloat16))
        elif cfg["recipe"] == "fp8block":
            q, s = quant_fp8_block_weight(w13.t().contiguous()); w13s.append(q); w13sc.append(s)
            q, s = quant_fp8_block_weight(w2.t().contiguous()); w2s.append(q); w2sc.append(s)
        elif cfg["recipe"] == "mxfp4":
            q, s = quant_mxfp4_weight(w13); w13s.append(q); w13sc.append(s)
            q, s = quant_mxfp4_weight(w2); w2s.append(q); w2sc.append(s)
    out["w13"] = torch.stack(w13s)
    out["w2"] = torch.stack(w2s)
    out["w13_scale"] = torch.stack(w13sc) if w13sc else None
    out["w2_scale"] = torch.stack(w2sc) if w2sc else None
    if cfg["bias"]:
        out["w13_bias"] = (torch.randn(En, 2 * I, generator=g) * 0.02).to(torch.bfloat16)
        out["w2_bias"] = (torch.randn(En, H, generator=g) * 0.02).to(torch.bfloat16)
    else:
        out["w13_bias"] = out["w2_bias"] = None
    return out


def route(cfg: dict, layer: dict):
    """Routing of a config through the oracle."""
    if cfg["routing"] == "softmax":
        return topk_softmax(layer["logits"], cfg["k"], True)
    return grouped_topk(layer["logits"], cfg["k"], True, cfg["n_group"],
                        cfg["topk_group"], "sigmoid", cfg["scale"], layer["score_bias"])
