"""Expert-parallel dispatch / combine around the local fused-MoE layer.

The reference project has no exchange step: its "expert parallel" mode gives every
rank all tokens and masks non-local experts (fused_moe_interface.py:297-312 there),
and the all-to-all lives in vLLM.  This module adds that step for one process per
GPU over ``torch.distributed`` (NCCL on NVLink; gloo works for the index logic):

  rank r owns experts [r*E_loc, (r+1)*E_loc) and its own slice of the tokens.

  1. plan      group the (token, slot) pairs by destination rank, stably
               (``remap_hidden_states`` with an expert -> rank map as its
               expert_map), which also packs the rows into the send buffer;
  2. counts    all-to-all of the per-destination row counts;
  3. dispatch  all-to-all-v of rows, their activation scales and local expert ids;
  4. compute   the local layer on the received rows (top-1, weight 1);
  5. combine   all-to-all-v of the results back, then the weighted sum of each
               token's k results (``moe_gather``).

Received data always lands in this GPU's own memory (NCCL) before any kernel
reads it.  Steps 1, 4 and 5 are injected as callables so that the exchange logic
can be exercised on CPU ranks with torch stand-ins.
"""
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


@dataclass
class Plan:
    send_rows: torch.Tensor            # [R, H(bytes)] rows grouped by destination rank
    send_scales: Optional[torch.Tensor]
    send_expert: torch.Tensor          # [R] int32 local expert id at the destination
    send_counts: torch.Tensor          # [G] int32
    row_map: torch.Tensor              # [T, k] int32 position of (t, j) in send_rows


def cuda_plan(hidden, scales, topk_ids, experts_per_rank: int, world: int) -> Plan:
    """Step 1 with the CUDA kernels."""
    T, k = topk_ids.shape
    dev = hidden.device
    E_total = experts_per_rank * world
    rank_of = (torch.arange(E_total, device=dev, dtype=torch.int32) // experts_per_rank)
    send_rows = torch.empty((T * k, hidden.shape[1]), dtype=hidden.dtype, device=dev)
    send_scales = (torch.empty((T * k, scales.shape[1]), dtype=scales.dtype, device=dev)
                   if scales is not None else None)
    counts = torch.zeros(world, dtype=torch.int32, device=dev)
    row_map = torch.empty((T, k), dtype=torch.int32, device=dev)
    torch.ops._moe_C.remap_hidden_states(hidden, scales, send_rows, send_scales, rank_of, counts,
                                         row_map, topk_ids, E_total, world)
    send_expert = torch.empty(T * k, dtype=torch.int32, device=dev)
    send_expert[row_map.flatten().long()] = (topk_ids.flatten() % experts_per_rank).to(torch.int32)
    return Plan(send_rows, send_scales, send_expert, counts, row_map)


def cuda_combine(output, returned, topk_weights, row_map):
    torch.ops._moe_C.moe_gather(output, returned, topk_weights, row_map, 0)


class ExpertParallel:
    """All-to-all dispatch/combine; see the module docstring."""

    def __init__(self, group, experts_per_rank: int,
                 local_fn: Callable[[torch.Tensor, Optional[torch.Tensor], torch.Tensor], torch.Tensor],
                 plan_fn: Callable = cuda_plan, combine_fn: Callable = cuda_combine,
                 out_dtype=torch.bfloat16):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.experts_per_rank = experts_per_rank
        self.local_fn, self.plan_fn, self.combine_fn = local_fn, plan_fn, combine_fn
        self.out_dtype = out_dtype
        self.last_recv_rows = 0

    def _a2a(self, send, recv_rows: int, in_splits, out_splits):
        """all_to_all_single on byte views (NCCL has no fp8 / e8m0 types)."""
        s = send.contiguous()
        as_bytes = s.dtype.itemsize == 1 and s.dtype != torch.uint8
        sv = s.view(torch.uint8) if as_bytes else s
        recv = torch.empty((recv_rows,) + tuple(sv.shape[1:]), dtype=sv.dtype, device=sv.device)
        dist.all_to_all_single(recv, sv, out_splits, in_splits, group=self.group)
        return recv.view(s.dtype) if as_bytes else recv

    def exchange_counts(self, send_counts: torch.Tensor) -> Tuple[list, list]:
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        # the split sizes of the data exchange are host values: one small sync per layer call
        both = torch.stack((send_counts, recv_counts)).cpu()
        return both[0].tolist(), both[1].tolist()

    def apply(self, output, hidden, topk_weights, topk_ids, scales=None):
        plan = self.plan_fn(hidden, scales, topk_ids, self.experts_per_rank, self.world)
        send_splits, recv_splits = self.exchange_counts(plan.send_counts)
        n_recv = sum(recv_splits)
        self.last_recv_rows = n_recv
        rows = self._a2a(plan.send_rows, n_recv, send_splits, recv_splits)
        rscales = (self._a2a(plan.send_scales, n_recv, send_splits, recv_splits)
                   if plan.send_scales is not None else None)
        experts = self._a2a(plan.send_expert, n_recv, send_splits, recv_splits)
        y = self.local_fn(rows, rscales, experts)                  # [n_recv, H]
        back = self._a2a(y, sum(send_splits), recv_splits, send_splits)
        self.combine_fn(output, back, topk_weights, plan.row_map)
        return output


def make_local_fn(moe):
    """Local layer on received rows: every row goes to exactly one local expert with
    weight 1, and comes back in the order it arrived."""
    ones_cache = {}

    def local_fn(rows, scales, experts):
        n = rows.shape[0]
        H = rows.shape[1]
        out = torch.empty((n, H), dtype=torch.bfloat16, device=rows.device)
        if n == 0:
            return out
        if n not in ones_cache:
            ones_cache.clear()
            ones_cache[n] = torch.ones((n, 1), dtype=torch.float32, device=rows.device)
        moe.apply(out, rows, ones_cache[n], experts.view(n, 1), a1q_scale=scales)
        return out

    return local_fn
