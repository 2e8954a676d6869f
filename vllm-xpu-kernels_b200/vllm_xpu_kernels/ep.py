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
import os
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


# dtype codes of the C interface
_FLOAT_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_INDEX_CODES = {torch.int32: 4, torch.int64: 5}


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


# --------------------------------------------------------------------------------------
# Exchange over peer-mapped (symmetric) memory: no collective-library call and no host
# round trip on the data path.
# --------------------------------------------------------------------------------------
def _align(n, a=256):
    return (n + a - 1) // a * a


class PeerExpertParallel:
    """Expert-parallel layer call whose dispatch and combine move rows through other GPUs'
    memory from this library's own kernels (see csrc/capi/ep.cu):

      rank my (token, slot) entries by global expert (remap_hidden_states, grouping only) ->
      put_counts -> barrier -> offsets -> dispatch every row to its final place in its owner's
      expert-grouped receive buffer -> barrier -> the two grouped GEMMs straight on the
      receive buffer -> barrier -> gather: the token's owner reads its k result rows from the
      owners' output buffers inside the weighted sum ("pull"; with combine="push" the second
      GEMM's epilogue stores the rows into the sender's return buffer instead).

    The receiving side runs no permutation: senders place rows where the grouped GEMM wants
    them.  Receive and output buffers are sized for the worst case (every routed row of
    every rank lands here); unused rows cost nothing in the GEMMs, whose row counts live on
    the device.  The three barriers are this library's own kernel (b200moe_ep_barrier: epoch
    flags stored into the peers' memory, a bounded poll of local memory), stream-ordered;
    there is no host synchronisation, and a peer that never arrives costs one time budget and
    leaves B200MOE_TIMEOUT in the device status word instead of hanging the GPU.
    """

    def __init__(self, group, moe, tokens_per_rank: int, topk: int, hidden: int, row_bytes: int,
                 scale_row_bytes: int, experts_per_rank: int, device, out_dtype=torch.bfloat16,
                 combine: str = None):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import capi
        self.lib, self.capi = capi.lib(), capi
        self.group, self.moe = group, moe
        self.G = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.T, self.k, self.H = tokens_per_rank, topk, hidden
        self.row_bytes, self.scale_row_bytes = row_bytes, scale_row_bytes
        self.E_loc, self.dev, self.out_dtype = experts_per_rank, device, out_dtype
        G, R = self.G, tokens_per_rank * topk
        self.E = G * experts_per_rank
        self.R, self.cap = R, G * R
        self.ret_row_bytes = hidden * torch.empty((), dtype=out_dtype).element_size()
        off = 0
        self.off_flags = off; off = _align(off + self.capi.EP_BARRIER_CHANNELS * 16 * 4)
        self.off_counts = off; off = _align(off + G * self.E * 4)
        self.off_rows = off; off = _align(off + self.cap * row_bytes)
        self.off_scales = off; off = _align(off + self.cap * max(scale_row_bytes, 4))
        self.off_meta = off; off = _align(off + self.cap * 8)
        # "pull": the second GEMM stores locally and the token's owner reads the result rows
        # from the peers inside the weighted sum.  "push": the second GEMM's epilogue stores
        # every row into its sender's return buffer.  Measured on 8 GPUs at the DeepSeek-V3
        # shape, the epilogue's per-lane 16-byte stores reach a fifth of the link rate and
        # stall the tensor pipeline (second GEMM 12.4 ms against 3.7 ms alone), so pull is
        # the default.
        self.combine = combine or os.environ.get("B200MOE_EP_COMBINE", "pull")
        assert self.combine in ("pull", "push")
        if self.combine == "push":
            self.off_ret = off; off = _align(off + R * self.ret_row_bytes)
            self.off_out = 0
        else:
            self.off_out = off; off = _align(off + self.cap * self.ret_row_bytes)
            self.off_ret = 0
        self.buf = symm_mem.empty(off, dtype=torch.uint8, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, group.group_name)
        self.buf.zero_()
        self.peer_bases = (ctypes.c_int64 * G)(*[int(p) for p in self.hdl.buffer_ptrs])
        b = self.buf
        self.counts = b[self.off_counts: self.off_counts + G * self.E * 4].view(torch.int32)
        self.recv_rows = b[self.off_rows: self.off_rows + self.cap * row_bytes]
        self.recv_scales = (b[self.off_scales: self.off_scales + self.cap * scale_row_bytes]
                            if scale_row_bytes else None)
        self.meta = b[self.off_meta: self.off_meta + self.cap * 8].view(torch.int64)
        if self.combine == "push":
            self.ret = b[self.off_ret: self.off_ret + R * self.ret_row_bytes].view(out_dtype).view(R, hidden)
            self.dst_addr = torch.zeros(self.cap, dtype=torch.int64, device=device)
        else:
            self.out_rows = b[self.off_out: self.off_out + self.cap * self.ret_row_bytes] \
                .view(out_dtype).view(self.cap, hidden)
            self.src_addr = torch.zeros(R, dtype=torch.int64, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        self.my_prefix = torch.zeros(self.E + 1, **i32)
        self.dst_start = torch.zeros(self.E, **i32)
        self.rows_per_expert = torch.zeros(experts_per_rank, **i32)
        self.recv_total = torch.zeros(1, **i32)
        self._ws = None
        self.epochs = torch.zeros(self.capi.EP_BARRIER_CHANNELS, **i32)
        # the flag words must be zero on every rank before anyone's first barrier writes one:
        # once, at construction, through the host
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def barrier(self, channel: int, budget_ns: int = 0):
        """Cross-rank barrier on the current stream (see b200moe_ep_barrier)."""
        self._check(self.lib.b200moe_ep_barrier(
            self.peer_bases, self.off_flags, self.rank, self.G, channel, self.epochs.data_ptr(),
            budget_ns, torch.cuda.current_stream().cuda_stream), "ep_barrier")

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: {self.capi.status_string(rc)} ({self.lib.b200moe_last_error().decode()})")

    def check_call(self, hidden, topk_ids, scales):
        """Refuses a call that does not fit the buffers sized at construction: more tokens or
        another top-k would make the address tables and the exchange buffers too small."""
        T, k = topk_ids.shape
        if T > self.T or k != self.k:
            raise ValueError(f"PeerExpertParallel was built for at most {self.T} tokens with top-{self.k}; "
                             f"got {T} tokens with top-{k}")
        if hidden.shape[0] != T or hidden.shape[1] * hidden.element_size() != self.row_bytes:
            raise ValueError(f"hidden states must be [{T}, .] rows of {self.row_bytes} bytes; "
                             f"got {tuple(hidden.shape)} {hidden.dtype}")
        got = 0 if scales is None else scales.shape[1] * scales.element_size()
        if got != self.scale_row_bytes or (scales is not None and scales.shape[0] != T):
            raise ValueError(f"activation scales must be rows of {self.scale_row_bytes} bytes; got {got}")

    def apply(self, output, hidden, topk_weights, topk_ids, scales=None):
        self.check_call(hidden, topk_ids, scales)
        lib, G, me = self.lib, self.G, self.rank
        T, k = topk_ids.shape
        dev = hidden.device
        st = torch.cuda.current_stream().cuda_stream
        # where each (token, slot) entry stands in my send order (stable by global expert), and
        # how many entries go to each expert; the rows themselves are not copied locally
        send_counts = torch.zeros(self.E, dtype=torch.int32, device=dev)
        row_map = torch.empty((T, k), dtype=torch.int32, device=dev)
        stage = self.moe._stage
        ids_code = _INDEX_CODES[topk_ids.dtype]
        ws_bytes = lib.b200moe_remap_hidden_states_workspace_bytes(T, k, self.E)
        if self._ws is None or self._ws.numel() < ws_bytes:
            self._ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        with stage("ep_group"):
            self._check(lib.b200moe_remap_hidden_states(
                None, None, None, None, self.row_bytes, self.scale_row_bytes, topk_ids.data_ptr(),
                ids_code, None, T, k, self.E, self.E, send_counts.data_ptr(), row_map.data_ptr(),
                self._ws.data_ptr(), self._ws.numel(), st), "remap_hidden_states")
        with stage("ep_counts"):
            self._check(lib.b200moe_ep_put_counts(send_counts.data_ptr(), self.E, self.peer_bases,
                                                  self.off_counts, me, G, st), "ep_put_counts")
            self.barrier(0)
            self._check(lib.b200moe_ep_offsets(self.counts.data_ptr(), me, G, self.E_loc,
                                               self.my_prefix.data_ptr(), self.dst_start.data_ptr(),
                                               self.rows_per_expert.data_ptr(),
                                               self.recv_total.data_ptr(), st), "ep_offsets")
        with stage("ep_push"):
            self._check(lib.b200moe_ep_dispatch(
                hidden.data_ptr(), scales.data_ptr() if scales is not None else None, self.row_bytes,
                self.scale_row_bytes, topk_ids.data_ptr(), ids_code, row_map.data_ptr(), T, k, me, G,
                self.E_loc, self.my_prefix.data_ptr(), self.dst_start.data_ptr(), self.peer_bases,
                self.off_rows, self.off_scales, self.off_meta, self.cap, st), "ep_dispatch")
            self.barrier(1)
        rows = self.recv_rows.view(hidden.dtype).view(self.cap, -1)
        rscales = self.recv_scales.view(scales.dtype).view(self.cap, -1) if scales is not None else None
        if self.combine == "push":
            with stage("ep_table"):
                self._check(lib.b200moe_ep_return_table(
                    self.meta.data_ptr(), self.recv_total.data_ptr(), G, self.peer_bases, self.off_ret,
                    self.ret_row_bytes, self.dst_addr.data_ptr(), st), "ep_return_table")
            self.moe.run_experts(rows, rscales, self.rows_per_expert, self.out_dtype, self.dst_addr)
            with stage("ep_combine"):
                self.barrier(2)
                torch.ops._moe_C.moe_gather(output, self.ret, topk_weights, row_map, 0)
            return output
        with stage("ep_table"):
            self._check(lib.b200moe_ep_source_table(
                self.my_prefix.data_ptr(), self.dst_start.data_ptr(), T * k, G, self.E_loc,
                self.peer_bases, self.off_out, self.ret_row_bytes, self.cap,
                self.src_addr.data_ptr(), st), "ep_source_table")
        self.moe.run_experts(rows, rscales, self.rows_per_expert, self.out_dtype, None, self.out_rows)
        with stage("ep_combine"):
            self.barrier(2)
            self._check(lib.b200moe_ep_gather(
                output.data_ptr(), _FLOAT_CODES[output.dtype], topk_weights.data_ptr(),
                row_map.data_ptr(), self.src_addr.data_ptr(), T, k, self.H, st), "ep_gather")
        return output


class TokenExpertParallel(PeerExpertParallel):
    """The same exchange at TOKEN granularity: a token crosses to a rank once, however many
    of its experts live there, and one partial sum per (token, rank) comes back.

      which ranks does each token hit (ep_rank_hits) -> rank the (token, rank) pairs by rank
      (remap_hidden_states, grouping only) -> put_counts -> barrier -> offsets -> dispatch each
      token's row + scales, and its k (expert id, weight) pairs, to every rank it hits ->
      barrier -> the receiving rank turns the ids into local ids (-1 elsewhere) and runs its
      ordinary local layer on the tokens it got (permutation, the two grouped GEMMs, weighted
      combine over the LOCAL experts of each token) -> barrier -> the token's owner reads one
      partial row per rank it hit and adds them in rank order (ep_gather with weights 1).

    With group-limited routing a token of the DeepSeek-V3 layer reaches at most 4 of 8 ranks
    (2 of 2 on two GPUs) with 8 experts, so rows out and results back are 2-4x fewer than with
    one row per (token, expert).  Every kernel is one the row-level exchange or the single-GPU
    layer already uses; a rank is "an expert" (experts_per_rank = 1, top-k = world) for the
    grouping, offset, dispatch, address-table and gather kernels.  The partial sums are
    rounded to the output dtype once per rank before the final fp32 sum.
    """

    def __init__(self, group, moe, tokens_per_rank: int, topk: int, hidden: int, row_bytes: int,
                 scale_row_bytes: int, experts_per_rank: int, device, out_dtype=torch.bfloat16):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import capi
        self.lib, self.capi = capi.lib(), capi
        self.group, self.moe = group, moe
        self.G = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.T, self.k, self.H = tokens_per_rank, topk, hidden
        self.row_bytes, self.scale_row_bytes = row_bytes, scale_row_bytes
        self.E_loc, self.dev, self.out_dtype = experts_per_rank, device, out_dtype
        G = self.G
        self.E = G * experts_per_rank
        self.cap = G * tokens_per_rank                     # tokens this rank can receive
        self.side_w = (2 * topk + 3) // 4 * 4              # i32 words of routing data per token
        self.ret_row_bytes = hidden * torch.empty((), dtype=out_dtype).element_size()
        cap, off = self.cap, 0
        self.off_flags = off; off = _align(off + capi.EP_BARRIER_CHANNELS * 16 * 4)
        self.off_counts = off; off = _align(off + G * G * 4)
        self.off_rows = off; off = _align(off + cap * row_bytes)
        self.off_scales = off; off = _align(off + cap * max(scale_row_bytes, 4))
        self.off_meta = off; off = _align(off + cap * 8)
        self.off_side = off; off = _align(off + cap * self.side_w * 4)
        self.off_out = off; off = _align(off + cap * self.ret_row_bytes)
        self.buf = symm_mem.empty(off, dtype=torch.uint8, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, group.group_name)
        self.buf.zero_()
        self.peer_bases = (ctypes.c_int64 * G)(*[int(p) for p in self.hdl.buffer_ptrs])
        b = self.buf
        self.counts = b[self.off_counts: self.off_counts + G * G * 4].view(torch.int32)
        self.recv_rows = b[self.off_rows: self.off_rows + cap * row_bytes]
        self.recv_scales = (b[self.off_scales: self.off_scales + cap * scale_row_bytes]
                            if scale_row_bytes else None)
        self.recv_side = b[self.off_side: self.off_side + cap * self.side_w * 4].view(torch.int32)
        self.partial = b[self.off_out: self.off_out + cap * self.ret_row_bytes] \
            .view(out_dtype).view(cap, hidden)
        i32 = dict(dtype=torch.int32, device=device)
        self.my_prefix = torch.zeros(G + 1, **i32)
        self.dst_start = torch.zeros(G, **i32)
        self.tokens_in = torch.zeros(1, **i32)             # "rows per expert" of the one-expert-per-rank view
        self.recv_total = torch.zeros(1, **i32)
        self.src_addr = torch.zeros(tokens_per_rank * G, dtype=torch.int64, device=device)
        self.hits = torch.empty(tokens_per_rank, G, **i32)
        self.side = torch.zeros(tokens_per_rank, self.side_w, **i32)
        self.ids_local = torch.empty(cap, topk, **i32)
        self.w_local = torch.empty(cap, topk, dtype=torch.float32, device=device)
        self.ones = torch.ones(tokens_per_rank, G, dtype=torch.float32, device=device)
        self._ws = None
        self.epochs = torch.zeros(capi.EP_BARRIER_CHANNELS, **i32)
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def apply(self, output, hidden, topk_weights, topk_ids, scales=None):
        self.check_call(hidden, topk_ids, scales)
        lib, G, me = self.lib, self.G, self.rank
        T, k = topk_ids.shape
        dev = hidden.device
        st = torch.cuda.current_stream().cuda_stream
        stage = self.moe._stage
        ids_code, I32 = _INDEX_CODES[topk_ids.dtype], _INDEX_CODES[torch.int32]
        send_counts = torch.zeros(G, dtype=torch.int32, device=dev)
        row_map = torch.empty((T, G), dtype=torch.int32, device=dev)
        hits = self.hits[:T]
        ws_bytes = lib.b200moe_remap_hidden_states_workspace_bytes(T, G, G)
        if self._ws is None or self._ws.numel() < ws_bytes:
            self._ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        with stage("ep_group"):
            self._check(lib.b200moe_ep_rank_hits(topk_ids.data_ptr(), ids_code, T, k, self.E_loc, G,
                                                 hits.data_ptr(), st), "ep_rank_hits")
            self._check(lib.b200moe_remap_hidden_states(
                None, None, None, None, self.row_bytes, self.scale_row_bytes, hits.data_ptr(), I32,
                None, T, G, G, G, send_counts.data_ptr(), row_map.data_ptr(), self._ws.data_ptr(),
                self._ws.numel(), st), "remap_hidden_states")
            self._check(lib.b200moe_ep_pack_routing(topk_ids.data_ptr(), ids_code, topk_weights.data_ptr(),
                                                    T, k, self.side_w, self.side.data_ptr(), st),
                        "ep_pack_routing")
        with stage("ep_counts"):
            self._check(lib.b200moe_ep_put_counts(send_counts.data_ptr(), G, self.peer_bases,
                                                  self.off_counts, me, G, st), "ep_put_counts")
            self.barrier(0)
            self._check(lib.b200moe_ep_offsets(self.counts.data_ptr(), me, G, 1, self.my_prefix.data_ptr(),
                                               self.dst_start.data_ptr(), self.tokens_in.data_ptr(),
                                               self.recv_total.data_ptr(), st), "ep_offsets")
        with stage("ep_push"):
            self._check(lib.b200moe_ep_dispatch(
                hidden.data_ptr(), scales.data_ptr() if scales is not None else None, self.row_bytes,
                self.scale_row_bytes, hits.data_ptr(), I32, row_map.data_ptr(), T, G, me, G, 1,
                self.my_prefix.data_ptr(), self.dst_start.data_ptr(), self.peer_bases, self.off_rows,
                self.off_scales, self.off_meta, self.cap, st), "ep_dispatch")
            self._check(lib.b200moe_ep_dispatch(
                self.side.data_ptr(), None, self.side_w * 4, 0, hits.data_ptr(), I32, row_map.data_ptr(),
                T, G, me, G, 1, self.my_prefix.data_ptr(), self.dst_start.data_ptr(), self.peer_bases,
                self.off_side, 0, self.off_meta, self.cap, st), "ep_dispatch (routing data)")
            self.barrier(1)
        with stage("ep_table"):
            self._check(lib.b200moe_ep_unpack_routing(
                self.recv_side.data_ptr(), self.recv_total.data_ptr(), self.cap, k, self.side_w, me,
                self.E_loc, self.ids_local.data_ptr(), self.w_local.data_ptr(), st), "ep_unpack_routing")
            self._check(lib.b200moe_ep_source_table(
                self.my_prefix.data_ptr(), self.dst_start.data_ptr(), T * G, G, 1, self.peer_bases,
                self.off_out, self.ret_row_bytes, self.cap, self.src_addr.data_ptr(), st),
                "ep_source_table")
        rows = self.recv_rows.view(hidden.dtype).view(self.cap, -1)
        rscales = self.recv_scales.view(scales.dtype).view(self.cap, -1) if scales is not None else None
        # the ordinary local layer on the tokens that arrived; rows past recv_total carry ids of
        # -1 and their partial rows are not written
        gate, done = getattr(self, "gemm_gate", None), getattr(self, "gemm_done", None)
        if gate is not None:    # second wave of WaveExpertParallel: after the first wave's GEMMs
            torch.cuda.current_stream().wait_event(gate)
        self.moe.apply(self.partial, rows, self.w_local, self.ids_local, a1q_scale=rscales,
                       valid_tokens=self.recv_total, after_gemms=done)
        with stage("ep_combine"):
            self.barrier(2)
            self._check(lib.b200moe_ep_gather(
                output.data_ptr(), _FLOAT_CODES[output.dtype], self.ones[:T].data_ptr(),
                row_map.data_ptr(), self.src_addr.data_ptr(), T, G, self.H, st), "ep_gather")
        return output


class WaveExpertParallel:
    """Two waves of tokens through two token-level exchanges on two streams, so that one
    wave's dispatch and combine run beside the other wave's grouped GEMMs:

        stream 1:  dispatch A, permute A, GEMMs A,                gather A, combine A
        stream 2:  dispatch B, permute B,          (GEMMs A done) GEMMs B, gather B, combine B

    The grouped GEMM is a persistent kernel with one CTA per SM, so the exchange kernels only
    find room beside it when its grid is capped (``gemm_sms``, default 132 of 148;
    B200MOE_GEMM_SMS for the duration of a call); the two waves' GEMMs are serialised by an
    event, not left to compete for the same SMs.  Worth it only where dispatch + combine are a
    large share of the step (many ranks); with few ranks the SMs given up cost more than the
    transfers hidden.
    """

    def __init__(self, group, moe, tokens_per_rank: int, topk: int, hidden: int, row_bytes: int,
                 scale_row_bytes: int, experts_per_rank: int, device, out_dtype=torch.bfloat16,
                 gemm_sms: int = 132):
        self.half = (tokens_per_rank + 1) // 2
        mk = lambda: TokenExpertParallel(group, moe, self.half, topk, hidden, row_bytes, scale_row_bytes,  # noqa: E731
                                         experts_per_rank, device, out_dtype)
        self.waves = (mk(), mk())
        self.streams = (torch.cuda.Stream(device), torch.cuda.Stream(device))
        self.gemm_sms = gemm_sms
        self.moe = moe

    def apply(self, output, hidden, topk_weights, topk_ids, scales=None):
        T = topk_ids.shape[0]
        cut = min(self.half, T)
        main = torch.cuda.current_stream()
        parts = ((0, cut), (cut, T))
        gemms_done = torch.cuda.Event()
        prev = os.environ.get("B200MOE_GEMM_SMS")
        os.environ["B200MOE_GEMM_SMS"] = str(self.gemm_sms)
        try:
            for i, (lo, hi) in enumerate(parts):
                if hi <= lo:
                    continue
                st = self.streams[i]
                st.wait_stream(main)
                with torch.cuda.stream(st):
                    ep = self.waves[i]
                    ep.gemm_gate = gemms_done if i == 1 else None      # wait for wave A's GEMMs
                    ep.gemm_done = gemms_done if i == 0 else None      # record after wave A's GEMMs
                    ep.apply(output[lo:hi], hidden[lo:hi], topk_weights[lo:hi], topk_ids[lo:hi],
                             scales=None if scales is None else scales[lo:hi])
            for st in self.streams:
                main.wait_stream(st)
        finally:
            if prev is None:
                os.environ.pop("B200MOE_GEMM_SMS", None)
            else:
                os.environ["B200MOE_GEMM_SMS"] = prev
        return output
