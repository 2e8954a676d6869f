"""The expert-parallel exchange kernels with several ranks emulated on ONE GPU.

None of these kernels waits on another rank (the ordering between steps is the caller's
barriers), so the ranks' launches can simply run one after the other on one device, each
rank with its own "symmetric" buffer and the table of all buffers' addresses.  Checked: the
receive buffers hold exactly the rows the grouped GEMM expects (experts back to back,
sources in rank order, stable inside a source), scales and tags travel with them, and the
pull combine (both kernels) and the push return table give the weighted sum of the owners'
results."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
I32, I64 = 4, 5


def _align(n, a=256):
    return (n + a - 1) // a * a


class Rank:
    def __init__(self, r, G, E_loc, T, k, H, scale_bytes, g):
        self.r = r
        E = G * E_loc
        self.x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
        ids[torch.rand(T, k, generator=g) < 0.05] = -1          # a few dropped entries
        self.ids = ids.to(DEV)
        self.w = torch.rand(T, k, generator=g).to(DEV)
        self.scales = (torch.randn(T, scale_bytes // 4, generator=g).to(DEV) if scale_bytes else None)
        cap = G * T * k
        off = 0
        self.off_counts = off; off = _align(off + G * E * 4)
        self.off_rows = off; off = _align(off + cap * H * 2)
        self.off_scales = off; off = _align(off + cap * max(scale_bytes, 4))
        self.off_meta = off; off = _align(off + cap * 8)
        self.off_out = off; off = _align(off + cap * H * 2)
        self.off_ret = off; off = _align(off + T * k * H * 2)
        self.buf = torch.zeros(off, dtype=torch.uint8, device=DEV)
        i32 = dict(dtype=torch.int32, device=DEV)
        self.send_counts = torch.zeros(E, **i32)
        self.row_map = torch.empty(T, k, **i32)
        self.my_prefix = torch.zeros(E + 1, **i32)
        self.dst_start = torch.zeros(E, **i32)
        self.rows_per_expert = torch.zeros(E_loc, **i32)
        self.recv_total = torch.zeros(1, **i32)

    def view(self, off, nbytes, dtype):
        return self.buf[off: off + nbytes].view(dtype)


@pytest.mark.parametrize("G,E_loc,T,k,H,scale_bytes", [(4, 3, 37, 3, 256, 16), (2, 8, 64, 4, 512, 8),
                                                       (3, 2, 50, 2, 128, 0), (1, 8, 33, 2, 256, 16)])
@pytest.mark.parametrize("gather", ["bulk", "loads"])
def test_exchange_with_emulated_ranks(ops, G, E_loc, T, k, H, scale_bytes, gather, monkeypatch):
    from vllm_xpu_kernels import capi
    monkeypatch.setenv("B200MOE_EP_GATHER", gather)
    lib = capi.lib()
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(G * 100 + T)
    E, cap, row_bytes = G * E_loc, G * T * k, H * 2
    ranks = [Rank(r, G, E_loc, T, k, H, scale_bytes, g) for r in range(G)]
    bases = (ctypes.c_int64 * G)(*[rk.buf.data_ptr() for rk in ranks])

    def ok(rc):
        assert rc == 0, (capi.status_string(rc), lib.b200moe_last_error().decode())

    ws = torch.empty(max(lib.b200moe_remap_hidden_states_workspace_bytes(T, k, E), 16), dtype=torch.uint8, device=DEV)
    for rk in ranks:        # step 1 + 2: rank my entries by global expert, publish the counts
        ok(lib.b200moe_remap_hidden_states(None, None, None, None, row_bytes, scale_bytes, rk.ids.data_ptr(),
                                           I32, None, T, k, E, E, rk.send_counts.data_ptr(),
                                           rk.row_map.data_ptr(), ws.data_ptr(), ws.numel(), st))
        ok(lib.b200moe_ep_put_counts(rk.send_counts.data_ptr(), E, bases, rk.off_counts, rk.r, G, st))
    for rk in ranks:        # step 3 + 4: offsets, then rows to their owners
        counts = rk.view(rk.off_counts, G * E * 4, torch.int32)
        ok(lib.b200moe_ep_offsets(counts.data_ptr(), rk.r, G, E_loc, rk.my_prefix.data_ptr(),
                                  rk.dst_start.data_ptr(), rk.rows_per_expert.data_ptr(),
                                  rk.recv_total.data_ptr(), st))
        ok(lib.b200moe_ep_dispatch(rk.x.data_ptr(), rk.scales.data_ptr() if scale_bytes else None, row_bytes,
                                   scale_bytes, rk.ids.data_ptr(), I32, rk.row_map.data_ptr(), T, k, rk.r, G,
                                   E_loc, rk.my_prefix.data_ptr(), rk.dst_start.data_ptr(), bases,
                                   rk.off_rows, rk.off_scales, rk.off_meta, cap, st))
    torch.cuda.synchronize()

    # what every owner must now hold: experts back to back, sources in rank order, stable inside
    for o, rk in enumerate(ranks):
        want_rows, want_scales, want_tags, want_counts = [], [], [], []
        for e in range(o * E_loc, (o + 1) * E_loc):
            n_e = 0
            for s in ranks:
                flat = s.ids.flatten()
                sel = (flat == e).nonzero().flatten()
                want_rows.append(s.x[sel // k])
                if scale_bytes:
                    want_scales.append(s.scales[sel // k])
                want_tags.append((s.r << 32) | s.row_map.flatten()[sel].long())
                n_e += sel.numel()
            want_counts.append(n_e)
        want_rows = torch.cat(want_rows)
        n = want_rows.shape[0]
        assert int(rk.recv_total) == n and rk.rows_per_expert.tolist() == want_counts
        got = rk.view(rk.off_rows, cap * row_bytes, torch.bfloat16).view(cap, H)[:n]
        assert torch.equal(got, want_rows)
        if scale_bytes:
            gs = rk.view(rk.off_scales, cap * scale_bytes, torch.float32).view(cap, -1)[:n]
            assert torch.equal(gs, torch.cat(want_scales))
        assert torch.equal(rk.view(rk.off_meta, cap * 8, torch.int64)[:n], torch.cat(want_tags))
        # stand-in for the experts: result row = received row * (1 + local expert index)
        factor = torch.repeat_interleave(torch.arange(1, E_loc + 1, device=DEV), rk.rows_per_expert.long())
        out = rk.view(rk.off_out, cap * row_bytes, torch.bfloat16).view(cap, H)
        out[:n] = (got.float() * factor.unsqueeze(1)).to(torch.bfloat16)

    def expected(rk):
        e_loc = (rk.ids % E_loc + 1).float()
        rows = (rk.x.float().unsqueeze(1) * e_loc.unsqueeze(2)).to(torch.bfloat16).float()   # [T, k, H]
        wgt = torch.where(rk.ids >= 0, rk.w, torch.zeros_like(rk.w))
        acc = torch.zeros(T, H, device=DEV)
        for j in range(k):                       # slot order, fp32, as the kernels do
            acc = acc + wgt[:, j: j + 1] * rows[:, j]
        return acc.to(torch.bfloat16)

    for rk in ranks:        # pull combine
        src = torch.zeros(T * k, dtype=torch.int64, device=DEV)
        ok(lib.b200moe_ep_source_table(rk.my_prefix.data_ptr(), rk.dst_start.data_ptr(), T * k, G, E_loc,
                                       bases, rk.off_out, row_bytes, cap, src.data_ptr(), st))
        res = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
        ok(lib.b200moe_ep_gather(res.data_ptr(), 2, rk.w.data_ptr(), rk.row_map.data_ptr(), src.data_ptr(),
                                 T, k, H, st))
        torch.cuda.synchronize()
        torch.testing.assert_close(res.float(), expected(rk).float(), atol=2e-2, rtol=2e-2)

    if gather == "bulk":    # push combine: the return table sends every result row home
        for rk in ranks:
            dst = torch.zeros(cap, dtype=torch.int64, device=DEV)
            ok(lib.b200moe_ep_return_table(rk.view(rk.off_meta, cap * 8, torch.int64).data_ptr(),
                                           rk.recv_total.data_ptr(), G, bases, rk.off_ret, row_bytes,
                                           dst.data_ptr(), st))
            n = int(rk.recv_total)
            out = rk.view(rk.off_out, cap * row_bytes, torch.bfloat16).view(cap, H)
            base_of = {int(b): s for b, s in zip(bases, ranks)}
            for j in range(n):           # what the second GEMM's epilogue does with the table
                addr = int(dst[j])
                owner = max((b for b in base_of if b <= addr), key=lambda b: b)
                s = base_of[owner]
                row = (addr - owner - s.off_ret) // row_bytes
                s.view(s.off_ret, T * k * row_bytes, torch.bfloat16).view(T * k, H)[row] = out[j]
        for rk in ranks:
            ret = rk.view(rk.off_ret, T * k * row_bytes, torch.bfloat16).view(T * k, H)
            res = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
            ops._moe_C.moe_gather(res, ret, rk.w, rk.row_map, 0)
            torch.testing.assert_close(res.float(), expected(rk).float(), atol=2e-2, rtol=2e-2)
    assert ops._xpu_C.b200_device_status() == 0


# ---- the cross-rank barrier, all ranks as the CTAs of one cooperative launch ----------------
CH = 4          # B200MOE_EP_BARRIER_CHANNELS
MAXR = 16


def _status(lib):
    st = ctypes.c_int(0)
    assert lib.b200moe_device_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(st)) == 0
    return st.value


def _barrier(lib, flags, epochs, G, channel, absent=0, budget_ns=0):
    return lib.b200moe_ep_barrier_emulated(flags.data_ptr(), epochs.data_ptr(), G, channel, absent,
                                           budget_ns, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("G", [1, 2, 8, 16])
def test_barrier_epochs_advance_together(ops, G):
    from vllm_xpu_kernels import capi
    lib = capi.lib()
    flags = torch.zeros(G * CH * MAXR, dtype=torch.int32, device=DEV)
    epochs = torch.zeros(G * CH, dtype=torch.int32, device=DEV)
    for _ in range(3):
        assert _barrier(lib, flags, epochs, G, 0) == capi.OK
    assert _barrier(lib, flags, epochs, G, 2) == capi.OK
    assert _status(lib) == 0
    want = torch.tensor([3, 0, 1, 0], dtype=torch.int32).repeat(G)
    assert torch.equal(epochs.cpu(), want)
    f = flags.cpu().view(G, CH, MAXR)
    assert (f[:, 0, :G] == 3).all() and (f[:, 2, :G] == 1).all()
    assert (f[:, :, G:] == 0).all() and (f[:, 1] == 0).all() and (f[:, 3] == 0).all()


def test_barrier_gives_up_on_a_missing_rank_and_recovers(ops):
    """Rank 2 of 4 does not arrive: the others wait out their budget, report B200MOE_TIMEOUT
    and carry on.  When the late rank then runs its barrier it finds the others' flags already
    there, and the next common barrier is clean again."""
    from vllm_xpu_kernels import capi
    lib = capi.lib()
    G = 4
    flags = torch.zeros(G * CH * MAXR, dtype=torch.int32, device=DEV)
    epochs = torch.zeros(G * CH, dtype=torch.int32, device=DEV)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    assert _barrier(lib, flags, epochs, G, 1, absent=0b0100, budget_ns=20_000_000) == capi.OK
    t1.record()
    assert _status(lib) == capi.TIMEOUT
    assert 15.0 < t0.elapsed_time(t1) < 500.0          # one budget of 20 ms, not a hang
    assert epochs.cpu().view(G, CH)[:, 1].tolist() == [1, 1, 0, 1]
    assert _barrier(lib, flags, epochs, G, 1, absent=0b1011, budget_ns=20_000_000) == capi.OK
    assert _status(lib) == 0
    assert epochs.cpu().view(G, CH)[:, 1].tolist() == [1, 1, 1, 1]
    assert _barrier(lib, flags, epochs, G, 1, budget_ns=20_000_000) == capi.OK
    assert _status(lib) == 0
    assert epochs.cpu().view(G, CH)[:, 1].tolist() == [2, 2, 2, 2]
    x = torch.ones(8, device=DEV)
    assert float((x * 2).sum()) == 16.0                # the context is still usable


def test_barrier_argument_checks(ops):
    from vllm_xpu_kernels import capi
    lib = capi.lib()
    flags = torch.zeros(2 * CH * MAXR, dtype=torch.int32, device=DEV)
    epochs = torch.zeros(2 * CH, dtype=torch.int32, device=DEV)
    assert _barrier(lib, flags, epochs, 17, 0) == capi.INVALID_ARG
    assert _barrier(lib, flags, epochs, 2, CH) == capi.INVALID_ARG
    bases = (ctypes.c_int64 * 2)(flags.data_ptr(), flags.data_ptr())
    st = torch.cuda.current_stream().cuda_stream
    assert lib.b200moe_ep_barrier(bases, 0, 2, 2, 0, epochs.data_ptr(), 0, st) == capi.INVALID_ARG
    assert lib.b200moe_ep_barrier(bases, 0, 0, 2, 0, None, 0, st) == capi.INVALID_ARG


# ---- the token-level exchange's own three kernels ---------------------------------------------
@pytest.mark.parametrize("T,k,E_loc,G,idt", [(37, 3, 4, 4, torch.int32), (200, 8, 32, 8, torch.int64),
                                             (5, 2, 8, 1, torch.int32)])
def test_token_exchange_helpers(ops, T, k, E_loc, G, idt):
    from vllm_xpu_kernels import capi
    lib = capi.lib()
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(T)
    E = E_loc * G
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(idt)
    ids[torch.rand(T, k, generator=g) < 0.1] = -1
    w = torch.rand(T, k, generator=g)
    code = I32 if idt == torch.int32 else I64
    d_ids, d_w = ids.to(DEV), w.to(DEV)
    # which ranks a token hits
    hits = torch.full((T, G), 77, dtype=torch.int32, device=DEV)
    assert lib.b200moe_ep_rank_hits(d_ids.data_ptr(), code, T, k, E_loc, G, hits.data_ptr(), st) == capi.OK
    want = torch.full((T, G), -1, dtype=torch.int32)
    for t in range(T):
        for e in ids[t].tolist():
            if e >= 0:
                want[t, e // E_loc] = e // E_loc
    assert torch.equal(hits.cpu(), want)
    # routing data out and back in: rank 1 (or 0) sees local ids of its own experts only
    sw = (2 * k + 3) // 4 * 4
    side = torch.zeros(T, sw, dtype=torch.int32, device=DEV)
    assert lib.b200moe_ep_pack_routing(d_ids.data_ptr(), code, d_w.data_ptr(), T, k, sw, side.data_ptr(),
                                       st) == capi.OK
    assert torch.equal(side[:, :k].cpu(), ids.to(torch.int32))
    assert torch.equal(side[:, k:2 * k].view(torch.float32).cpu(), w)
    me, cap, n_in = G - 1, T + 9, T - 2
    buf = torch.full((cap, sw), 3, dtype=torch.int32, device=DEV)      # stale rows route to expert 3
    buf[:T] = side
    total = torch.tensor([n_in], dtype=torch.int32, device=DEV)
    ids_local = torch.empty(cap, k, dtype=torch.int32, device=DEV)
    w_local = torch.empty(cap, k, dtype=torch.float32, device=DEV)
    assert lib.b200moe_ep_unpack_routing(buf.data_ptr(), total.data_ptr(), cap, k, sw, me, E_loc,
                                         ids_local.data_ptr(), w_local.data_ptr(), st) == capi.OK
    loc = ids.to(torch.int32) - me * E_loc
    ok = (loc >= 0) & (loc < E_loc)
    ok[n_in:] = False
    want_ids = torch.full((cap, k), -1, dtype=torch.int32)
    want_ids[:T][ok] = loc[ok]
    want_w = torch.zeros(cap, k)
    want_w[:T][ok] = w[ok]
    assert torch.equal(ids_local.cpu(), want_ids) and torch.equal(w_local.cpu(), want_w)


def test_bounded_gather_leaves_rows_past_the_count_alone(ops):
    T, k, H = 40, 3, 256
    g = torch.Generator().manual_seed(0)
    y = torch.randn(T * k, H, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.rand(T, k, generator=g).to(DEV)
    rm = torch.randperm(T * k, generator=g).to(torch.int32).view(T, k).to(DEV)
    out = torch.full((T, H), 5.0, dtype=torch.bfloat16, device=DEV)
    ref = torch.empty_like(out)
    ops._moe_C.moe_gather(ref, y, w, rm, 1)
    ops._moe_C.b200_moe_gather_bounded(out, y, w, rm, torch.tensor([25], dtype=torch.int32, device=DEV))
    assert torch.equal(out[:25], ref[:25]) and (out[25:] == 5.0).all()


# ---- the token-level exchange end to end, ranks emulated one after the other ------------------
@pytest.mark.parametrize("G,E_loc,T,k,recipe", [(2, 4, 40, 2, "bf16"), (4, 2, 33, 3, "bf16"),
                                                 (2, 4, 48, 2, "fp8block"), (8, 1, 20, 4, "fp8block")])
def test_token_level_exchange_with_emulated_ranks(ops, G, E_loc, T, k, recipe):
    """Every step of TokenExpertParallel.apply with the ranks' launches run one after the other
    on one GPU (none of the kernels waits on another rank): which ranks a token hits, one row
    per (token, rank) to its owner, the owner's ordinary layer on what arrived (ids made
    local, rows past the count masked), one partial sum per (token, rank) pulled back.  The
    result of every rank's tokens is compared with the oracle for the whole layer."""
    from oracle import moe_oracle as O
    from vllm_xpu_kernels import capi
    from vllm_xpu_kernels.fused_moe_interface import XpuFusedMoe
    from vllm_xpu_kernels.moe_utils import quant_fp8_block_act
    lib = capi.lib()
    st = torch.cuda.current_stream().cuda_stream
    E, H, I = G * E_loc, 256, 256
    cfg = dict(T=T, H=H, I=I, E=E, k=k, recipe=recipe, routing="softmax", activation="silu", bias=False)
    layer = O.make_layer(cfg, seed=3)
    fp8 = recipe == "fp8block"
    row_bytes, scale_bytes = H * (1 if fp8 else 2), (H // 128) * 4 if fp8 else 0
    cap, side_w = G * T, (2 * k + 3) // 4 * 4

    def ok(rc):
        assert rc == 0, (capi.status_string(rc), lib.b200moe_last_error().decode())

    class R:
        pass
    ranks = []
    for r in range(G):
        rk = R()
        rk.r = r
        tok = O.make_layer(cfg, seed=100 + r, E_limit=1)
        rk.x_host, rk.logits = tok["x"], tok["logits"]
        rk.w_host, rk.ids_host = O.topk_softmax(rk.logits, k, True)
        rk.ids = rk.ids_host.to(torch.int32).to(DEV)
        rk.w = rk.w_host.to(DEV)
        x = rk.x_host.to(DEV)
        rk.x, rk.scales = quant_fp8_block_act(x) if fp8 else (x, None)
        sl = slice(r * E_loc, (r + 1) * E_loc)
        d = lambda t: None if t is None else t[sl].to(DEV)  # noqa: E731
        rk.moe = XpuFusedMoe(d(layer["w13"]), d(layer["w13_scale"]), None, d(layer["w2"]), d(layer["w2_scale"]),
                             None, k, "silu", E_loc)
        off = 0
        rk.off_counts = off; off = _align(off + G * G * 4)
        rk.off_rows = off; off = _align(off + cap * row_bytes)
        rk.off_scales = off; off = _align(off + cap * max(scale_bytes, 4))
        rk.off_meta = off; off = _align(off + cap * 8)
        rk.off_side = off; off = _align(off + cap * side_w * 4)
        rk.off_out = off; off = _align(off + cap * H * 2)
        rk.buf = torch.zeros(off, dtype=torch.uint8, device=DEV)
        rk.buf[rk.off_side: rk.off_side + cap * side_w * 4].view(torch.int32).fill_(1)   # stale rows route to expert 1
        i32 = dict(dtype=torch.int32, device=DEV)
        rk.hits = torch.empty(T, G, **i32)
        rk.send_counts = torch.zeros(G, **i32)
        rk.row_map = torch.empty(T, G, **i32)
        rk.side = torch.zeros(T, side_w, **i32)
        rk.my_prefix, rk.dst_start = torch.zeros(G + 1, **i32), torch.zeros(G, **i32)
        rk.tokens_in, rk.recv_total = torch.zeros(1, **i32), torch.zeros(1, **i32)
        ranks.append(rk)
    bases = (ctypes.c_int64 * G)(*[rk.buf.data_ptr() for rk in ranks])
    ws = torch.empty(max(lib.b200moe_remap_hidden_states_workspace_bytes(T, G, G), 16), dtype=torch.uint8, device=DEV)
    for rk in ranks:
        ok(lib.b200moe_ep_rank_hits(rk.ids.data_ptr(), I32, T, k, E_loc, G, rk.hits.data_ptr(), st))
        ok(lib.b200moe_remap_hidden_states(None, None, None, None, row_bytes, scale_bytes, rk.hits.data_ptr(), I32,
                                           None, T, G, G, G, rk.send_counts.data_ptr(), rk.row_map.data_ptr(),
                                           ws.data_ptr(), ws.numel(), st))
        ok(lib.b200moe_ep_pack_routing(rk.ids.data_ptr(), I32, rk.w.data_ptr(), T, k, side_w, rk.side.data_ptr(), st))
        ok(lib.b200moe_ep_put_counts(rk.send_counts.data_ptr(), G, bases, rk.off_counts, rk.r, G, st))
    for rk in ranks:
        counts = rk.buf[rk.off_counts: rk.off_counts + G * G * 4].view(torch.int32)
        ok(lib.b200moe_ep_offsets(counts.data_ptr(), rk.r, G, 1, rk.my_prefix.data_ptr(), rk.dst_start.data_ptr(),
                                  rk.tokens_in.data_ptr(), rk.recv_total.data_ptr(), st))
        ok(lib.b200moe_ep_dispatch(rk.x.data_ptr(), rk.scales.data_ptr() if fp8 else None, row_bytes, scale_bytes,
                                   rk.hits.data_ptr(), I32, rk.row_map.data_ptr(), T, G, rk.r, G, 1,
                                   rk.my_prefix.data_ptr(), rk.dst_start.data_ptr(), bases, rk.off_rows,
                                   rk.off_scales, rk.off_meta, cap, st))
        ok(lib.b200moe_ep_dispatch(rk.side.data_ptr(), None, side_w * 4, 0, rk.hits.data_ptr(), I32,
                                   rk.row_map.data_ptr(), T, G, rk.r, G, 1, rk.my_prefix.data_ptr(),
                                   rk.dst_start.data_ptr(), bases, rk.off_side, 0, rk.off_meta, cap, st))
    torch.cuda.synchronize()
    # every rank received exactly the tokens that have an expert there, sources in rank order
    for o, rk in enumerate(ranks):
        want = sum(int(((s.ids_host // E_loc) == o).any(dim=1).sum()) for s in ranks)
        assert int(rk.recv_total) == want
    for rk in ranks:        # the owner's ordinary layer on what arrived
        ids_local = torch.empty(cap, k, dtype=torch.int32, device=DEV)
        w_local = torch.empty(cap, k, dtype=torch.float32, device=DEV)
        side = rk.buf[rk.off_side: rk.off_side + cap * side_w * 4].view(torch.int32)
        ok(lib.b200moe_ep_unpack_routing(side.data_ptr(), rk.recv_total.data_ptr(), cap, k, side_w, rk.r, E_loc,
                                         ids_local.data_ptr(), w_local.data_ptr(), st))
        n = int(rk.recv_total)
        assert (ids_local[n:] == -1).all() and (ids_local[:n] < E_loc).all()
        rows = rk.buf[rk.off_rows: rk.off_rows + cap * row_bytes].view(rk.x.dtype).view(cap, H)
        rsc = (rk.buf[rk.off_scales: rk.off_scales + cap * scale_bytes].view(torch.float32).view(cap, -1)
               if fp8 else None)
        partial = rk.buf[rk.off_out: rk.off_out + cap * H * 2].view(torch.bfloat16).view(cap, H)
        partial.fill_(9.0)
        rk.moe.apply(partial, rows, w_local, ids_local, a1q_scale=rsc, valid_tokens=rk.recv_total)
        assert (partial[n:] == 9.0).all()            # rows past the count are not written
    torch.cuda.synchronize()
    ones = torch.ones(T, G, dtype=torch.float32, device=DEV)
    for rk in ranks:        # one partial sum per (token, rank), added in rank order
        src = torch.zeros(T * G, dtype=torch.int64, device=DEV)
        ok(lib.b200moe_ep_source_table(rk.my_prefix.data_ptr(), rk.dst_start.data_ptr(), T * G, G, 1, bases,
                                       rk.off_out, H * 2, cap, src.data_ptr(), st))
        res = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
        ok(lib.b200moe_ep_gather(res.data_ptr(), 2, ones.data_ptr(), rk.row_map.data_ptr(), src.data_ptr(),
                                 T, G, H, st))
        torch.cuda.synchronize()
        ref = O.fused_moe(recipe, rk.x_host, layer["w13"], layer["w13_scale"], None, layer["w2"],
                          layer["w2_scale"], None, rk.w_host, rk.ids_host, "silu", out_dtype=torch.float32)
        err = (res.float().cpu() - ref).abs()
        assert (err <= 2e-2 + 2e-2 * ref.abs()).all(), f"rank {rk.r}: max err {err.max():.4g}"
    assert ops._xpu_C.b200_device_status() == 0
