"""Generate tests/golden/*.npz from the reference project's own torch oracles.

Run once, in a container where the reference tree is mounted:

    python tests/golden/make_golden.py /path/to/reference

The reference's three native extension modules are only imported for their
registration side effect, so empty stand-ins are enough to import its pure
torch test oracles on CPU.  The stored arrays (seeded inputs and the
reference's outputs) travel with the repository; the reference tree does not
need to exist where the tests run.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(root):
    sys.dont_write_bytecode = True
    sys.path.insert(0, root)
    import importlib.machinery
    pkg = types.ModuleType("vllm_xpu_kernels")
    pkg.__path__ = [os.path.join(root, "vllm_xpu_kernels")]
    pkg.__spec__ = importlib.machinery.ModuleSpec("vllm_xpu_kernels", None, is_package=True)
    sys.modules["vllm_xpu_kernels"] = pkg
    for name in ("_C", "_moe_C", "_xpu_C"):
        m = types.ModuleType("vllm_xpu_kernels." + name)
        sys.modules["vllm_xpu_kernels." + name] = m
        setattr(pkg, name, m)


def _np(t):
    if t is None:
        return None
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu):
        return t.view(torch.uint8).numpy()
    if hasattr(torch, "float4_e2m1fn_x2") and t.dtype == torch.float4_e2m1fn_x2:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def save(name, **arrays):
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        **{k: _np(v) if isinstance(v, torch.Tensor) else np.asarray(v)
                           for k, v in arrays.items() if v is not None})
    print("wrote", name)


def main(root):
    _import_reference(root)
    from tests.ops import topk_op, grouped_topk_op
    from tests.ops.activation_op import SiluAndMul
    from tests.ops.swigluoai_and_mul_op import SwigluOAIAndMul
    from tests.ops.mx_utils import to_mxfp
    from tests.test_moe_align_block_size import torch_moe_align_block_size
    from tests.test_moe_gather import ref_moe_gather
    from tests.fused_moe.test_remap_hidden_states import ref_remap_hidden_states
    from tests.fused_moe.test_fused_moe import ref_fused_moe
    from tests.test_fp8_quant import ref_per_block_quant
    import vllm_xpu_kernels.moe_utils as mu

    g = torch.Generator().manual_seed(1234)

    # ---- routing -------------------------------------------------------
    for tag, (T, E, k) in {"a": (33, 8, 2), "b": (64, 128, 4), "c": (17, 60, 6)}.items():
        logits = torch.randn(T, E, generator=g)
        bias = torch.randn(E, generator=g) * 0.05
        pad = torch.rand(T, generator=g) < 0.2
        for renorm in (False, True):
            w, i = topk_op.topk_softmax(None, logits, k, renorm)
            wb, ib = topk_op.topk_softmax(None, logits, k, renorm, bias=bias, is_padding=pad)
            ws, is_ = topk_op.topk_sigmoid(None, logits, k, renorm, bias=bias,
                                           routed_scaling_factor=2.5)
            save(f"topk_{tag}_{int(renorm)}", logits=logits, bias=bias, pad=pad, k=k,
                 renorm=renorm, w=w, i=i, wb=wb, ib=ib, ws=ws, is_=is_)
    # ties: many equal logits -> lower index must win
    logits = torch.randint(-2, 3, (40, 16), generator=g).float()
    w, i = topk_op.topk_softmax(None, logits, 4, True)
    save("topk_ties", logits=logits, k=4, w=w, i=i)

    for tag, (T, E, ng, tg, k) in {"a": (48, 256, 8, 4, 8), "b": (19, 64, 4, 2, 6),
                                   "c": (7, 16, 2, 1, 2)}.items():
        logits = torch.randn(T, E, generator=g)
        bias = torch.randn(E, generator=g) * 0.01
        for renorm in (False, True):
            w, i = grouped_topk_op.grouped_topk(logits, logits, k, renorm, ng, tg, "sigmoid",
                                                2.5, bias)
            w2, i2 = grouped_topk_op.grouped_topk(logits, logits, k, renorm, ng, tg, "softmax",
                                                  1.0, bias)
            save(f"grouped_{tag}_{int(renorm)}", logits=logits, bias=bias, k=k, ng=ng, tg=tg,
                 renorm=renorm, w=w, i=i, w_softmax=w2, i_softmax=i2)
    logits = torch.randn(21, 256, generator=g).to(torch.bfloat16)
    bias = (torch.randn(256, generator=g) * 0.01)
    w, i = grouped_topk_op.grouped_topk(logits, logits, 8, True, 8, 4, "sigmoid", 2.5, bias)
    save("grouped_bf16", logits=logits, bias=bias, k=8, ng=8, tg=4, w=w, i=i)

    # ---- align ---------------------------------------------------------
    for tag, (T, k, E, bs) in {"a": (37, 2, 8, 16), "b": (200, 8, 256, 128), "c": (3, 4, 64, 32),
                               "d": (1, 1, 4, 4)}.items():
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
        s, e, n = torch_moe_align_block_size(ids, bs, E)
        emap = torch.full((E,), -1, dtype=torch.int32)
        loc = torch.randperm(E, generator=g)[: max(1, E // 2)].sort().values
        emap[loc] = torch.arange(loc.numel(), dtype=torch.int32)
        sm, em, nm = torch_moe_align_block_size(ids, bs, E, expert_map=emap)
        save(f"align_{tag}", ids=ids, E=E, bs=bs, sorted=s, experts=e, total=n, emap=emap,
             sorted_m=sm, experts_m=em, total_m=nm)

    # ---- remap / gather -------------------------------------------------
    for tag, (T, H, E_tot, k, ep) in {"a": (32, 128, 16, 2, 1), "b": (50, 64, 32, 4, 2)}.items():
        hs = torch.randn(T, H, generator=g).to(torch.bfloat16)
        ids = torch.stack([torch.randperm(E_tot, generator=g)[:k] for _ in range(T)]).to(torch.int64)
        E_loc = E_tot // ep
        emap = None
        if ep > 1:
            emap = torch.full((E_tot,), -1, dtype=torch.int64)
            emap[E_loc: 2 * E_loc] = torch.arange(E_loc)
        out = torch.zeros(T * k, H, dtype=torch.bfloat16)
        rows = torch.zeros(E_loc, dtype=torch.int32)
        rmap = torch.zeros(T, k, dtype=torch.int32)
        ref_remap_hidden_states(hs, None, out, None, emap, rows, rmap, ids, E_tot, E_loc)
        w = torch.rand(T, k, generator=g)
        y = torch.randn(T * k, H, generator=g).to(torch.bfloat16)
        gout = torch.zeros(T, H, dtype=torch.bfloat16)
        ref_moe_gather(gout, y, w, rmap, E_loc)
        save(f"remap_{tag}", hs=hs, ids=ids, emap=emap, E_loc=E_loc, out=out, rows=rows,
             rmap=rmap, w=w, y=y, gout=gout)

    # ---- activations / quant -------------------------------------------
    x = torch.randn(24, 512, generator=g).to(torch.bfloat16) * 3
    save("act", x=x, silu=SiluAndMul().forward_native(x),
         oai=SwigluOAIAndMul().forward_native(x))
    from tests.ops.activation_op import GeluAndMul, Relu2NoMul
    from tests.ops.swiglustep_and_mul_op import SwigluStepAndMul
    xs = {"bf16": x, "f16": x.to(torch.float16), "f32": x.float()}
    arrays = {}
    for tag, xx in xs.items():
        arrays["x_" + tag] = xx
        arrays["gelu_" + tag] = GeluAndMul("none").forward_native(xx)
        arrays["gelu_tanh_" + tag] = GeluAndMul("tanh").forward_native(xx)
        arrays["relu2_" + tag] = Relu2NoMul.forward_native(None, xx)  # its constructor wants the native op
        arrays["swiglustep_" + tag] = SwigluStepAndMul().forward_native(xx)
        # the situ oracle is inline in the reference's test (tests/test_activation.py:98-103)
        for lb in (-1.0, 2.0):
            gate, up = xx.float().chunk(2, dim=-1)
            gate = 1.7 * torch.tanh(gate / 1.7) * torch.sigmoid(gate)
            if lb > 0:
                up = lb * torch.tanh(up / lb)
            arrays[f"situ_{'lin' if lb > 0 else 'raw'}_{tag}"] = (gate * up).to(xx.dtype)
    save("act_more", **arrays)
    x = torch.randn(16, 512, generator=g) * 2
    q, s = ref_per_block_quant(x, 1, 128)
    save("fp8_group", x=x, q=q, s=s)
    x = torch.randn(16, 256, generator=g).to(torch.bfloat16)
    s_e8, q4 = to_mxfp(x, 32, "mxfp4")
    save("mxfp4_ref", x=x, q=q4, s=s_e8, deq=mu.dequant_mxfp4(q4, s_e8.to(torch.float32)))
    # weight dequant helpers
    w8 = (torch.randn(256, 384, generator=g)).to(torch.float8_e4m3fn)
    s8 = torch.rand(2, 3, generator=g) + 0.5
    save("fp8_block_w", w=w8, s=s8, deq=mu.dequant_fp8_block_wei(w8, s8))

    # ---- the "next" operators of the registry ------------------------------
    from tests.test_topk_softplus_sqrt import _torch_topk_softplus_sqrt
    from tests.fused_moe.test_reorder_mxfp_scales import ref_reorder
    logits = torch.randn(29, 64, generator=g)
    bias = torch.randn(64, generator=g) * 0.05
    table = torch.stack([torch.randperm(64, generator=g)[:6] for _ in range(50)]).to(torch.int32)
    iid = torch.randint(0, 50, (29,), generator=g).to(torch.int32)
    pad = torch.rand(29, generator=g) < 0.2
    w1, i1 = _torch_topk_softplus_sqrt(logits, 6, True, 2.5, bias, None, None, pad)
    w2, i2 = _torch_topk_softplus_sqrt(logits, 6, False, 1.0, None, iid, table, None)
    save("softplus_sqrt", logits=logits, bias=bias, table=table, iid=iid, pad=pad, w1=w1, i1=i1, w2=w2, i2=i2)
    rows = [16, 0, 33, 100, 1]
    sc = torch.randint(0, 256, (sum(rows), 8), generator=g, dtype=torch.uint8)
    ref, tot = ref_reorder(sc, rows, 8)
    save("reorder_scales", scales=sc, rows=torch.tensor(rows, dtype=torch.int32), out=ref, total=tot)

    # ---- whole layer, tiny bf16 -----------------------------------------
    T, H, I, E, k = 16, 64, 128, 4, 2
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) / 8).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) / 11).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    tw, ti = topk_op.topk_softmax(None, logits, k, True)
    out = ref_fused_moe(x, w13, None, w2, None, tw.flatten().unsqueeze(1).to(torch.bfloat16),
                        ti.flatten().to(torch.int64), k, "silu", E)
    save("layer_bf16", x=x, w13=w13, w2=w2, tw=tw, ti=ti, out=out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the reference tree>")
    main(sys.argv[1])
