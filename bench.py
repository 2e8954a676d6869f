"""Fused-MoE layer benchmark: tokens/s of one layer pass on seeded synthetic data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config c1]

One step = routing + activation quantisation + XpuFusedMoe.apply over one batch.
Default workload: the Mixtral-8x7B-shaped FP8 layer (T=4096, H=4096, I=14336,
E=8, top-2, 128x128 block scales), the largest configuration that is quoted on
one GPU.  Prints one JSON line (rank 0).

* ``value``  : tokens/s with inputs already in HBM, CUDA-event timed, max over ranks.
* ``e2e``    : tokens/s through the same public calls with pinned HOST inputs
               copied in and the layer output copied back inside the timed region.
* ``roofline``: the w13 grouped GEMM, FLOPs of one launch / its mean duration
               (CUDA events around that launch inside the timed steps).
* ``cpu_baseline``: the CPU oracle (a port of the reference's torch path) on a
               bounded token sample, on this host's cores.

``--impl reference`` times only that CPU path (rank 0; other ranks exit).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "vllm-xpu-kernels_b200"))

import torch  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum of one w13 GEMM launch, from the ncu capture
# summarised under profiles/ (captured on a 2-expert slice, scaled by the expert count).
TRAFFIC_BYTES_PER_LAUNCH = {"c1": 4 * 269.44e6}  # profiles/grouped_gemm_fp8_c1_small.md

# The benchmark configurations (shapes of BASELINE.json's configs 0-3).
CONFIGS = {
    "c0": dict(T=64, H=1024, I=2048, E=8, k=2, recipe="bf16", routing="softmax", activation="silu",
               bias=False, name="tiny bf16 layer"),
    "c1": dict(T=4096, H=4096, I=14336, E=8, k=2, recipe="fp8block", routing="softmax",
               activation="silu", bias=False,
               name="Mixtral-8x7B-shaped layer, FP8 e4m3 weights with 128x128 fp32 block scales, "
                    "per-token-group-128 FP8 activations, softmax top-2"),
    "c2": dict(T=8192, H=2880, I=2880, E=128, k=4, recipe="mxfp4", routing="softmax",
               activation="swigluoai", bias=True,
               name="gpt-oss-120b-shaped layer, MXFP4 weights (expanded to bf16 once, W4A16), bf16 "
                    "biases, SwigluOAI, softmax top-4"),
    "c3": dict(T=16384, H=7168, I=2048, E=256, k=8, recipe="fp8block", routing="grouped",
               activation="silu", bias=False, n_group=8, topk_group=4, scale=2.5,
               name="DeepSeek-V3-shaped routed experts, FP8 block-scaled, sigmoid + bias grouped "
                    "top-8 (8 groups, 4 kept), scale 2.5; shared expert not included"),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.stop = index, [], threading.Event()

    def _run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                      "--format=csv,noheader,nounits"], capture_output=True,
                                     text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self.stop.wait(0.1)

    def __enter__(self):
        self.t = threading.Thread(target=self._run, daemon=True)
        self.t.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.t.join()

    def summary(self):
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(sm)}


# --------------------------------------------------------------------------------------
def _quant_fp8_block(w):
    K, N = w.shape
    blk = w.view(K // 128, 128, N // 128, 128)
    s = (blk.abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-12)
    q = (blk / s.view(K // 128, 1, N // 128, 1)).clamp(-448, 448).view(K, N).to(torch.float8_e4m3fn)
    return q, s


def _quant_mxfp4(w):
    """[N, K] -> packed e2m1 pairs [N, K/2] + e8m0 [N, K/32], scale rounded up to a power of two,
    values to the nearest code point."""
    N, K = w.shape
    g = w.view(N, K // 32, 32)
    amax = g.abs().amax(-1).clamp_min(1e-30)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    y = (g * torch.exp2(-e).unsqueeze(-1)).clamp(-6.0, 6.0)
    a = y.abs()
    code = torch.zeros_like(a, dtype=torch.uint8)
    for bnd in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        code += (a > bnd).to(torch.uint8)
    code |= (y < 0).to(torch.uint8) << 3
    code = code.view(N, K)
    return (code[:, 1::2] << 4) | code[:, 0::2], (e + 127).to(torch.uint8)


def make_device_layer(cfg, dev, seed=0, experts=None):
    """Synthetic weights generated on the device (the CPU generator of the oracle is too slow
    at GB sizes): N(0, 1/fan_in), quantised per recipe, in the layouts the operators take.
    Each expert has its own seed, so a rank that owns a slice of the experts builds only those."""
    import vllm_xpu_kernels._C  # noqa: F401
    H, I, recipe = cfg["H"], cfg["I"], cfg["recipe"]
    experts = list(range(cfg["E"])) if experts is None else list(experts)

    def build(K, N, tag):
        qs, ss = [], []
        for e in experts:
            g = torch.Generator(device=dev).manual_seed(seed * 100003 + e * 7 + tag)
            w = torch.randn(K, N, generator=g, device=dev) / K ** 0.5
            if recipe == "fp8block":
                q, s = _quant_fp8_block(w)
            elif recipe == "mxfp4":
                q, s = _quant_mxfp4(w.t().contiguous())
            else:
                q, s = w.to(torch.bfloat16), None
            qs.append(q)
            ss.append(s)
            del w
        return torch.stack(qs), (torch.stack(ss) if ss[0] is not None else None)

    w13, s13 = build(H, 2 * I, 1)
    w2, s2 = build(I, H, 2)
    out = dict(w13=w13, w13_scale=s13, w2=w2, w2_scale=s2, w13_bias=None, w2_bias=None)
    if cfg["bias"]:
        g = torch.Generator(device=dev).manual_seed(seed + 17)
        out["w13_bias"] = (torch.randn(len(experts), 2 * I, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        out["w2_bias"] = (torch.randn(len(experts), H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    return out


def make_inputs(cfg, T, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, cfg["H"], generator=g).to(torch.bfloat16)
    logits = torch.randn(T, cfg["E"], generator=g)
    if cfg.get("skew"):  # Zipf-like expert load of the decode sweep
        rank = torch.randperm(cfg["E"], generator=torch.Generator().manual_seed(1)) + 1
        logits = logits + 1.5 * torch.log(1.0 / rank.float())
    return x, logits


class Layer:
    """Routing + quantisation + XpuFusedMoe.apply, the sequence a caller runs per batch."""

    def __init__(self, cfg, weights, T, dev, group=None):
        from vllm_xpu_kernels.fused_moe_interface import XpuFusedMoe
        from vllm_xpu_kernels.moe_utils import quant_fp8_block_act
        self.cfg, self.T, self.dev = cfg, T, dev
        self.quant = quant_fp8_block_act
        E_loc = weights["w13"].shape[0]
        w13, w2 = weights["w13"], weights["w2"]
        if cfg["recipe"] == "mxfp4":
            w13, w2 = w13.view(torch.float4_e2m1fn_x2), w2.view(torch.float4_e2m1fn_x2)
        self.moe = XpuFusedMoe(w13, weights["w13_scale"], weights["w13_bias"], w2, weights["w2_scale"],
                               weights["w2_bias"], cfg["k"], cfg["activation"], E_loc)
        self.ep = None
        self.ep_backend = None
        if group is not None:
            from vllm_xpu_kernels.ep import ExpertParallel, PeerExpertParallel, make_local_fn
            self.ep_backend = os.environ.get("B200MOE_EP", "peer")
            if self.ep_backend == "peer":
                fp8 = cfg["recipe"] == "fp8block"
                self.ep = PeerExpertParallel(group, self.moe, T, cfg["k"], cfg["H"],
                                             cfg["H"] * (1 if fp8 else 2),
                                             (cfg["H"] // 128) * 4 if fp8 else 0, E_loc, dev)
            else:
                self.ep = ExpertParallel(group, E_loc, make_local_fn(self.moe))
        k = cfg["k"]
        self.w = torch.empty(T, k, dtype=torch.float32, device=dev)
        self.ids = torch.empty(T, k, dtype=torch.int32, device=dev)
        self.src = torch.empty(T, k, dtype=torch.int32, device=dev)
        self.out = torch.empty(T, cfg["H"], dtype=torch.bfloat16, device=dev)
        self.score_bias = None
        if cfg["routing"] == "grouped":
            g = torch.Generator().manual_seed(3)
            self.score_bias = (torch.randn(cfg["E"], generator=g) * 0.01).to(dev)

    def route(self, logits):
        cfg = self.cfg
        if cfg["routing"] == "softmax":
            torch.ops._moe_C.topk_softmax(self.w, self.ids, self.src, logits, True, None, None)
            return self.w, self.ids
        return torch.ops._moe_C.grouped_topk(logits, cfg["n_group"], cfg["topk_group"], cfg["k"], True,
                                             cfg["scale"], self.score_bias, 1)

    def step(self, x, logits):
        w, ids = self.route(logits)
        scales = None
        if self.cfg["recipe"] == "fp8block":
            x, scales = self.quant(x)
        if self.ep is not None:
            self.ep.apply(self.out, x, w, ids, scales=scales)
        else:
            self.moe.apply(self.out, x, w, ids, a1q_scale=scales)
        return self.out

    def launches_per_step(self):
        return 1 + (1 if self.cfg["recipe"] == "fp8block" else 0) + self.moe.launches_per_apply(self.T)


def same_dtype_probe(dev, n=8192, iters=10):
    """TFLOP/s of one unscaled e4m3 x e4m3 GEMM of n^3 on the library's own tcgen05 pipeline."""
    a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
    b = torch.randn(1, n, n, device=dev).to(torch.float8_e4m3fn)
    d = torch.empty(n, n, dtype=torch.bfloat16, device=dev)
    rows = torch.tensor([n], dtype=torch.int32, device=dev)
    run = lambda: torch.ops._xpu_C.b200_grouped_gemm(a, None, b, None, None, d, rows, n, n, 1, 0, 0)
    for _ in range(3):
        run()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(iters):
        run()
    e.record()
    torch.cuda.synchronize()
    return 2.0 * n ** 3 / (s.elapsed_time(e) / iters * 1e-3) / 1e12


def flops_per_token(cfg):
    return 6.0 * cfg["k"] * cfg["H"] * cfg["I"]


def cpu_layer_step(cfg, layer_cpu, x, logits, O):
    """One pass of the CPU oracle (a port of the reference's torch path) over a token sample."""
    if cfg["routing"] == "softmax":
        w, ids = O.topk_softmax(logits, cfg["k"], True)
    else:
        bias = torch.randn(cfg["E"], generator=torch.Generator().manual_seed(3)) * 0.01
        w, ids = O.grouped_topk(logits, cfg["k"], True, cfg["n_group"], cfg["topk_group"], "sigmoid",
                                cfg["scale"], bias)
    return O.fused_moe(cfg["recipe"], x, layer_cpu["w13"], layer_cpu["w13_scale"], layer_cpu["w13_bias"],
                       layer_cpu["w2"], layer_cpu["w2_scale"], layer_cpu["w2_bias"], w, ids,
                       cfg["activation"], quant_act=cfg["recipe"] == "fp8block")


def cpu_sample_tokens(cfg):
    """Tokens per CPU pass: sized so one pass is seconds, not minutes, on a 16-core host."""
    return 256 if cfg["E"] <= 8 else 64


def run_reference(args, cfg):
    """The reference's torch CPU path (restated in oracle/) on this host's cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import moe_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Tc = min(cpu_sample_tokens(cfg), cfg["T"])
    layer = make_device_layer(cfg, torch.device("cpu"))
    x, logits = make_inputs(cfg, Tc, seed=0)
    for _ in range(min(args.warmup, 1)):
        cpu_layer_step(cfg, layer, x, logits, O)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_layer_step(cfg, layer, x, logits, O)
    dt = (time.perf_counter() - t0) / args.steps
    v = Tc / dt
    sample = f"{Tc} of {cfg['T']} tokens per step, all {cfg['E']} experts, dequantise-then-fp32-matmul"
    print(json.dumps({
        "impl": "reference", "metric": "fused_moe_layer_tokens_per_s", "value": v, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args, cfg),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(args, cfg):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    how = ("NCCL all-to-all dispatch/combine" if os.environ.get("B200MOE_EP", "peer") == "nccl" else
           "dispatch and combine as stores into peer GPU memory from the library's own kernels "
           "(second GEMM's epilogue writes the combine)")
    par = "1 GPU" if world == 1 else (f"expert-parallel over {world} GPUs ({cfg['E'] // world} experts each), "
                                      f"tokens data-parallel, {how}")
    return {"workload": f"{args.config}: {cfg['name']}", "parallelism": par, "tokens_per_gpu": cfg["T"], "hidden": cfg["H"], "intermediate": cfg["I"],
            "experts": cfg["E"], "topk": cfg["k"],
            "l2": "value: 256 MiB buffer written between timed steps; e2e: no flush, each step streams "
                  "its expert weights (far larger than the 126 MB L2) again"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--config", default="c1")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tokens", type=int, default=0, help="override tokens per GPU (profiling, sweeps)")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count (profiling)")
    ap.add_argument("--skew", action="store_true", help="Zipf-like expert load (decode sweep)")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.skew:
        cfg["skew"] = True
    if args.tokens:
        cfg["T"] = args.tokens
    if args.experts:
        cfg["E"] = args.experts
    if args.impl == "reference":
        return run_reference(args, cfg)

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    T = cfg["T"]
    assert cfg["E"] % world == 0, "the expert count must divide over the ranks"
    per = cfg["E"] // world
    weights = make_device_layer(cfg, dev, experts=range(rank * per, (rank + 1) * per))
    layer = Layer(cfg, weights, T, dev, group=dist.group.WORLD if world > 1 else None)
    x_host, logits_host = make_inputs(cfg, T, seed=rank)
    x_pin, logits_pin = x_host.pin_memory(), logits_host.pin_memory()
    out_pin = torch.empty(T, cfg["H"], dtype=torch.bfloat16).pin_memory()
    x, logits = x_pin.to(dev), logits_pin.to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # per-stage events of the dominant kernel
    gemm_ms = []
    layer.moe.stage_timer = None

    def timed_region(fn, steps):
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(steps)]
        barrier()
        for s, e in evs:
            flush.fill_(1)
            s.record()
            fn()
            e.record()
        barrier()
        return sum(s.elapsed_time(e) for s, e in evs) / steps

    for _ in range(args.warmup):
        layer.step(x, logits)
    barrier()

    with ClockSampler(local) as clk:
        # The dominant kernel (w13 grouped GEMM) carries its own event pair inside the timed
        # steps, so its duration is taken under exactly the clocks `value` is taken under.
        gemm1_ev = []
        layer.moe.stage_timer, layer.moe.stage_only = gemm1_ev, {"gemm1"}
        ms = timed_region(lambda: layer.step(x, logits), args.steps)
        layer.moe.stage_timer, layer.moe.stage_only = None, None

        # the same step sequence once more with an event pair around every stage, for the
        # per-stage breakdown (`stages_ms`; later in the run, so under a warmer power state)
        layer.moe.stage_timer = gemm_ms
        for _ in range(args.steps):
            flush.fill_(1)
            layer.step(x, logits)
        torch.cuda.synchronize()
        layer.moe.stage_timer = None

        def e2e_region(steps):
            """K steps through the public calls from pinned host buffers: each step's x and
            logits are copied in, its [T, H] result is copied out.  Copies run on their own
            streams so step i+1's upload and step i-1's download overlap step i's kernels
            (double-buffered device tensors), as a serving loop would arrange it."""
            main = torch.cuda.current_stream()
            s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
            xd = [torch.empty_like(x) for _ in range(2)]
            ld = [torch.empty_like(logits) for _ in range(2)]
            od = [torch.empty_like(layer.out) for _ in range(2)]
            ev_in, ev_comp, ev_out = [None] * steps, [None] * steps, [None] * steps
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            start.record(main)
            s_in.wait_stream(main)
            s_out.wait_stream(main)
            for i in range(steps):
                b = i % 2
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev_comp[i - 2])
                    xd[b].copy_(x_pin, non_blocking=True)
                    ld[b].copy_(logits_pin, non_blocking=True)
                    ev_in[i] = torch.cuda.Event()
                    ev_in[i].record(s_in)
                main.wait_event(ev_in[i])
                if i >= 2:
                    main.wait_event(ev_out[i - 2])
                layer.out = od[b]
                layer.step(xd[b], ld[b])
                ev_comp[i] = torch.cuda.Event()
                ev_comp[i].record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp[i])
                    out_pin.copy_(od[b], non_blocking=True)
                    ev_out[i] = torch.cuda.Event()
                    ev_out[i].record(s_out)
            main.wait_stream(s_out)
            end.record(main)
            barrier()
            return start.elapsed_time(end) / steps
        e2e_region(2)
        ms_e2e = e2e_region(args.steps)

    gemm1 = [s.elapsed_time(e) for name, s, e in gemm1_ev if name == "gemm1"]
    gemm1_ms = sum(gemm1) / max(len(gemm1), 1)
    stages = {}
    for name, s, e in gemm_ms:
        stages.setdefault(name, []).append(s.elapsed_time(e))
    stages = {k: round(sum(v) / len(v), 4) for k, v in stages.items()}

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = t.tolist()

    if rank == 0:
        peaks = load_peaks()
        R = T * cfg["k"]
        gemm1_flops = 2.0 * R * cfg["H"] * 2 * cfg["I"]
        achieved = gemm1_flops / (gemm1_ms * 1e-3) / 1e12 if gemm1_ms > 0 else 0.0
        fp8 = cfg["recipe"] == "fp8block"
        peak = (2.0 if fp8 else 1.0) * peaks["bf16_tflops_sustained"]
        # distinct experts this batch touches: in the decode regime the layer streams their weights
        # once and the w13 GEMM is bound by HBM, not by the tensor pipe
        _, ids_now = layer.route(logits)
        active = int(torch.unique(ids_now).numel())
        wbytes = {"fp8block": 1.0, "bf16": 2.0, "mxfp4": 2.0}[cfg["recipe"]]
        gemm1_bytes = (active * cfg["H"] * 2 * cfg["I"] * wbytes
                       + (active * (cfg["H"] // 128) * (2 * cfg["I"] // 128) * 4 if fp8 else 0)
                       + R * cfg["H"] * (1 if fp8 else 2) + R * cfg["I"] * (1 if fp8 else 2))
        decode = R / max(active, 1) < 64
        line = {
            "metric": "fused_moe_layer_tokens_per_s", "value": world * T / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"fp8block": "fp8_e4m3 (fp32 accumulate)", "bf16": "bf16 (fp32 accumulate)",
                      "mxfp4": "mxfp4 weights as bf16 x bf16 (fp32 accumulate)"}[cfg["recipe"]],
            "data": "synthetic",
            "config": workload_config(args, cfg),
            "tflops": world * T * flops_per_token(cfg) / (ms * 1e-3) / 1e12,
            "e2e": {"value": world * T / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": x_pin.numel() * 2 + logits_pin.numel() * 4,
                    "d2h_bytes_per_step": out_pin.numel() * 2},
            "gpu_launches": layer.launches_per_step() * args.steps,
            "roofline": {"bound": "tensor",
                         "kernel": "grouped_gemm_kernel (w13" + (", fp8 block-scaled, fused SiLU*mul + "
                                                                 "group quantisation)" if fp8 else ")"),
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": TRAFFIC_BYTES_PER_LAUNCH.get(args.config)
                         if not (args.tokens or args.experts) else None,
                         "peak_source": (f"2 x {peaks['source']} sustained bf16 cuBLAS rate (fp8 issues at "
                                         "twice the bf16 rate on tcgen05; MEASURED_PEAKS has no fp8 figure)")
                         if fp8 else f"{peaks['source']} sustained bf16 cuBLAS rate",
                         "flops_per_launch": gemm1_flops, "ms_per_launch": gemm1_ms},
            "clocks": clk.summary(),
            "stages_ms": stages, "active_experts": active,
        }
        # the streaming stages either side of the GEMMs: algorithmic bytes / stage time
        b_in = 1 if fp8 else 2
        H = cfg["H"]
        stream_bytes = {
            "remap": T * H * b_in + R * H * b_in + (R + T) * (H // 128) * 4 * (1 if fp8 else 0) + T * cfg["k"] * 8,
            "gather": R * H * 2 + T * H * 2 + T * cfg["k"] * 8,
        }
        line["hbm_stages"] = {
            name: {"gbs": round(stream_bytes[name] / (stages[name] * 1e-3) / 1e9, 1),
                   "frac_of_measured_copy": round(stream_bytes[name] / (stages[name] * 1e-3) / 1e9 / peaks["hbm_gbs"], 3),
                   "bytes": stream_bytes[name], "ms": stages[name]}
            for name in stream_bytes if stages.get(name)}
        nominal = 4500.0 if fp8 else 2250.0   # dense TFLOP/s of the part's data sheet
        line["roofline"]["frac_of_nominal"] = achieved / nominal
        line["roofline"]["nominal_peak"] = nominal
        if fp8 and world == 1 and not decode:
            # Same-dtype ceiling measured in this run: one plain e4m3 x e4m3 problem of 8192^3
            # (unit scales, so no per-K-block promotion) through the same kernel family.
            probe = same_dtype_probe(dev)
            line["roofline"]["same_dtype_probe"] = {
                "tflops": probe, "what": "plain tcgen05 e4m3 GEMM, M=N=K=8192, unit scales, bf16 out"}
            line["roofline"]["frac_of_probe"] = achieved / probe if probe > 0 else None
        if decode and gemm1_ms > 0:
            gbs = gemm1_bytes / (gemm1_ms * 1e-3) / 1e9
            line["roofline"] = {"bound": "hbm", "kernel": "grouped_gemm_kernel (w13), weight streaming",
                                "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                                "peak_source": f"{peaks['source']} copy bandwidth",
                                "bytes_per_launch": gemm1_bytes, "ms_per_launch": gemm1_ms}
        if not args.no_cpu_baseline and world == 1:
            from oracle import moe_oracle as O  # CPU-baseline leg only
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            Tc = min(cpu_sample_tokens(cfg), T)
            cpu_layer = {k: (v.cpu() if v is not None else None) for k, v in weights.items()}
            xs, ls = x_host[:Tc], logits_host[:Tc]
            t0 = time.perf_counter()
            cpu_layer_step(cfg, cpu_layer, xs, ls, O)
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {
                "value": Tc / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
                "sample": f"first {Tc} of {T} tokens, one pass, all {cfg['E']} experts "
                          "(dequantise-then-fp32 matmul per expert)"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
