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
def make_device_layer(cfg, dev, seed=0, experts=None):
    """Synthetic layer generated on the device (the CPU generator of the oracle is too slow at
    1.4 GB of weights): weights N(0, 1/fan_in) quantised to e4m3 per 128x128 block.  Each
    expert has its own seed, so a rank that owns a slice of the experts builds only those."""
    import vllm_xpu_kernels._C  # noqa: F401
    H, I = cfg["H"], cfg["I"]
    experts = list(range(cfg["E"])) if experts is None else list(experts)

    def quant(K, N):
        qs, ss = [], []
        for e in experts:
            g = torch.Generator(device=dev).manual_seed(seed * 100003 + e * 7 + (K % 5))
            w = torch.randn(K, N, generator=g, device=dev) / K ** 0.5
            blk = w.view(K // 128, 128, N // 128, 128)
            s = (blk.abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-12)
            qs.append((blk / s.view(K // 128, 1, N // 128, 1)).clamp(-448, 448).view(K, N)
                      .to(torch.float8_e4m3fn))
            ss.append(s)
            del w, blk
        return torch.stack(qs), torch.stack(ss)

    w13, s13 = quant(H, 2 * I)
    w2, s2 = quant(I, H)
    return dict(w13=w13, w13_scale=s13, w2=w2, w2_scale=s2)


def make_inputs(cfg, T, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, cfg["H"], generator=g).to(torch.bfloat16)
    logits = torch.randn(T, cfg["E"], generator=g)
    return x, logits


class Layer:
    """Routing + quantisation + XpuFusedMoe.apply, the sequence a caller runs per batch."""

    def __init__(self, cfg, weights, T, dev, group=None):
        from vllm_xpu_kernels.fused_moe_interface import XpuFusedMoe
        from vllm_xpu_kernels.moe_utils import quant_fp8_block_act
        self.cfg, self.T, self.dev = cfg, T, dev
        self.quant = quant_fp8_block_act
        E_loc = weights["w13"].shape[0]
        self.moe = XpuFusedMoe(weights["w13"], weights["w13_scale"], None, weights["w2"],
                               weights["w2_scale"], None, cfg["k"], cfg["activation"], E_loc)
        self.ep = None
        if group is not None:
            from vllm_xpu_kernels.ep import ExpertParallel, make_local_fn
            self.ep = ExpertParallel(group, E_loc, make_local_fn(self.moe))
        k = cfg["k"]
        self.w = torch.empty(T, k, dtype=torch.float32, device=dev)
        self.ids = torch.empty(T, k, dtype=torch.int32, device=dev)
        self.src = torch.empty(T, k, dtype=torch.int32, device=dev)
        self.out = torch.empty(T, cfg["H"], dtype=torch.bfloat16, device=dev)

    def step(self, x, logits):
        torch.ops._moe_C.topk_softmax(self.w, self.ids, self.src, logits, True, None, None)
        xq, xs = self.quant(x)
        if self.ep is not None:
            self.ep.apply(self.out, xq, self.w, self.ids, scales=xs)
        else:
            self.moe.apply(self.out, xq, self.w, self.ids, a1q_scale=xs)
        return self.out


def flops_per_token(cfg):
    return 6.0 * cfg["k"] * cfg["H"] * cfg["I"]


def cpu_layer_step(cfg, layer_cpu, x, logits, O):
    w, ids = O.topk_softmax(logits, cfg["k"], True)
    return O.fused_moe(cfg["recipe"], x, layer_cpu["w13"], layer_cpu["w13_scale"], None,
                       layer_cpu["w2"], layer_cpu["w2_scale"], None, w, ids, cfg["activation"])


def cpu_sample_tokens(cfg):
    return 256


def run_reference(args, cfg):
    """The reference's torch CPU path (restated in oracle/) on this host's cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import moe_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Tc = cpu_sample_tokens(cfg)
    layer = O.make_layer(cfg, T=Tc)
    x, logits = layer["x"], layer["logits"]
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
    par = "1 GPU" if world == 1 else (f"expert-parallel over {world} GPUs ({cfg['E'] // world} experts each), "
                                      "tokens data-parallel, NCCL all-to-all dispatch/combine")
    return {"workload": f"{args.config}: Mixtral-8x7B-shaped fused-MoE layer, FP8 e4m3 weights with "
                        "128x128 fp32 block scales, per-token-group-128 FP8 activations, softmax top-2",
            "parallelism": par, "tokens_per_gpu": cfg["T"], "hidden": cfg["H"], "intermediate": cfg["I"],
            "experts": cfg["E"], "topk": cfg["k"], "l2": "256 MiB buffer written between timed steps"}


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
    args = ap.parse_args()
    from oracle import moe_oracle as O  # workload table (and the CPU baseline leg)
    cfg = dict(O.CONFIGS[args.config])
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
        ms = timed_region(lambda: layer.step(x, logits), args.steps)

        def e2e_step():
            xd = x_pin.to(dev, non_blocking=True)
            ld = logits_pin.to(dev, non_blocking=True)
            out = layer.step(xd, ld)
            out_pin.copy_(out, non_blocking=True)
        e2e_step()
        ms_e2e = timed_region(e2e_step, args.steps)

        # the dominant kernel alone, inside the same step sequence
        layer.moe.stage_timer = gemm_ms
        for _ in range(args.steps):
            flush.fill_(1)
            layer.step(x, logits)
        torch.cuda.synchronize()
        layer.moe.stage_timer = None
    gemm1 = [s.elapsed_time(e) for name, s, e in gemm_ms if name == "gemm1"]
    gemm1_ms = sum(gemm1) / max(len(gemm1), 1)

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = t.tolist()

    if rank == 0:
        peaks = load_peaks()
        R = T * cfg["k"]
        gemm1_flops = 2.0 * R * cfg["H"] * 2 * cfg["I"]
        achieved = gemm1_flops / (gemm1_ms * 1e-3) / 1e12 if gemm1_ms > 0 else 0.0
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        line = {
            "metric": "fused_moe_layer_tokens_per_s", "value": world * T / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": workload_config(args, cfg),
            "tflops": world * T * flops_per_token(cfg) / (ms * 1e-3) / 1e12,
            "e2e": {"value": world * T / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": x_pin.numel() * 2 + logits_pin.numel() * 4,
                    "d2h_bytes_per_step": out_pin.numel() * 2},
            "gpu_launches": (2 + layer.moe.launches_per_apply(T)) * args.steps,  # + topk, quant
            "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (w13, fp8 block-scaled)",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": None,
                         "peak_source": f"2 x {peaks['source']} sustained bf16 cuBLAS rate "
                                        "(fp8 runs at twice the bf16 rate on tcgen05)",
                         "ms_per_launch": gemm1_ms},
            "clocks": clk.summary(),
        }
        if not args.no_cpu_baseline and world == 1:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            Tc = cpu_sample_tokens(cfg)
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
