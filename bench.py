#!/usr/bin/env python
"""Benchmark of the FP8 linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c3ref|c4|c5] [--impl reference]

A step is one pass of a layer stack (per-token e4m3 quantisers, FP8 GEMMs and their consumers
in the reference engines' call order) over one batch of synthetic activations.  The default
workload is the pi05 PaliGemma prefix stack (18 layers, M = 816).  With N > 1 every rank runs
its own independent stack (independent robot episodes: data parallel, no collective) and the
reported value is the aggregate.  Prints ONE JSON line on rank 0.

``--impl reference`` times the reference's CPU form of the path (torch per-token quantiser +
dequantise-and-matmul, restated in ``oracle/``) on the host cores over a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "fp8_linear_stack_tflops"
UNIT = "TFLOP/s"
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.t_begin = self.t_end = None

    def begin(self):
        """Mark the start of the timed region (samples outside the marks are dropped)."""
        self.t_begin = time.monotonic()

    def end(self):
        self.t_end = time.monotonic()

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        deadline = time.monotonic() + 5.0   # nvidia-smi needs a moment before its first line
        while self.proc is not None and not self.rows and time.monotonic() < deadline:
            time.sleep(0.05)
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, smax, reasons = [], [], set()
        inside = [r for t, r in self.rows if self.t_begin is None or (self.t_begin <= t <= (self.t_end or t))]
        for r in inside or [r for _, r in self.rows[-1:]]:
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_step(spec, layers, sample_layers, threads):
    """One bounded sample of the reference's CPU form of the path: per linear the torch per-token
    quantiser and dequantise-and-matmul (instinctflash benchmarks/native/fp8_probe.py:32-36),
    over `sample_layers` layers of the stack.  Returns (seconds, flops)."""
    from oracle import oracle as O
    torch.set_num_threads(threads)
    E4M3 = torch.float8_e4m3fn
    t0 = time.perf_counter()
    flops = 0.0
    for lw in layers[:sample_layers]:
        for name, n, k in spec.linears():
            x, wq, ws, b = lw[name]
            amax = x.float().abs().amax(1).clamp_min(1e-8)
            q = (x.float() * (448.0 / amax)[:, None]).to(E4M3)
            O.dequantise_and_matmul(q, amax / 448.0, wq, ws, b)
            flops += 2.0 * spec.M * n * k
    return time.perf_counter() - t0, flops


def build_cpu_sample(spec, sample_layers):
    gen = torch.Generator().manual_seed(spec.seed)
    E4M3 = torch.float8_e4m3fn
    layers = []
    for _ in range(sample_layers):
        lw = {}
        for name, n, k in spec.linears():
            w = torch.randn(n, k, generator=gen) * spec.sigma
            amax = w.abs().amax(1).clamp_min(1e-12)
            ws = amax / 448.0
            wq = (w / ws[:, None]).clamp_(-448, 448).to(E4M3)
            x = torch.randn(spec.M, k, generator=gen).to(torch.bfloat16)
            lw[name] = (x, wq, ws, torch.randn(n, generator=gen) * 0.01)
        layers.append(lw)
    return layers


def run_reference(args, spec, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample_layers = 1
    layers = build_cpu_sample(spec, sample_layers)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_step(spec, layers, sample_layers, threads)
    secs, flops = 0.0, 0.0
    for _ in range(args.steps):
        s, f = cpu_reference_step(spec, layers, sample_layers, threads)
        secs += s
        flops += f
    value = flops / secs / 1e12
    sample = f"{sample_layers} of {spec.layers} layers of {spec.name} per step (all {len(spec.linears())} linears, M={spec.M})"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 (computed in f32 on the CPU)", "data": "synthetic",
        "config": {"workload": workload_name(spec), "note": "CPU dequantise-and-matmul port of the reference path"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(spec):
    names = {"c2": "pi05 PaliGemma prefix stack, 18 layers, M=816, hidden 2048 (qkv 2560, o 2048, gate_up 2x16384 GELU-tanh, down)",
             "c3": "pi05 action-expert stack, 18 layers x 10 flow steps, M=50, hidden 1024",
             "c3ref": "pi05 action-expert stack with the reference engine's true shapes, 18 layers x 10 steps, M=50",
             "c4": "Wan2.2-5B-shape DiT linears, 30 blocks, M=4680, hidden 3072",
             "c5": "Wan-14B-shape DiT linears, 40 blocks, M=16384, hidden 5120"}
    return names.get(spec.name, spec.name)


def run_tensor_parallel(args, spec, dev, dist, rank, world):
    """Strong scaling of one Wan-shape stack over `world` GPUs (total work fixed)."""
    from instinctflash_b200.stack import make_inputs, make_weights
    from instinctflash_b200.tp import Comm, WanTPStack
    if dist is None:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29555")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    torch.manual_seed(1234)   # identical full weights on every rank, sharded afterwards
    weights = make_weights(spec, dev)
    stack = WanTPStack(spec, weights, dev, Comm())
    del weights
    torch.cuda.empty_cache()
    x, attn = make_inputs(spec, dev)
    stack.load(x, attn)
    stream = torch.cuda.current_stream(dev)
    graph = None
    try:
        side = torch.cuda.Stream(dev)
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            stack.forward()
        stream.wait_stream(side)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            stack.forward()
    except Exception:
        graph = None

    def step():
        if graph is not None:
            graph.replay()
        else:
            stack.forward()

    for _ in range(args.warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index) as clocks:
        clocks.begin()
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        dist.barrier()
        torch.cuda.synchronize(dev)
        clocks.end()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    if rank == 0:
        p = world
        D, M = spec.hidden, spec.M
        n_row = 3 if spec.cross else 2
        comm_bytes = spec.layers * n_row * ((4 * M * D) + (M * D + 4 * M) + 4 * M) * (p - 1) / p
        line = {"metric": METRIC, "value": spec.flops() * args.steps / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
                "config": {"workload": workload_name(spec), "parallelism": f"tp{world} (column-split qkv/cross-q/ff1, "
                           "row-split o/cross-o/ff2, NCCL all-reduce-max + fp32 reduce-scatter + all-gather)",
                           "cuda_graph": graph is not None,
                           "nvlink_bytes_per_rank_per_step": comm_bytes},
                "clocks": clocks.summary(), "gpu_launches": None}
        print(json.dumps(line), flush=True)
    # A captured graph holds NCCL work, and tearing the process group down under it has hung
    # (watchdog stuck in event destruction): finish all work, then leave without the teardown.
    torch.cuda.synchronize(dev)
    dist.barrier()
    torch.cuda.synchronize(dev)
    sys.stdout.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--episodes", type=int, default=1,
                    help="c3 only: independent episodes stacked along M on each GPU (rows are independent: "
                         "per-token scales and per-row norms, so this is arithmetically the same as separate runs)")
    ap.add_argument("--persistent", action="store_true",
                    help="c3: the whole stack as one cooperative launch (stack_persistent_kernel) instead of one "
                         "launch per operator (the default: with dependent launches it is the faster of the two)")
    ap.add_argument("--per-op", action="store_true", help="accepted for compatibility: one launch per operator is the default")
    ap.add_argument("--parallel", default="dp", choices=["dp", "tp", "tokens"],
                    help="dp: every rank runs its own stack (default, weak scaling); tp: the Wan-shape stacks "
                         "(c4, c5) are column/row split over the ranks with NCCL all-gather / reduce-scatter; "
                         "tokens: the rows of one stack are split over the ranks (every linear and every row "
                         "operator of the path is row-independent: no collective, strong scaling)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    from instinctflash_b200.stack import SPECS, LinearStack, make_inputs, make_weights
    spec = SPECS[args.workload]
    if args.episodes > 1:
        from instinctflash_b200.stack import StackSpec
        spec = StackSpec(**{**spec.__dict__, "M": spec.M * args.episodes})
    total_flops_all_ranks = None
    if args.parallel == "tokens":
        # strong scaling over tokens: rank r owns rows [r*M/p, (r+1)*M/p) (ceil), full weights everywhere
        from instinctflash_b200.stack import StackSpec
        total_flops_all_ranks = spec.flops()
        spec = StackSpec(**{**spec.__dict__, "M": -(-spec.M // world)})

    if args.impl == "reference":
        run_reference(args, spec, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the FP8 linear path has no CPU fallback")
    from instinctflash_b200 import _lib
    _lib.lib()  # fail loudly when the CUDA library is missing
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    if args.parallel == "tp":
        run_tensor_parallel(args, spec, dev, dist, rank, world)
        return

    weights = make_weights(spec, dev)
    persistent = (spec.kind == "gemma" and not spec.o_in and spec.M <= 128 and args.persistent and not args.per_op)
    if persistent:
        # skinny expert loop: the whole stack is one cooperative launch
        from instinctflash_b200.stack_persistent import PersistentExpertStack

        class _Persistent(PersistentExpertStack):
            def load(self, x, attn=None):
                super().load(x)

            def capture(self):
                self.forward()
                torch.cuda.synchronize(self.dev)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.forward()
                return g

            def _q8(self, cols):
                return (self.q8 if cols == self.spec.hidden else self.q8f)

            def _raw(self, cols):
                return torch.empty(self.spec.M, cols, dtype=torch.bfloat16, device=self.dev)

        stack = _Persistent(spec, weights, dev)
    else:
        stack = LinearStack(spec, weights, dev)
    x_dev, attn = make_inputs(spec, dev)
    x_host = x_dev.cpu().pin_memory()
    out_host = torch.empty(spec.M, spec.hidden, dtype=stack.res.dtype).pin_memory()
    stack.load(x_dev, attn)
    graph = stack.capture()
    launches_per_step = stack.launches_per_forward
    flops = spec.flops()
    stream = torch.cuda.current_stream(dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident timing: inputs in HBM, one graph replay per step --------------------
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.warmup):
            stack.load(x_dev, attn)
            graph.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks.begin()
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        barrier()
        clocks.end()
    ms = e0.elapsed_time(e1)
    clock_summary = clocks.summary()

    # ---- end to end: pinned host activations in, residual stream out, every step ---------------
    x_stage = torch.empty_like(x_dev)
    for _ in range(2):
        x_stage.copy_(x_host, non_blocking=True)
        stack.load(x_stage, attn)
        graph.replay()
        out_host.copy_(stack.res, non_blocking=True)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for _ in range(args.steps):
        x_stage.copy_(x_host, non_blocking=True)
        stack.load(x_stage, attn)
        graph.replay()
        out_host.copy_(stack.res, non_blocking=True)
    f1.record(stream)
    barrier()
    ms_e2e = f0.elapsed_time(f1)

    # ---- dominant kernel: the widest FP8 GEMM of the stack, timed alone over rotating layers ----
    from instinctflash_b200.kernels import fp8 as K
    dom = max(spec.linears(), key=lambda t: t[1] * t[2])
    name, n_dom, k_dom = dom
    a_dom = stack._q8(k_dom)
    out_dom = stack._raw(n_dom)
    reps = max(args.steps, 10)
    for lw in weights[:3]:
        K.gemm(a_dom, lw.w[name], out_dom)
    torch.cuda.synchronize(dev)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record(stream)
    for i in range(reps):
        K.gemm(a_dom, weights[i % len(weights)].w[name], out_dom)
    g1.record(stream)
    torch.cuda.synchronize(dev)
    dom_ms = g0.elapsed_time(g1) / reps
    dom_flops = 2.0 * spec.M * n_dom * k_dom
    dom_bytes = n_dom * k_dom + spec.M * k_dom + 2.0 * spec.M * n_dom
    peaks = measured_peaks()
    tensor_bound = spec.M > 400
    if tensor_bound:
        peak = 2.0 * peaks["bf16_tflops"]   # dense FP8 runs at twice the bf16 rate on the same tensor pipe
        achieved = dom_flops / (dom_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": None, "kernel": f"gemm_fp8_tc5_kernel {spec.M}x{n_dom}x{k_dom} ({name})",
                    "peak_source": f"2 x bf16_tflops of MEASURED_PEAKS.json ({peaks['source']})",
                    "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS, "ms_per_launch": dom_ms}
    else:
        peak = peaks["hbm_gbs"]
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": None, "kernel": f"gemm_fp8_tc5_kernel {spec.M}x{n_dom}x{k_dom} ({name})",
                    "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']})",
                    "frac_of_nominal_8000": achieved / NOMINAL_HBM_GBS, "ms_per_launch": dom_ms}
    if persistent:
        # the step is one launch of the persistent kernel: its algorithmic bytes are every weight
        # matrix once per layer and flow step plus the activations each operator reads and writes
        lin = spec.linears()
        act = sum(spec.M * k + 2.0 * spec.M * n for _, n, k in lin) + spec.M * spec.ffn * 5.0 + spec.M * spec.hidden * 11.0
        step_bytes = (spec.weight_bytes() + act * spec.layers) * spec.steps
        achieved = step_bytes / (ms / args.steps * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                    "kernel": f"stack_persistent_kernel ({spec.layers} layers x {spec.steps} steps, M={spec.M})",
                    "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']})",
                    "frac_of_nominal_8000": achieved / NOMINAL_HBM_GBS, "ms_per_launch": ms / args.steps,
                    "note": "bound by the chain of grid-wide dependencies (4 per layer and step), not by bandwidth"}
    traffic_file = ROOT / "profiles" / "traffic.json"
    if traffic_file.exists():
        roofline["traffic"] = json.loads(traffic_file.read_text()).get(f"{spec.name}:{name}")

    # ---- max over ranks -------------------------------------------------------------------------
    if dist is not None:
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    # ---- CPU baseline (rank 0, N = 1): bounded sample of the same workload ----------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        sample_layers = 1
        layers = build_cpu_sample(spec, sample_layers)
        cpu_reference_step(spec, layers, sample_layers, threads)
        best = None
        spent = 0.0
        while spent < 12.0:
            secs, fl = cpu_reference_step(spec, layers, sample_layers, threads)
            spent += secs
            best = secs if best is None else min(best, secs)
        cpu = {"value": fl / best / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{sample_layers} of {spec.layers} layers of {spec.name} (all {len(spec.linears())} linears, M={spec.M}), "
                         f"best of repeats within 12 s"}

    if rank == 0:
        tokens = args.parallel == "tokens"
        job_flops = total_flops_all_ranks if tokens else world * flops   # rows actually asked for, padding not counted
        value = job_flops * args.steps / (ms * 1e-3) / 1e12
        e2e_value = job_flops * args.steps / (ms_e2e * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if tokens else "weak",
            "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
            "config": {"workload": workload_name(spec) + (f", {args.episodes} episodes stacked along M (M={spec.M})" if args.episodes > 1 else ""),
                       "execution": "persistent whole-stack kernel (one cooperative launch per step)" if persistent else "one launch per operator, CUDA graph",
                       "parallelism": (f"tokens/{world}: rows of one stack split over the ranks ({spec.M} per rank), full "
                                       f"weights on every rank, no collective" if tokens
                                       else f"dp{world} (independent stacks, no collective)"),
                       "l2": f"weights streamed per step ({spec.weight_bytes() / 1e9:.2f} GB) exceed the 126 MB L2",
                       "timing": "one CUDA-graph replay per step, CUDA events on the launching stream"},
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * x_host.element_size(),
                    "d2h_bytes_per_step": out_host.numel() * out_host.element_size(), "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clock_summary,
            "stack_ms": ms / args.steps,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
