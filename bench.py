#!/usr/bin/env python
"""Benchmark of the FP8 linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c3ref|c4|c5]
                    [--impl reference] [--parallel dp|tp|tokens] [--no-configs] [--no-sharded]

A step is one pass of a layer stack (per-token e4m3 quantisers, FP8 GEMMs and their consumers in
the reference engines' call order) over one batch of synthetic activations.  The default workload
is the pi05 PaliGemma prefix stack (18 layers, M = 816).  With N > 1 every rank runs its own
independent stack (independent robot episodes: data parallel, no collective) and the reported
value is the aggregate.  Prints ONE JSON line on rank 0.

Beside the headline the line carries
  * ``gpu_reference``: the reference's own GPU kernels (its Triton row kernels and
    ``torch._scaled_mm``, imported unmodified from ``baseline/_ref``) run through the same stack
    driver and CUDA graph, timed interleaved with this build (A-B-B-A);
  * ``configs``: short runs of the other benchmark configurations in the same process, each with
    its roofline fraction and its ratio against the reference's GPU kernels;
  * ``sharded``: the splits of the configurations that shard -- 64 independent action-expert
    episodes divided over the ranks (no collective), the Wan-shape stack split over tokens (no
    collective) and tensor parallel (NCCL) -- measured at this N (strong scaling);
  * ``roofline``, ``cpu_baseline``, ``e2e``, ``clocks`` as the contract asks.

``--impl reference`` times the reference's CPU form of the path (torch per-token quantiser +
dequantise-and-matmul, restated in ``oracle/``) on the host cores over a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path
from types import SimpleNamespace

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "fp8_linear_stack_tflops"
UNIT = "TFLOP/s"
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0
EPISODES = 64           # independent action-expert episodes of the sharded c3 configuration
EPISODE_BRANCHES = 8    # episodes in flight on one GPU (parallel branches of one CUDA graph)


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


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU form of the path
# ------------------------------------------------------------------------------------------------
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


# ------------------------------------------------------------------------------------------------
# GPU helpers
# ------------------------------------------------------------------------------------------------
def reference_gpu_ops():
    """The reference's own GPU operators (unmodified, from ``baseline/_ref``) with the signatures the
    stack driver calls, or (None, reason)."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "instinctflash").is_dir():
        return None, "the reference is not installed under baseline/_ref"
    if str(ref) not in sys.path:
        sys.path.insert(0, str(ref))
    try:
        from instinctflash.kernels import activation as RA
        from instinctflash.kernels import fp8 as RF
        from instinctflash.kernels import norm as RN
    except Exception as exc:   # noqa: BLE001
        return None, f"the reference's kernel modules do not import: {exc}"
    return SimpleNamespace(gemm=RF.gemm, row_quant=RN.row_quant, dequant_rows=RN.dequant_rows,
                           residual_norm_quant=RN.residual_norm_quant, gated_act_quant=RA.gated_act_quant,
                           GELU_TANH=RA.GELU_TANH, Fp8Weight=RF.Fp8Weight), None


def replay_ms(graph, n, stream, dev):
    """Device time of n back-to-back replays, CUDA events on the launching stream."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    e0.record(stream)
    for _ in range(n):
        graph.replay()
    e1.record(stream)
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1)


def abba(native, reference, n, stream, dev):
    """native, reference, reference, native: n replays each; (native ms, reference ms) per replay."""
    a1 = replay_ms(native, n, stream, dev)
    b1 = replay_ms(reference, n, stream, dev)
    b2 = replay_ms(reference, n, stream, dev)
    a2 = replay_ms(native, n, stream, dev)
    return (a1 + a2) / (2 * n), (b1 + b2) / (2 * n)


def check_no_timeout(dev):
    """Every wait inside the tcgen05 kernels is bounded; a wait that ran out left a record and an
    incomplete output.  A benchmark number from such a run is worthless: fail."""
    from instinctflash_b200 import _lib
    rec = ctypes.c_uint32(0)
    st = _lib.lib().iflb200_gemm_take_timeout_record(ctypes.byref(rec), torch.cuda.current_stream(dev).cuda_stream)
    if st != 0 or rec.value != 0:
        raise SystemExit(f"a wait inside a GEMM kernel timed out during the benchmark (status {st}, record {rec.value:#x})")


def measure_fp8_peak(dev, seconds=2.0):
    """torch._scaled_mm (cuBLASLt) e4m3 8192^3 with unit scales: best of 10 single launches (burst)
    and back to back for `seconds` (sustained).  The measured FP8 tensor peak of this GPU, this run."""
    n = 8192
    a = (torch.randn(n, n, device=dev) * 0.5).to(torch.float8_e4m3fn)
    b = (torch.randn(n, n, device=dev) * 0.5).to(torch.float8_e4m3fn)
    one = torch.ones((), device=dev)
    out = torch.empty(n, n, device=dev, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream(dev)

    def mm():
        torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=out)
    for _ in range(3):
        mm()
    best = None
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        mm()
        e1.record(stream)
        torch.cuda.synchronize(dev)
        t = e0.elapsed_time(e1)
        best = t if best is None else min(best, t)
    flops = 2.0 * n ** 3
    reps = max(10, int(seconds * 1e3 / best))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        mm()
    e1.record(stream)
    torch.cuda.synchronize(dev)
    sustained = e0.elapsed_time(e1) / reps
    return {"burst_tflops": flops / (best * 1e-3) / 1e12, "sustained_tflops": flops / (sustained * 1e-3) / 1e12,
            "how": f"torch._scaled_mm e4m3 {n}^3, unit scales, bf16 out: best of 10 / {reps} back to back"}


def stack_bytes(spec):
    """Algorithmic bytes of one pass: per linear N*K + 4N + M*K + 4M + 2*M*N, plus the quantisers'
    3*M*K + 4M, over all layers and flow steps."""
    per_layer = 0.0
    for _, n, k in spec.linears():
        per_layer += n * k + 4.0 * n + spec.M * k + 4.0 * spec.M + 2.0 * spec.M * n
        per_layer += 3.0 * spec.M * k + 4.0 * spec.M
    return per_layer * spec.layers * spec.steps


def time_config(spec, dev, ref_ops, steps, warmup, *, persistent=False):
    """Short run of one configuration: this build and, when available, the reference's GPU kernels,
    through the same driver and CUDA graph, interleaved.  Returns a dict for the JSON line."""
    from instinctflash_b200.stack import LinearStack, make_inputs, make_weights
    stream = torch.cuda.current_stream(dev)
    weights = make_weights(spec, dev)
    x, attn = make_inputs(spec, dev)
    st = LinearStack(spec, weights, dev)
    st.load(x, attn)
    g = st.capture()
    for _ in range(warmup):
        g.replay()
    out = {"workload": workload_name(spec), "launches_per_step": st.launches_per_forward}
    g_ref = None
    if ref_ops is not None:
        try:
            st_ref = LinearStack(spec, weights, dev, ops=ref_ops)
            st_ref.load(x, attn)
            g_ref = st_ref.capture()
            for _ in range(warmup):
                g_ref.replay()
        except Exception as exc:   # noqa: BLE001
            out["gpu_reference"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
            g_ref = None
    if g_ref is not None:
        ms, ms_ref = abba(g, g_ref, steps, stream, dev)
        out["gpu_reference"] = {"ms_per_step": ms_ref, "ratio": ms_ref / ms}
    else:
        ms = replay_ms(g, 2 * steps, stream, dev) / (2 * steps)
    out["ms_per_step"] = ms
    out["tflops"] = spec.flops() / (ms * 1e-3) / 1e12
    peaks = measured_peaks()
    if spec.M > 400:
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        out["roofline"] = {"bound": "tensor", "frac": out["tflops"] / peak, "peak": peak, "unit": UNIT,
                           "peak_source": "2 x bf16_tflops_sustained (a whole stack is a long step)",
                           "frac_of_nominal_4500": out["tflops"] / NOMINAL_FP8_TFLOPS}
    else:
        gbs = stack_bytes(spec) / (ms * 1e-3) / 1e9
        out["roofline"] = {"bound": "hbm", "frac": gbs / peaks["hbm_gbs"], "achieved": gbs, "peak": peaks["hbm_gbs"],
                           "unit": "GB/s", "frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS}
    if persistent:
        from instinctflash_b200.stack_persistent import PersistentExpertStack
        ps = PersistentExpertStack(spec, weights, dev)
        ps.load(x)
        ps.forward()
        torch.cuda.synchronize(dev)
        gp = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gp):
            ps.forward()
        for _ in range(warmup):
            gp.replay()
        out["persistent_kernel_ms_per_step"] = replay_ms(gp, 2 * steps, stream, dev) / (2 * steps)
        if ps.timeout_record() != 0:
            raise SystemExit(f"a wait inside the persistent kernel timed out: {ps.timeout_record():#x}")
        del ps, gp
    del st, g, g_ref, weights
    torch.cuda.empty_cache()
    return out


def qkv_consumer_calls(dev, which, ref=False):
    """The consumers of a fused QKV accumulator at benchmark sizes, as zero-argument callables over
    rotated inputs larger than L2: ``qkv_split`` at the C2 prefix shape (816 tokens, 8 + 2x1 heads of
    256: instinctflash/engines/pi05/engine.py:200-201) and ``wan_qkv`` at the C5 shape (2 x 8192
    tokens, 40 heads of 128, q/k norm, three-axis rotary, pooled K/V:
    instinctflash/engines/wan_va/engine.py:215-217).  ``ref``: the reference's Triton kernels."""
    if ref:
        ref_root = ROOT / "baseline" / "_ref"
        if str(ref_root) not in sys.path:
            sys.path.insert(0, str(ref_root))
        from instinctflash.kernels.rope import qkv_split, rope_inv_freq
        from instinctflash.kernels.wan import wan_qkv
    else:
        from instinctflash_b200.kernels.rope import qkv_split, rope_inv_freq
        from instinctflash_b200.kernels.wan import wan_qkv
    g = torch.Generator(device=dev).manual_seed(7)
    if which == "qkv_split":
        T, HQ, HKV, HD = 816, 8, 1, 256
        W = (HQ + 2 * HKV) * HD
        copies = 48                                            # 48 x 4.2 MB of accumulators: 200 MB
        raws = [torch.randn(T, W, device=dev, generator=g).to(torch.bfloat16) for _ in range(copies)]
        row = torch.rand(T, device=dev, generator=g) * 0.02
        col = torch.rand(W, device=dev, generator=g)
        inv = rope_inv_freq(HD, 10000.0, dev)
        pos = torch.arange(T, device=dev).float()[:, None].contiguous()
        q = torch.empty(T, HQ, HD, device=dev, dtype=torch.float16)
        k = torch.empty(1024, HKV, HD, device=dev, dtype=torch.float16)
        v = torch.empty_like(k)
        kw = dict(heads_q=HQ, heads_kv=HKV, head_dim=HD, row=row, col=col, inv_freq=inv, pos=pos)
        calls = [lambda r=r: qkv_split(r, q, k, v, **kw) for r in raws]
        return calls, T * W * 4.0, f"qkv_split {T} x {W} bf16 -> f16 heads, row/col scales, rotary"
    B, T, H, HD = 2, 8192, 40, 128
    D, R = H * HD, B * T
    raws = [torch.randn(R, 3 * D, device=dev, generator=g).to(torch.bfloat16) for _ in range(2)]   # 2 x 503 MB
    row = torch.rand(R, device=dev, generator=g) * 0.02
    col = torch.rand(3 * D, device=dev, generator=g)
    bias = torch.randn(3 * D, device=dev, generator=g)
    qn = torch.rand(D, device=dev, generator=g) + 0.5
    kn = torch.rand(D, device=dev, generator=g) + 0.5
    inv = rope_inv_freq(HD, 10000.0, dev)
    pos = (torch.rand(T, 3, device=dev, generator=g) * 60).floor()
    sec = (torch.arange(HD // 2, device=dev) % 3).int()
    q = torch.empty(R, D, device=dev, dtype=torch.float16)
    kp = torch.empty(B, T, D, device=dev, dtype=torch.float16)
    vp = torch.empty_like(kp)
    kw = dict(heads=H, head_dim=HD, tokens=T, k_pool=kp, v_pool=vp, row=row, col=col, bias=bias, q_norm=qn, k_norm=kn,
              pos=pos, sections=sec, inv_freq=inv)
    calls = [lambda r=r: wan_qkv(r, q, **kw) for r in raws]
    return calls, R * 3 * D * 4.0, f"wan_qkv {R} x {3 * D} bf16 -> f16 q + pooled k/v, scales, bias, q/k norm, 3-axis rotary"


def time_qkv_consumers(dev, with_reference):
    """µs per launch of the two QKV consumers (CUDA events around a graph of launches over rotated
    inputs), this build and -- when the reference imports -- its Triton kernels, A-B-B-A."""
    stream = torch.cuda.current_stream(dev)
    peaks = measured_peaks()
    out = {}
    for which in ("qkv_split", "wan_qkv"):
        def graph_of(calls):
            side = torch.cuda.Stream(dev)
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                for c in calls:
                    c()
            stream.wait_stream(side)
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for c in calls:
                    c()
            return gr
        calls, nbytes, what = qkv_consumer_calls(dev, which)
        gn = graph_of(calls)
        gn.replay()
        entry = {"workload": what}
        gr = None
        if with_reference:
            try:
                rcalls, _, _ = qkv_consumer_calls(dev, which, ref=True)
                gr = graph_of(rcalls)
                gr.replay()
            except Exception as exc:   # noqa: BLE001
                entry["gpu_reference"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:160]}
        n = 5
        if gr is not None:
            ms, ms_ref = abba(gn, gr, n, stream, dev)
            entry["gpu_reference"] = {"us_per_launch": ms_ref / len(calls) * 1e3, "ratio": ms_ref / ms}
        else:
            ms = replay_ms(gn, 2 * n, stream, dev) / (2 * n)
        us = ms / len(calls) * 1e3
        gbs = nbytes / (us * 1e-6) / 1e9
        entry.update({"us_per_launch": us, "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"],
                                                        "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"]}})
        out[which] = entry
        del calls, gn, gr
        torch.cuda.empty_cache()
    return out


def time_single_linear(dev, ref_ops, steps, warmup):
    """Configuration 1: one FP8 linear, x bf16 [64, 1024] -> per-token quantiser -> [4096, 1024]
    weight + bias -> bf16.  Thirty-two weight copies are rotated so the 4 MB weight is not served
    from L2 (134 MB per pass)."""
    from instinctflash_b200.kernels import fp8, norm
    E4M3 = torch.float8_e4m3fn
    M, K, N, copies = 64, 1024, 4096, 32
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    ws = []
    for _ in range(copies):
        w = torch.randn(N, K, device=dev, generator=g) * 0.02
        ws.append(fp8.quantize_weight(w, torch.randn(N, device=dev, generator=g) * 0.01))
    q = torch.empty(M, K, device=dev, dtype=E4M3)
    s = torch.empty(M, device=dev)
    raw = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream(dev)

    def native():
        for w in ws:
            norm.row_quant(x, q, s)
            fp8.fp8_linear(q, s, w, y)

    def reference():
        for w in ws:
            ref_ops.row_quant(x, q, s)
            ref_ops.gemm(q, ref_ops.Fp8Weight(w.w, w.scale, w.bias), raw)
            ref_ops.dequant_rows(raw, y, row=s, col=w.scale, bias=w.bias)

    def capture(fn):
        side = torch.cuda.Stream(dev)
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            fn()
            fn()
        stream.wait_stream(side)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            fn()
        return gr
    gn = capture(native)
    for _ in range(warmup):
        gn.replay()
    out = {"workload": "single FP8 linear 64 x 4096 x 1024 with bias, quantiser + fused GEMM epilogue, 32 rotated weights",
           "launches_per_step": 2 * copies}
    if ref_ops is not None:
        gr = capture(reference)
        for _ in range(warmup):
            gr.replay()
        ms, ms_ref = abba(gn, gr, steps, stream, dev)
        out["gpu_reference"] = {"us_per_linear": ms_ref / copies * 1e3, "ratio": ms_ref / ms}
    else:
        ms = replay_ms(gn, 2 * steps, stream, dev) / (2 * steps)
    us = ms / copies * 1e3
    nbytes = N * K + 8.0 * N + 3.0 * M * K + 8.0 * M + 2.0 * M * N
    peaks = measured_peaks()
    gbs = nbytes / (us * 1e-6) / 1e9
    out.update({"us_per_linear": us, "tflops": 2.0 * M * N * K / (us * 1e-6) / 1e12,
                "roofline": {"bound": "hbm", "frac": gbs / peaks["hbm_gbs"], "achieved": gbs, "peak": peaks["hbm_gbs"],
                             "unit": "GB/s", "frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS}})
    return out


# ------------------------------------------------------------------------------------------------
# Sharded configurations (strong scaling over the ranks of this run)
# ------------------------------------------------------------------------------------------------
def max_over_ranks(ms, dist, dev):
    if dist is None:
        return ms
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def sharded_c3_episodes(dev, dist, rank, world, steps, warmup, max_branches=EPISODE_BRANCHES):
    """64 independent action-expert episodes (M = 50 each, 18 layers x 10 flow steps), 64 / p per
    GPU, no collective.  On each GPU up to 8 episodes are in flight as parallel branches of one CUDA
    graph (every GEMM still has M = 50 rows; branches that reach the same layer together find its
    weights in L2)."""
    from instinctflash_b200.stack import SPECS, EpisodeBatch, make_inputs, make_weights
    spec = SPECS["c3"]
    mine = EPISODES // world + (1 if rank < EPISODES % world else 0)
    branches = min(max_branches, max(1, mine))
    rounds = -(-mine // branches)
    weights = make_weights(spec, dev)
    x, attn = make_inputs(spec, dev)
    batch = EpisodeBatch(spec, weights, dev, branches)
    batch.load(x, attn)
    g = batch.capture()
    stream = torch.cuda.current_stream(dev)
    for _ in range(warmup):
        g.replay()
    if dist is not None:
        dist.barrier()
    ms = replay_ms(g, rounds * steps, stream, dev) / steps      # all of this rank's episodes, once
    ms = max_over_ranks(ms, dist, dev)
    per_episode_bytes = stack_bytes(spec)
    peaks = measured_peaks()
    out = {"episodes": EPISODES, "episodes_per_rank": mine, "branches_per_gpu": branches, "ms_all_episodes": ms,
           "episodes_per_s": EPISODES / (ms * 1e-3), "ms_per_episode_per_gpu": ms / max(1, mine),
           "algorithmic_gbs_per_gpu": per_episode_bytes * mine / (ms * 1e-3) / 1e9,
           "frac_of_hbm_peak": per_episode_bytes * mine / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
           "note": "algorithmic bytes count every weight once per episode and flow step; branches that share a layer's "
                   "weights through L2 read less from DRAM than that", "collective": "none"}
    del batch, g, weights
    torch.cuda.empty_cache()
    return out


def sharded_c4_tokens(dev, dist, rank, world, steps, warmup):
    """The Wan2.2-5B-shape stack with its M = 4680 rows split over the ranks: every operator of the
    path is row-independent and the weights fit every GPU, so there is no collective."""
    from instinctflash_b200.stack import SPECS, LinearStack, StackSpec, make_inputs, make_weights
    full = SPECS["c4"]
    spec = StackSpec(**{**full.__dict__, "M": -(-full.M // world)})
    weights = make_weights(spec, dev)
    x, attn = make_inputs(spec, dev)
    st = LinearStack(spec, weights, dev)
    st.load(x, attn)
    g = st.capture()
    stream = torch.cuda.current_stream(dev)
    for _ in range(warmup):
        g.replay()
    if dist is not None:
        dist.barrier()
    ms = max_over_ranks(replay_ms(g, steps, stream, dev) / steps, dist, dev)
    out = {"rows_per_rank": spec.M, "ms_per_step": ms, "tflops": full.flops() / (ms * 1e-3) / 1e12, "collective": "none"}
    del st, g, weights
    torch.cuda.empty_cache()
    return out


def _time_tp_stack(stack, dev, dist, steps, warmup):
    """ms per pass of a tensor-parallel stack (graph replay when capture works), max over ranks."""
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
    except Exception:   # noqa: BLE001
        graph = None
    runner = graph if graph is not None else SimpleNamespace(replay=stack.forward)
    for _ in range(warmup):
        runner.replay()
    if dist is not None:
        dist.barrier()
    ms = max_over_ranks(replay_ms(runner, steps, stream, dev) / steps, dist, dev)
    if stack.link is not None:
        stack.link.check()
    return ms, graph


def sharded_c4_tp(dev, dist, rank, world, steps, warmup):
    """The Wan2.2-5B-shape stack tensor parallel: column-split qkv / cross-q / ff1, row-split
    o / cross-o / ff2; the exchange steps over peer memory (the GEMM's stores into the row owner's
    planes, single-CTA barrier kernels), with the NCCL transport timed beside it."""
    from instinctflash_b200.stack import SPECS, make_inputs, make_weights
    from instinctflash_b200.tp import Comm, PeerLink, WanTPStack
    spec = SPECS["c4"]
    if spec.M % world:
        return {"unavailable": f"M={spec.M} is not divisible by {world}"}
    torch.manual_seed(1234)   # identical full weights on every rank, sharded afterwards
    weights = make_weights(spec, dev)
    comm = Comm() if dist is not None else Comm.single()
    x, attn = make_inputs(spec, dev)
    out, keep = {}, []
    link, why = None, None
    if world > 1:
        try:
            link = PeerLink(WanTPStack.peer_layout(spec, world), dev)
        except Exception as exc:   # noqa: BLE001
            why = f"{type(exc).__name__}: {exc}"[:200]
        ok = torch.tensor([1.0 if link is not None else 0.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0.0:
            link = None
    stacks = [("nccl", None)] + ([("peer", link)] if link is not None else [])
    for name, lk in stacks:
        stack = WanTPStack(spec, weights, dev, comm, link=lk)
        stack.load(x, attn)
        ms, graph = _time_tp_stack(stack, dev, dist, steps, warmup)
        out[name] = {"ms_per_step": ms, "tflops": spec.flops() / (ms * 1e-3) / 1e12, "cuda_graph": graph is not None,
                     "nvlink_bytes_per_rank_per_step": stack.comm_bytes_per_step(), "collective": stack.collectives}
        keep.append((stack, graph))
    del weights
    best = min(out, key=lambda k: out[k]["ms_per_step"])
    res = dict(out[best], transport=best if world > 1 else "none")
    if world > 1:
        res["transports"] = {k: {"ms_per_step": v["ms_per_step"]} for k, v in out.items()}
        if why:
            res["peer_unavailable"] = why
    res["_keep"] = keep
    return res


# ------------------------------------------------------------------------------------------------
def run_tensor_parallel(args, spec, dev, dist, rank, world):
    """--parallel tp: strong scaling of one Wan-shape stack over `world` GPUs as the headline."""
    from instinctflash_b200.stack import make_inputs, make_weights
    from instinctflash_b200.tp import Comm, WanTPStack
    torch.manual_seed(1234)
    weights = make_weights(spec, dev)
    stack = WanTPStack(spec, weights, dev, Comm() if dist is not None else Comm.single())
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
    except Exception:   # noqa: BLE001
        graph = None
    runner = graph if graph is not None else SimpleNamespace(replay=stack.forward)
    for _ in range(args.warmup):
        runner.replay()
    if dist is not None:
        dist.barrier()
    with ClockSampler(dev.index) as clocks:
        clocks.begin()
        ms = replay_ms(runner, args.steps, stream, dev)
        clocks.end()
    ms = max_over_ranks(ms, dist, dev)
    check_no_timeout(dev)
    if rank == 0:
        line = {"metric": METRIC, "value": spec.flops() * args.steps / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
                "config": {"workload": workload_name(spec), "parallelism": f"tp{world}: " + stack.collectives,
                           "cuda_graph": graph is not None,
                           "nvlink_bytes_per_rank_per_step": stack.comm_bytes_per_step()},
                "clocks": clocks.summary(), "gpu_launches": None}
        print(json.dumps(line), flush=True)
    leave(dev, dist)


def profile_operator(args, spec, dev):
    """One layer of the workload and `--steps` launches of one operator, nothing timed: the small,
    self-ending program a profiler capture wants."""
    from instinctflash_b200.kernels import fp8 as K
    from instinctflash_b200.stack import LinearStack, StackSpec, make_inputs, make_weights
    one = StackSpec(**{**spec.__dict__, "layers": 1, "steps": 1})
    weights = make_weights(one, dev)
    x, attn = make_inputs(one, dev)
    st = LinearStack(one, weights, dev, fused=False if args.unfused else "auto")
    st.load(x, attn)
    st.forward()            # every buffer holds plausible values
    torch.cuda.synchronize(dev)
    if args.profile_op in ("qkv_split", "wan_qkv"):
        calls, _, _ = qkv_consumer_calls(dev, args.profile_op)
        for i in range(args.steps):
            calls[i % len(calls)]()
    elif args.profile_op == "layer":
        for _ in range(args.steps):
            st.forward()
    else:
        lin = {n: (nn, kk) for n, nn, kk in one.linears()}
        if args.profile_op not in lin:
            raise SystemExit(f"--profile-op: {args.profile_op} is not one of {sorted(lin)} or 'layer'")
        n, k = lin[args.profile_op]
        w = weights[0].w[args.profile_op]
        a = st._q8(k)
        gated = st.fused and args.profile_op == "gate_up"
        for _ in range(args.steps):
            if gated:
                K.fp8_linear_gated(a, st.scale[0], w, st.h, st.amax[0], act=0)
            else:
                K.gemm(a, w, st._raw(n))
    torch.cuda.synchronize(dev)
    check_no_timeout(dev)
    print(json.dumps({"profiled": args.profile_op, "workload": workload_name(spec), "launches": args.steps}), flush=True)


def leave(dev, dist):
    """A captured graph may hold NCCL work, and tearing the process group down under it has hung
    (watchdog stuck in event destruction): finish all work, then leave without the teardown."""
    torch.cuda.synchronize(dev)
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize(dev)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the short runs of the other configurations")
    ap.add_argument("--no-sharded", action="store_true", help="skip the sharded configurations (c3 episodes, c4 tokens / tp)")
    ap.add_argument("--no-gpu-reference", action="store_true", help="do not time the reference's GPU kernels")
    ap.add_argument("--unfused", action="store_true", help="the reference's three-launch structure per linear")
    ap.add_argument("--fuse-residual", action="store_true", help="residual update in the GEMM epilogue as well")
    ap.add_argument("--profile-op", default=None,
                    help="for profilers: build ONE layer of the workload, launch only the named operator of the path "
                         "`--steps` times (a linear of the stack: qkv, o, gate_up, down, ff1, ff2 ...; 'qkv_split' / 'wan_qkv' for the "
                         "QKV consumers at benchmark size; or 'layer' for "
                         "one eager pass of the whole layer) and exit without timing anything")
    ap.add_argument("--gemm-group-m", type=int, default=0, help="band height of the GEMM's tile walk for the whole run (experiments)")
    ap.add_argument("--gemm-mode", type=int, default=0, help="iflb200_gemm_set_mode value for the whole run (experiments)")
    ap.add_argument("--branches", type=int, default=EPISODE_BRANCHES, help="c3 episodes in flight per GPU")
    ap.add_argument("--episodes", type=int, default=1,
                    help="c3 only: independent episodes stacked along M on each GPU (rows are independent: "
                         "per-token scales and per-row norms, so this is arithmetically the same as separate runs)")
    ap.add_argument("--persistent", action="store_true",
                    help="c3: the whole stack as one cooperative launch (stack_persistent_kernel) instead of one "
                         "launch per operator")
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

    from instinctflash_b200.stack import SPECS, LinearStack, StackSpec, make_inputs, make_weights
    spec = SPECS[args.workload]
    if args.episodes > 1:
        spec = StackSpec(**{**spec.__dict__, "M": spec.M * args.episodes})
    total_flops_all_ranks = None
    if args.parallel == "tokens":
        # strong scaling over tokens: rank r owns rows [r*M/p, (r+1)*M/p) (ceil), full weights everywhere
        total_flops_all_ranks = spec.flops()
        spec = StackSpec(**{**spec.__dict__, "M": -(-spec.M // world)})

    if args.impl == "reference":
        run_reference(args, spec, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the FP8 linear path has no CPU fallback")
    from instinctflash_b200 import _lib
    _lib.lib()  # fail loudly when the CUDA library is missing
    if args.gemm_mode and _lib.lib().iflb200_gemm_set_mode(args.gemm_mode) != 0:
        raise SystemExit(f"--gemm-mode {args.gemm_mode} is not a valid mode")
    if args.gemm_group_m and _lib.lib().iflb200_gemm_set_config(0, 0, args.gemm_group_m) != 0:
        raise SystemExit(f"--gemm-group-m {args.gemm_group_m} is not valid")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    if args.parallel == "tp":
        run_tensor_parallel(args, spec, dev, dist, rank, world)
        return

    if args.profile_op:
        profile_operator(args, spec, dev)
        return

    ref_ops, ref_reason = (None, "switched off") if args.no_gpu_reference else reference_gpu_ops()
    weights = make_weights(spec, dev)
    persistent = (spec.kind == "gemma" and not spec.o_in and spec.M <= 128 and args.persistent)
    if persistent:
        # skinny expert loop: the whole stack is one cooperative launch
        from instinctflash_b200.stack_persistent import PersistentExpertStack

        class _Persistent(PersistentExpertStack):
            fused = False

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
        stack = LinearStack(spec, weights, dev, fused=False if args.unfused else "auto", fuse_residual=args.fuse_residual)
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
    # Through the package's serving loop (stack.HostPipeline): every step copies its input from pinned
    # host memory and its residual stream back; the copies of neighbouring steps overlap the compute.
    from instinctflash_b200.stack import HostPipeline
    if hasattr(stack, "res") and not persistent:
        pipe = HostPipeline(stack, graph)
        submit, drain = (lambda: pipe.submit(x_host, out_host, attn)), pipe.drain
    else:
        x_stage = torch.empty_like(x_dev)

        def submit():
            x_stage.copy_(x_host, non_blocking=True)
            stack.load(x_stage, attn)
            graph.replay()
            out_host.copy_(stack.res, non_blocking=True)

        def drain():
            return None
    for _ in range(3):
        submit()
    drain()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for _ in range(args.steps):
        submit()
    drain()
    f1.record(stream)
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    check_no_timeout(dev)

    # ---- the reference's GPU kernels through the same driver, interleaved with this build -------
    gpu_reference = {"unavailable": ref_reason}
    if ref_ops is not None and not persistent:
        try:
            st_ref = LinearStack(spec, weights, dev, ops=ref_ops)
            st_ref.load(x_dev, attn)
            g_ref = st_ref.capture()
            for _ in range(args.warmup):
                g_ref.replay()
            n = max(3, min(args.steps, 10))
            ms_nat, ms_ref = abba(graph, g_ref, n, stream, dev)
            # parity of ONE pass from the same input (untimed): both stacks reloaded, one replay each
            stack.load(x_dev, attn)
            graph.replay()
            st_ref.load(x_dev, attn)
            g_ref.replay()
            torch.cuda.synchronize(dev)
            rel = float((stack.res.float() - st_ref.res.float()).norm() / st_ref.res.float().norm())
            # and of ONE layer: what a single pass through every operator differs by, before depth amplifies it
            one = StackSpec(**{**spec.__dict__, "layers": 1, "steps": 1})
            pair = []
            for ops_one in (None, ref_ops):
                st1 = LinearStack(one, weights[:1], dev, ops=ops_one)
                st1.load(x_dev, attn)
                pair.append(st1.forward().float().clone())
            rel_layer = float((pair[0] - pair[1]).norm() / pair[1].norm())
            del pair, st1
            gpu_reference = {"ms_per_step": ms_ref, "native_ms_per_step": ms_nat, "value": flops / (ms_ref * 1e-3) / 1e12,
                             "ratio": ms_ref / ms_nat, "replays_per_segment": n, "order": "native, reference, reference, native",
                             "what": "the reference's Triton row kernels + torch._scaled_mm (cuBLASLt), unmodified, through "
                                     "the same stack driver and CUDA graph, same weights",
                             "residual_stream_rel_diff_one_layer": rel_layer,
                             "residual_stream_rel_diff_one_pass": rel,
                             "rel_diff_note": "same input, one pass each; per layer the two differ by summation order only "
                                              "(split-K, row sums of the norm: single e4m3 code flips), and a stack of "
                                              "synthetic random layers amplifies that roughly eightfold per doubling of depth"}
            del st_ref, g_ref
        except Exception as exc:   # noqa: BLE001
            gpu_reference = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}

    # ---- dominant kernel: the widest FP8 GEMM of the stack, timed alone over rotating layers ----
    from instinctflash_b200.kernels import fp8 as K
    dom = max(spec.linears(), key=lambda t: t[1] * t[2])
    name, n_dom, k_dom = dom
    a_dom = stack._q8(k_dom)
    gated_dom = bool(getattr(stack, "fused", False)) and name == "gate_up"
    if gated_dom:
        def dom_call(w):
            K.fp8_linear_gated(a_dom, stack.scale[0], w, stack.h, stack.amax[0], act=0)
        kernel_name = f"gemm_fp8_tc5_kernel (gated epilogue) {spec.M}x{n_dom}x{k_dom} ({name})"
        out_bytes = 4.0 * spec.M * (n_dom // 2)
    else:
        out_dom = stack._raw(n_dom)

        def dom_call(w):
            K.gemm(a_dom, w, out_dom)
        kernel_name = f"gemm_fp8_tc5_kernel {spec.M}x{n_dom}x{k_dom} ({name})"
        out_bytes = 2.0 * spec.M * n_dom
    reps = max(args.steps, 10)
    for lw in weights[:3]:
        dom_call(lw.w[name])
    torch.cuda.synchronize(dev)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record(stream)
    for i in range(reps):
        dom_call(weights[i % len(weights)].w[name])
    g1.record(stream)
    torch.cuda.synchronize(dev)
    if gated_dom:
        stack.amax.zero_()
    dom_ms = g0.elapsed_time(g1) / reps
    dom_flops = 2.0 * spec.M * n_dom * k_dom
    dom_bytes = n_dom * k_dom + spec.M * k_dom + out_bytes
    peaks = measured_peaks()
    fp8_peak = measure_fp8_peak(dev) if (rank == 0 and spec.M > 400) else None
    if spec.M > 400:
        peak = 2.0 * peaks["bf16_tflops"]   # dense FP8 runs at twice the bf16 rate on the same tensor pipe
        achieved = dom_flops / (dom_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": None, "kernel": kernel_name,
                    "peak_source": f"2 x bf16_tflops of MEASURED_PEAKS.json ({peaks['source']}; the file has no FP8 entry)",
                    "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS, "ms_per_launch": dom_ms}
        if fp8_peak is not None:
            roofline["measured_fp8_peak"] = fp8_peak
            roofline["frac_of_measured_fp8_burst"] = achieved / fp8_peak["burst_tflops"]
    else:
        peak = peaks["hbm_gbs"]
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": None, "kernel": kernel_name,
                    "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']})",
                    "frac_of_nominal_8000": achieved / NOMINAL_HBM_GBS, "ms_per_launch": dom_ms}
    if persistent:
        step_bytes = stack_bytes(spec)
        achieved = step_bytes / (ms / args.steps * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                    "kernel": f"stack_persistent_kernel ({spec.layers} layers x {spec.steps} steps, M={spec.M})",
                    "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']})",
                    "frac_of_nominal_8000": achieved / NOMINAL_HBM_GBS, "ms_per_launch": ms / args.steps,
                    "note": "bound by the chain of grid-wide dependencies, not by bandwidth"}
        if stack.timeout_record() != 0:
            raise SystemExit(f"a wait inside the persistent kernel timed out: {stack.timeout_record():#x}")
    traffic_file = ROOT / "profiles" / "traffic.json"
    if traffic_file.exists():
        entry = json.loads(traffic_file.read_text()).get(f"{spec.name}:{name}:{'gated' if gated_dom else 'raw'}")
        if entry is not None:
            roofline["traffic"] = entry["bytes_per_launch"]
            roofline["traffic_source"] = entry["source"]

    # ---- max over ranks -------------------------------------------------------------------------
    if dist is not None:
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    # ---- the other configurations, short runs in the same process (rank 0 of a 1-GPU run) --------
    configs = None
    if world == 1 and not args.no_configs:
        del stack, graph
        torch.cuda.empty_cache()
        configs = {}
        short = {"c2": (10, 3), "c3": (10, 3), "c4": (5, 3), "c5": (3, 2)}
        try:
            configs["c1"] = time_single_linear(dev, ref_ops, 10, 3)
            for cfg, (k, w) in short.items():
                if cfg == args.workload:
                    continue
                configs[cfg] = time_config(SPECS[cfg], dev, ref_ops, k, w, persistent=cfg == "c3")
            torch.cuda.empty_cache()
            configs["qkv_consumers"] = time_qkv_consumers(dev, ref_ops is not None)
        except Exception as exc:   # noqa: BLE001
            configs["error"] = f"{type(exc).__name__}: {exc}"[:300]
        check_no_timeout(dev)

    # ---- sharded configurations at this N ----------------------------------------------------------
    sharded = None
    keep = []
    if not args.no_sharded:
        del weights
        torch.cuda.empty_cache()
        sharded = {"ranks": world, "scaling": "strong"}
        c3 = lambda *a: sharded_c3_episodes(*a, max_branches=args.branches)   # noqa: E731
        for key, fn in (("c3_dp", c3), ("c4_tokens", sharded_c4_tokens), ("c4_tp", sharded_c4_tp)):
            try:
                r = fn(dev, dist, rank, world, 3, 2)
                keep.append(r.pop("_keep", None))
                sharded[key] = r
            except Exception as exc:   # noqa: BLE001
                sharded[key] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        check_no_timeout(dev)

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
        execution = ("persistent whole-stack kernel (one cooperative launch per step)" if persistent else
                     "one launch per operator, CUDA graph; " +
                     ("reference's three-launch structure per linear" if args.unfused else
                      "gated activation in the gate_up GEMM's epilogue" + (", residual update in the GEMM epilogue" if args.fuse_residual else "")))
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if tokens else "weak",
            "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
            "config": {"workload": workload_name(spec) + (f", {args.episodes} episodes stacked along M (M={spec.M})" if args.episodes > 1 else ""),
                       "execution": execution,
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
            "gpu_reference": gpu_reference,
            "configs": configs,
            "sharded": sharded,
        }
        print(json.dumps(line), flush=True)
    leave(dev, dist)


if __name__ == "__main__":
    main()
