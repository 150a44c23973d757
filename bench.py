#!/usr/bin/env python3
"""Benchmark of the quantized hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline (the `value` of the JSON line): W4 g128 decode qmatmul throughput in GB/s of ALGORITHMIC
bytes (packed weights + fp16 scale/zero-point + activations in + outputs out, per launch).  One
step = one decode pass of M in {1,2,4,8,16} tokens over a stack of Llama-3-8B-shaped W4 g128
linears (4096->4096, 4096->1024, 4096->14336, 14336->4096), `--layers` distinct copies of each so
that every launch reads weights that are not in L2.  With N > 1 GPUs every rank runs that step on
its own layer copies -- REPLICAS, no collective on the data path; the line says so.

What scales over GPUs is reported under `extra.tp70b` at EVERY N, N = 1 included, on a fixed
problem (strong scaling): Llama-3-70B-shaped decoder layers (hidden 8192, 64 q / 8 kv heads x 128,
FFN 28672), W4 g128, tensor-parallel over the N ranks (column-parallel q/k/v/gate/up, row-parallel
o/down, one NCCL all-reduce after each row-parallel linear), decode batch 64 and prefill 4096
tokens, with the time per decoder layer and the all-reduces' share of it; plus RTN quantize+pack
over the weights of 80 such layers, sharded by layer with no communication.

Synthetic data: weights ~ N(0, 0.02) rounded to bf16 and RTN-quantized on the device by this
library's own kernel; activations ~ N(0, 1) bf16.  No checkpoint or dataset is involved.

The line carries `value` (inputs resident in HBM), `e2e` (the same work through the host-buffer
call: pinned host activations in, host outputs back, copies inside the timed region), `roofline`
for the decode kernel against the measured HBM peak, `cpu_baseline` (the CPU oracle on the host
cores over a bounded sample) and, under `extra`, RTN GB/s, W8 decode, the prefill grid
(M in {512, 2048, 8192} x {W4 g128, W2 g64} x the four shapes) and decode at 64 tokens.
`--impl reference` times the CPU implementation of the same path instead (the oracle port of the
reference's CPU code; the reference's own forward cannot run without a GPU).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA8B_SHAPES = [("q_o_proj", 4096, 4096), ("kv_proj", 1024, 4096), ("gate_up_proj", 14336, 4096),
                  ("down_proj", 4096, 14336)]
DECODE_M = [1, 2, 4, 8, 16]
FALLBACK_HBM_GBS = 6650.0

# Llama-3-70B decoder linears: (name, out_features, in_features, tensor-parallel mode)
HIDDEN70, KV70, FFN70 = 8192, 1024, 28672
LLAMA70B_LINEARS = [("q_proj", HIDDEN70, HIDDEN70, "column"), ("k_proj", KV70, HIDDEN70, "column"),
                    ("v_proj", KV70, HIDDEN70, "column"), ("o_proj", HIDDEN70, HIDDEN70, "row"),
                    ("gate_proj", FFN70, HIDDEN70, "column"), ("up_proj", FFN70, HIDDEN70, "column"),
                    ("down_proj", HIDDEN70, FFN70, "row")]

# DRAM bytes of one qmm_decode_kernel launch (dram__bytes_read.sum + dram__bytes_write.sum of an ncu
# capture of `bench.py --case decode:<shape>:<tokens>`, second captured launch) divided by its
# algorithmic bytes, at 1 and 16 tokens per shape; token counts in between are interpolated.
# Constants from those captures, not measured during the run.  Below 1.0: the outputs (and part of
# the activations) never leave L2 within the launch.
DECODE_TRAFFIC_FACTOR = {"q_o_proj": {1: 1.0064, 16: 0.9937}, "kv_proj": {1: 1.0285, 16: 1.0170},
                         "gate_up_proj": {1: 1.0012, 16: 0.9881}, "down_proj": {1: 1.0019, 16: 0.9982}}


def decode_traffic_factor(name, M):
    f1, f16 = DECODE_TRAFFIC_FACTOR[name][1], DECODE_TRAFFIC_FACTOR[name][16]
    return f1 + (f16 - f1) * (min(max(M, 1), 16) - 1) / 15.0


def decode_bytes(M, N, K, bits, g, bias=False):
    """Algorithmic bytes of one decode qmatmul launch."""
    return N * K * bits // 8 + 2 * N * (K // g) * 2 + 2 * M * K + 2 * M * N + (2 * N if bias else 0)


def rtn_bytes(N, K, bits, g, s_in):
    return N * K * s_in + N * K * bits // 8 + N * (K // g) * 8


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 0)),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0)), "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
            t0 = time.time()
            while not self.lines and time.time() - t0 < 3.0:   # nvidia-smi needs a moment to start
                time.sleep(0.02)
            self.lines.clear()                                  # keep only samples taken under load
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        time.sleep(0.05)
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's CPU code, all host threads
# ------------------------------------------------------------------------------------------

def cpu_threads():
    """All host threads for the CPU oracle, whatever the launcher exported (torchrun forces
    OMP_NUM_THREADS=1 on its workers)."""
    from oracle import oracle
    n = os.cpu_count() or 1
    oracle.set_num_threads(n)
    return oracle.num_threads()


def cpu_decode_sample(sample_shapes, Ms, bits=4, g=128, repeats=1):
    """Times the CPU oracle (quantized forward = dequantize + matmul, restating the reference's
    bitween/functional.py:47-71 + bitween/modules.py:97-101) on a bounded sample."""
    import numpy as np
    from bitween_b200 import synth
    from oracle import oracle
    total_bytes, total_s = 0, 0.0
    for (name, N, K) in sample_shapes:
        w = synth.normal(11, (N, K), 0.02)
        q, s, z = oracle.quantize_rtn(w, oracle.F32, bits, g)
        s_h = oracle.f16_bits(s)
        z_h = oracle.f16_bits(z.astype(np.float32))
        for M in Ms:
            x = oracle.f16_bits(synth.normal(12 + M, (M, K), 1.0))
            for _ in range(repeats):
                t0 = time.perf_counter()
                oracle.qlinear_forward(x, q, s_h, z_h, None, bits, g)
                total_s += time.perf_counter() - t0
                total_bytes += decode_bytes(M, N, K, bits, g)
    return total_bytes, total_s


def run_reference_arm(args, rank):
    if rank != 0:
        return
    from oracle import oracle
    oracle.build()
    cores = cpu_threads()
    sample = [LLAMA8B_SHAPES[1], LLAMA8B_SHAPES[0]]      # 4096->1024 and 4096->4096
    Ms = DECODE_M
    for _ in range(args.warmup):
        cpu_decode_sample(sample[:1], [1])
    t_all, b_all = 0.0, 0
    for _ in range(args.steps):
        b, s = cpu_decode_sample(sample, Ms)
        t_all += s
        b_all += b
    val = b_all / t_all / 1e9
    desc = "M in {1,2,4,8,16} x {4096->1024, 4096->4096} W4 g128 per step (bounded sample of the decode sweep)"
    line = {"impl": "reference", "metric": "w4g128_qmatmul_decode_GBps", "value": val, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": t_all / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "decode8b", "sample": desc},
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------

class Layer:
    """One RTN-quantized linear resident on the device (packed codes + fp16 scale/zero-point)."""

    def __init__(self, N, K, bits, g, device, gen, torch, fn):
        w = (torch.randn(N, K, device=device, generator=gen) * 0.02).to(torch.bfloat16)
        self.q, self.scale, self.zp = fn.quantize_rtn_to_module_buffers(w, bits, g)
        self.N, self.K, self.bits, self.g = N, K, bits, g


def time_region(torch, fn, stream=None):
    """CUDA-event duration (ms) of fn() on the current stream, synchronised on both sides."""
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def max_over_ranks(torch, dist, device, ms):
    if dist is None:
        return ms
    t = torch.tensor([ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def graph_ms(torch, body, flush=None, reps=5):
    """CUDA-event time (ms) of one replay of `body` captured as a CUDA graph, L2 flushed before each replay."""
    body()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    g.replay()
    total = 0.0
    for _ in range(reps):
        if flush is not None:
            flush.fill_(1)
        total += time_region(torch, g.replay)
    return total / reps


def run_decode8b(args, torch, dist, rank, world, device):
    from bitween_b200 import functional as fn
    from bitween_b200.kernels import _lib
    from bitween_b200.kernels.cuda_loader import quantized_matmul_cuda, quantized_matmul_host
    bits, g = 4, 128
    gen = torch.Generator(device=device).manual_seed(1234 + rank)
    layers = [[Layer(N, K, bits, g, device, gen, torch, fn) for (_, N, K) in LLAMA8B_SHAPES]
              for _ in range(args.layers)]
    xs = {M: {K: torch.randn(M, K, device=device, generator=gen).to(torch.bfloat16) for K in (4096, 14336)}
          for M in DECODE_M}
    outs = {M: {N: torch.empty(M, N, device=device, dtype=torch.float16) for N in (4096, 1024, 14336)}
            for M in DECODE_M}

    def step():
        for M in DECODE_M:
            for stack in layers:
                for L in stack:
                    quantized_matmul_cuda(xs[M][L.K], L.q, L.scale, L.zp, None, bits, g, out=outs[M][L.N])

    calls_per_step = len(DECODE_M) * args.layers * len(LLAMA8B_SHAPES)
    launches_per_step = calls_per_step                      # the decode kernel is the only launch of a call
    per_shape = {name: sum(decode_bytes(M, N, K, bits, g) for M in DECODE_M) for (name, N, K) in LLAMA8B_SHAPES}
    bytes_per_step = sum(per_shape.values()) * args.layers
    traffic_per_step = sum(decode_bytes(M, N, K, bits, g) * decode_traffic_factor(name, M)
                           for M in DECODE_M for (name, N, K) in LLAMA8B_SHAPES) * args.layers

    for _ in range(max(args.warmup, 1) if not args.graph else 1):
        step()
    if args.graph:
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run_step = graph.replay
    else:
        run_step = step
    for _ in range(args.warmup):
        run_step()

    sampler = ClockSampler(device.index)
    if dist is not None:
        dist.barrier()
    sampler.start()
    ms = time_region(torch, lambda: [run_step() for _ in range(args.steps)])
    clocks = sampler.stop()
    ms = max_over_ranks(torch, dist, device, ms)
    value = bytes_per_step * args.steps * world / (ms * 1e-3) / 1e9
    decode_kernel = _lib.last_qmatmul_kernel()

    # ---- end to end: pinned host activations in, host outputs back, per launch ----------
    hx = {M: {K: torch.randn(M, K).to(torch.bfloat16).pin_memory() for K in (4096, 14336)} for M in DECODE_M}
    hy = {M: {N: torch.empty(M, N, dtype=torch.float16).pin_memory() for N in (4096, 1024, 14336)} for M in DECODE_M}

    def e2e_step():
        for M in DECODE_M:
            for stack in layers:
                for L in stack:
                    quantized_matmul_host(hx[M][L.K], L.q, L.scale, L.zp, None, bits, g, hy[M][L.N],
                                          xs[M][L.K], outs[M][L.N])
    h2d = sum(2 * M * K for M in DECODE_M for (_, N, K) in LLAMA8B_SHAPES) * args.layers
    d2h = sum(2 * M * N for M in DECODE_M for (_, N, K) in LLAMA8B_SHAPES) * args.layers
    for _ in range(2):
        e2e_step()
    e2e_steps = max(1, min(args.steps, 5))
    ms_e2e = max_over_ranks(torch, dist, device, time_region(torch, lambda: [e2e_step() for _ in range(e2e_steps)]))
    e2e_eager = bytes_per_step * e2e_steps * world / (ms_e2e * 1e-3) / 1e9
    e2e_val, e2e_mode = e2e_eager, "eager: one host-buffer call per linear, issued from Python"
    if args.graph:
        # the same calls captured once as a CUDA graph (per call, in stream order: the staging of the
        # pinned activations to the device, the kernel, the staging of the outputs to pinned host
        # memory) and replayed per step, the way a serving loop issues a fixed step; the caller
        # refills the pinned input buffers between replays
        torch.cuda.synchronize()
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph):
            e2e_step()
        for _ in range(2):
            e2e_graph.replay()
        ms_g = max_over_ranks(torch, dist, device,
                              time_region(torch, lambda: [e2e_graph.replay() for _ in range(e2e_steps)]))
        e2e_val = bytes_per_step * e2e_steps * world / (ms_g * 1e-3) / 1e9
        e2e_mode = ("cuda graph of the host-buffer calls (per call: pinned host -> device staging of the activations, "
                    "kernel, device -> pinned host staging of the outputs), replayed per step")

    # ---- per-shape breakdown (M = 1 and 16): the layer copies of one shape replayed as one graph,
    # L2 flushed before every replay ----
    breakdown = {}
    if rank == 0:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        for si, (name, N, K) in enumerate(LLAMA8B_SHAPES):
            for M in (1, 16):
                def one():
                    for stack in layers:
                        L = stack[si]
                        quantized_matmul_cuda(xs[M][K], L.q, L.scale, L.zp, None, bits, g, out=outs[M][N])
                t_ms = graph_ms(torch, one, flush, reps=10) / args.layers
                breakdown[f"{name}_{N}x{K}_M{M}"] = {
                    "us": round(t_ms * 1e3, 2),
                    "GBps": round(decode_bytes(M, N, K, bits, g) / (t_ms * 1e-3) / 1e9, 1)}

    config = {"workload": "decode8b", "shapes": "Llama-3-8B linears x M{1,2,4,8,16}",
              "bits": bits, "group_size": g, "layer_copies": args.layers,
              "l2_policy": f"inputs larger than L2: {args.layers} distinct copies of every layer "
                           f"({args.layers * 69} MB of packed weights per pass)",
              "cuda_graph": bool(args.graph)}
    if world > 1:
        config["parallelism"] = (f"replicas x{world}: every rank runs the sweep on its own layer copies, no collective "
                                 "(the tensor-parallel workload is extra.tp70b)")
    return {"value": value, "ms": ms, "launches": launches_per_step * args.steps, "calls": calls_per_step * args.steps,
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "mode": e2e_mode, "eager_value": e2e_eager},
            "bytes_per_launch": bytes_per_step / calls_per_step, "launches_per_step": launches_per_step,
            "breakdown": breakdown, "kernel": decode_kernel,
            "traffic": traffic_per_step / calls_per_step,
            "traffic_source": "constants from ncu captures of single launches (DRAM bytes / algorithmic bytes per shape at "
                              "1 and 16 tokens: " + ", ".join(f"{k} {v[1]}/{v[16]}" for k, v in DECODE_TRAFFIC_FACTOR.items())
                              + "), interpolated in the token count and weighted over the sweep",
            "config": config}


def run_single_gpu_extras(args, torch, device, gen):
    """RTN quantize+pack GB/s, W8 g128 decode GB/s, decode at 64 tokens and the prefill grid on the
    Llama-3-8B shapes (reported, not the headline).  Every measurement replays a CUDA graph of
    launches on distinct layer copies with the L2 flushed (256 MB written) before each replay."""
    from bitween_b200 import functional as fn
    from bitween_b200.kernels.cuda_loader import quantized_matmul_cuda as qmm
    out = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    # RTN: bf16 weights, fp32 arithmetic, fp32 scale + int32 zero-point out
    tot_b, tot_ms = 0, 0.0
    per = {}
    for (name, N, K) in LLAMA8B_SHAPES:
        ws = [(torch.randn(N, K, device=device, generator=gen) * 0.02).to(torch.bfloat16) for _ in range(3)]
        bits, g = 4, 128
        ms = graph_ms(torch, lambda: [fn._rtn_launch(w, bits, g, torch.float32, torch.int32, True) for w in ws], flush) / len(ws)
        b = rtn_bytes(N, K, bits, g, 2)
        per[f"{name}_{N}x{K}"] = round(b / (ms * 1e-3) / 1e9, 1)
        tot_b += b
        tot_ms += ms
        del ws
    out["rtn_w4g128_bf16in_GBps"] = round(tot_b / (tot_ms * 1e-3) / 1e9, 1)
    out["rtn_per_shape_GBps"] = per
    # W8 g128 decode (the second weight format of the decode configuration), M = 1 and 16;
    # W4 g128 at 64 tokens (the tensor-parallel decode batch) on the same shapes
    w8, d64 = {}, {}
    for (name, N, K) in LLAMA8B_SHAPES:
        layers = [Layer(N, K, 8, 128, device, gen, torch, fn) for _ in range(4)]
        for M in (1, 16):
            x = torch.randn(M, K, device=device, generator=gen).to(torch.bfloat16)
            y = torch.empty(M, N, device=device, dtype=torch.float16)
            ms = graph_ms(torch, lambda: [qmm(x, L.q, L.scale, L.zp, None, 8, 128, out=y) for L in layers], flush) / len(layers)
            w8[f"{name}_{N}x{K}_M{M}"] = round(decode_bytes(M, N, K, 8, 128) / (ms * 1e-3) / 1e9, 1)
        del layers
        layers = [Layer(N, K, 4, 128, device, gen, torch, fn) for _ in range(4)]
        x = torch.randn(64, K, device=device, generator=gen).to(torch.bfloat16)
        y = torch.empty(64, N, device=device, dtype=torch.float16)
        ms = graph_ms(torch, lambda: [qmm(x, L.q, L.scale, L.zp, None, 4, 128, out=y) for L in layers], flush) / len(layers)
        d64[f"{name}_{N}x{K}_M64"] = round(decode_bytes(64, N, K, 4, 128) / (ms * 1e-3) / 1e9, 1)
        del layers
    out["decode_w8g128_GBps"] = w8
    out["decode_w4g128_M64_GBps"] = d64
    # prefill grid: bf16 activations (cast to fp16 by the library, as the reference does)
    for bits, g in ((4, 128), (2, 64)):
        pf = {}
        for (name, N, K) in LLAMA8B_SHAPES:
            L = Layer(N, K, bits, g, device, gen, torch, fn)
            for M in (512, 2048, 8192):
                x = torch.randn(M, K, device=device, generator=gen).to(torch.bfloat16)
                y = torch.empty(M, N, device=device, dtype=torch.float16)
                ms = graph_ms(torch, lambda: [qmm(x, L.q, L.scale, L.zp, None, bits, g, out=y) for _ in range(3)], flush, reps=3) / 3
                pf[f"{name}_{N}x{K}_M{M}"] = round(2.0 * M * N * K / (ms * 1e-3) / 1e12, 1)
                del x, y
            del L
        out[f"prefill_w{bits}g{g}_TFLOPs"] = pf
    # gated feed-forward of a Llama-3-8B block in decode: gate and up as ONE [2 x 14336, 4096] GEMM with the
    # SiLU * up epilogue, against two plain calls followed by torch's silu and mul
    from bitween_b200.kernels.cuda_loader import interleave_gate_up
    glu = {}
    Fg, Kg = 14336, 4096
    pairs = [(Layer(Fg, Kg, 4, 128, device, gen, torch, fn), Layer(Fg, Kg, 4, 128, device, gen, torch, fn)) for _ in range(3)]
    fusedw = [(interleave_gate_up(a.q, b.q), interleave_gate_up(a.scale, b.scale), interleave_gate_up(a.zp, b.zp)) for a, b in pairs]
    for M in (1, 16):
        x = torch.randn(M, Kg, device=device, generator=gen).to(torch.bfloat16)
        yf = torch.empty(M, Fg, device=device, dtype=torch.float16)
        ms_f = graph_ms(torch, lambda: [qmm(x, q, s_, z, None, 4, 128, out=yf, activation="silu_mul") for (q, s_, z) in fusedw], flush) / len(fusedw)
        ms_s = graph_ms(torch, lambda: [torch.nn.functional.silu(qmm(x, a.q, a.scale, a.zp, None, 4, 128)) *
                                        qmm(x, b.q, b.scale, b.zp, None, 4, 128) for a, b in pairs], flush) / len(pairs)
        glu[f"M{M}"] = {"fused_us": round(ms_f * 1e3, 2), "separate_us": round(ms_s * 1e3, 2),
                        "fused_GBps": round(decode_bytes(M, 2 * Fg, Kg, 4, 128) / (ms_f * 1e-3) / 1e9, 1)}
    out["gate_up_silu_mul_decode_w4g128"] = glu
    del pairs, fusedw
    # backward of the frozen layer (grad_input = grad_output @ W, bitween/modules.py:108-141) at 4096 tokens
    from bitween_b200.kernels.cuda_loader import quantized_matmul_grad_input as qgrad
    gi = {}
    for (name, N, K) in LLAMA8B_SHAPES:
        L = Layer(N, K, 4, 128, device, gen, torch, fn)
        go = torch.randn(4096, N, device=device, generator=gen).to(torch.float16)
        ms = graph_ms(torch, lambda: [qgrad(go, L.q, L.scale, L.zp, 4, 128) for _ in range(3)], flush, reps=3) / 3
        gi[f"{name}_{N}x{K}_M4096"] = round(2.0 * 4096 * N * K / (ms * 1e-3) / 1e12, 1)
        del L, go
    out["grad_input_w4g128_TFLOPs"] = gi
    # trainable mode: fake-quantized weight of WrapperLinear (bitween/wrapper.py:116-172), forward and the
    # backward for the per-group factors, bf16 weights W4 g128; bytes = weight + perturbation in, fp32 out
    from bitween_b200.wrapper import WrapperLinear
    fq = {}
    for (name, N, K) in LLAMA8B_SHAPES[2:3]:
        lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16, device=device)
        wl = WrapperLinear(lin, bits=4, group_size=128)
        r = torch.randn(N, K, device=device, generator=gen)

        def fwd_bwd():
            wl.min_scale.grad = wl.max_scale.grad = None
            w_dq = wl._quantize_weight_with_learnable_params()[0]
            w_dq.backward(r)
        with torch.no_grad():
            ms_f = graph_ms(torch, lambda: wl._quantize_weight_with_learnable_params(), flush, reps=3)
        fwd_bwd()
        torch.cuda.synchronize()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(5):
            fwd_bwd()
        t1.record()
        torch.cuda.synchronize()
        fq[f"{name}_{N}x{K}_forward_GBps"] = round(N * K * (2 + 2 + 4 + 4) / (ms_f * 1e-3) / 1e9, 1)
        fq[f"{name}_{N}x{K}_forward_backward_us"] = round(t0.elapsed_time(t1) / 5 * 1e3, 1)
        del wl, lin, r
    out["fake_quant_w4g128_bf16"] = fq
    return out


def run_case(args, torch, device):
    """`--case kind:shape:tokens[:bits[:group]]` -- one kernel on one Llama-3-8B shape, a handful of
    plain (ungraphed) launches over 4 distinct layer copies, so that a profiler can capture a single
    launch without the rest of the benchmark.  kind: decode | prefill (both the qmatmul call),
    rtn, gradinput, fakequant.  Prints one small JSON line with the CUDA-event time per launch."""
    from bitween_b200 import functional as fn
    from bitween_b200.kernels import _lib
    from bitween_b200.kernels.cuda_loader import quantized_matmul_cuda as qmm, quantized_matmul_grad_input as qgrad
    parts = args.case.split(":")
    kind, shape = parts[0], parts[1]
    M = int(parts[2]) if len(parts) > 2 else 1
    bits = int(parts[3]) if len(parts) > 3 else 4
    g = int(parts[4]) if len(parts) > 4 else 128
    name, N, K = next(t for t in LLAMA8B_SHAPES if t[0] == shape)
    gen = torch.Generator(device=device).manual_seed(5)
    copies = 4
    if kind in ("decode", "prefill", "gradinput"):
        layers = [Layer(N, K, bits, g, device, gen, torch, fn) for _ in range(copies)]
        if kind == "gradinput":
            a = torch.randn(M, N, device=device, generator=gen).to(torch.float16)
            body = lambda L: qgrad(a, L.q, L.scale, L.zp, bits, g)
        else:
            x = torch.randn(M, K, device=device, generator=gen).to(torch.bfloat16)
            y = torch.empty(M, N, device=device, dtype=torch.float16)
            body = lambda L: qmm(x, L.q, L.scale, L.zp, None, bits, g, out=y)
    elif kind == "rtn":
        layers = [(torch.randn(N, K, device=device, generator=gen) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        body = lambda w: fn._rtn_launch(w, bits, g, torch.float32, torch.int32, True)
    elif kind == "fakequant":
        from bitween_b200.wrapper import WrapperLinear, fake_quantize
        layers = [WrapperLinear(torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16, device=device), bits=bits, group_size=g)
                  for _ in range(copies)]
        r = torch.randn(N, K, device=device, generator=gen)

        def body(wl):
            wl.min_scale.grad = wl.max_scale.grad = None
            wl._quantize_weight_with_learnable_params()[0].backward(r)
    else:
        raise SystemExit(f"unknown case kind {kind!r}")
    for L in layers:                       # warm-up pass (also the launches a profiler skips)
        body(L)
    ms = time_region(torch, lambda: [body(L) for L in layers]) / copies
    print(json.dumps({"case": args.case, "kernel": _lib.last_qmatmul_kernel() if kind in ("decode", "prefill") else kind,
                      "us_per_launch": round(ms * 1e3, 2), "copies": copies,
                      "note": "plain launches, back to back, no L2 flush: a profiling aid, not a benchmark value"}), flush=True)


def shard_shape(N, K, mode, world):
    return (N // world, K) if mode == "column" else (N, K // world)


def run_tp70b(args, torch, dist, rank, world, device):
    """Llama-3-70B-shaped decoder layers, tensor-parallel over the ranks, a FIXED number of layers
    at every N (strong scaling): decode batch 64 and prefill 4096 tokens; RTN over 80 layers'
    weights sharded by layer.  Returns the dict reported under extra.tp70b."""
    from bitween_b200 import functional as fn
    from bitween_b200 import tp
    from bitween_b200.kernels import _lib
    from bitween_b200.kernels.cuda_loader import quantized_matmul_cuda as qmm
    bits, g = 4, 128
    layers_n = args.tp_layers
    gen = torch.Generator(device=device).manual_seed(4321 + rank)
    layers = []
    for _ in range(layers_n):
        lay = []
        for (name, N, K, mode) in LLAMA70B_LINEARS:
            n, k = shard_shape(N, K, mode, world)
            w = (torch.randn(n, k, device=device, generator=gen) * 0.02).to(torch.bfloat16)
            q, s, z = fn.quantize_rtn_to_module_buffers(w, bits, g)
            lay.append((name, mode, n, k, q, s, z))
            del w
        layers.append(lay)
    shard_bytes = sum(n * k // 2 for (_, _, n, k, _, _, _) in layers[0])
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    res = {"parallelism": f"tp{world}", "layers": layers_n, "scaling": "strong",
           "packed_MB_per_rank_per_layer": round(shard_bytes / 1e6, 1)}

    def measure(M, allreduce, use_graph, chunks=1, steps=None, peer=None):
        ks = {k for (_, _, _, k, _, _, _) in layers[0]}
        ns = {n for (_, _, n, _, _, _, _) in layers[0]}
        xs = {k: torch.randn(M, k, device=device, generator=gen).to(torch.bfloat16) for k in ks}
        outs = {n: torch.empty(M, n, device=device, dtype=torch.float16) for n in ns}
        comm = torch.cuda.Stream(device=device) if chunks > 1 else None

        def step():
            for lay in layers:
                for (name, mode, n, k, q, s, z) in lay:
                    if mode == "row" and allreduce and dist is not None and chunks > 1:
                        # GEMM of token chunk i+1 while the all-reduce of chunk i runs on a second stream
                        main = torch.cuda.current_stream(device)
                        bounds = [M * i // chunks for i in range(chunks + 1)]
                        for i in range(chunks):
                            lo, hi = bounds[i], bounds[i + 1]
                            qmm(xs[k][lo:hi], q, s, z, None, bits, g, out=outs[n][lo:hi])
                            ev = torch.cuda.Event()
                            ev.record(main)
                            with torch.cuda.stream(comm):
                                comm.wait_event(ev)
                                dist.all_reduce(outs[n][lo:hi])
                        main.wait_stream(comm)
                    elif mode == "row" and allreduce and peer is not None:
                        # partial sums straight into peer-mapped memory, one kernel sums them over the ranks
                        qmm(xs[k], q, s, z, None, bits, g, out=peer.partial(M, n))
                        peer.allreduce(outs[n])
                    else:
                        y = qmm(xs[k], q, s, z, None, bits, g, out=outs[n])
                        if mode == "row" and allreduce and dist is not None:
                            dist.all_reduce(y)
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        run_step = step
        if use_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step()
                run_step = graph.replay
            except Exception:   # noqa: BLE001  (a collective that cannot be captured: report eager only)
                torch.cuda.synchronize()
                return None
        for _ in range(3):
            run_step()
        steps = steps or (10 if M > 1024 else 30)
        if dist is not None:
            dist.barrier()
        total = 0.0
        for _ in range(steps):
            flush.fill_(1)
            total += time_region(torch, run_step)
        return max_over_ranks(torch, dist, device, total / steps)

    algo = {M: world * layers_n * sum(decode_bytes(M, n, k, bits, g) for (_, _, n, k, _, _, _) in layers[0]) for M in (64, 4096)}
    flops = {M: 2.0 * M * layers_n * sum(N * K for (_, N, K, _) in LLAMA70B_LINEARS) for M in (64, 4096)}
    # decode batch 64: eager and CUDA-graph replays, with and without the all-reduces
    dec = {}
    for label, graph in (("eager", False), ("graph", True)):
        ms = measure(64, True, graph)
        if ms is not None:
            dec[label] = ms
    best = min(dec, key=dec.get)
    ms_no_ar = measure(64, False, best == "graph") if world > 1 else dec[best]
    res["decode64"] = {
        "GBps": round(algo[64] / (dec[best] * 1e-3) / 1e9, 1), "us_per_layer": round(dec[best] * 1e3 / layers_n, 1),
        "us_per_layer_without_allreduce": round(ms_no_ar * 1e3 / layers_n, 1),
        "allreduce_share": round(max(0.0, 1.0 - ms_no_ar / dec[best]), 3), "mode": best,
        "us_per_layer_by_mode": {k: round(v * 1e3 / layers_n, 1) for k, v in dec.items()},
        "kernel": _lib.last_qmatmul_kernel(), "allreduce_bytes": 64 * HIDDEN70 * 2}
    # the same decode step with the launches a decoder really issues: q/k/v as one column-parallel GEMM,
    # gate and up as one GEMM with the SiLU * up epilogue (interleaved row pairs), fp16 activations
    # throughout (no per-call cast): 4 GEMMs and 2 all-reduces per layer instead of 7 and 2
    from bitween_b200.kernels.cuda_loader import interleave_gate_up
    fused_layers = []
    for lay in layers:
        d = {name: (n, k, q, s, z) for (name, mode, n, k, q, s, z) in lay}
        cat = lambda i: torch.cat([d["q_proj"][i], d["k_proj"][i], d["v_proj"][i]], dim=0).contiguous()   # noqa: E731
        fused_layers.append({
            "qkv": (d["q_proj"][0] + d["k_proj"][0] + d["v_proj"][0], d["q_proj"][1], cat(2), cat(3), cat(4)),
            "o": d["o_proj"],
            "gate_up": (2 * d["gate_proj"][0], d["gate_proj"][1]) + tuple(interleave_gate_up(d["gate_proj"][i], d["up_proj"][i]) for i in (2, 3, 4)),
            "down": d["down_proj"]})

    def measure_fused(M, allreduce, peer=None):
        fl = fused_layers[0]
        x_h = torch.randn(M, fl["qkv"][1], device=device, generator=gen).to(torch.float16)
        x_o = torch.randn(M, fl["o"][1], device=device, generator=gen).to(torch.float16)
        x_d = torch.randn(M, fl["down"][1], device=device, generator=gen).to(torch.float16)
        y_qkv = torch.empty(M, fl["qkv"][0], device=device, dtype=torch.float16)
        y_h = torch.empty(M, fl["o"][0], device=device, dtype=torch.float16)
        y_act = torch.empty(M, fl["gate_up"][0] // 2, device=device, dtype=torch.float16)

        def step():
            for fl in fused_layers:
                n, k, q, s, z = fl["qkv"]
                qmm(x_h, q, s, z, None, bits, g, out=y_qkv)
                n, k, q, s, z = fl["o"]
                if allreduce and peer is not None:
                    qmm(x_o, q, s, z, None, bits, g, out=peer.partial(M, n))
                    peer.allreduce(y_h)
                else:
                    y = qmm(x_o, q, s, z, None, bits, g, out=y_h)
                    if allreduce and dist is not None:
                        dist.all_reduce(y)
                n, k, q, s, z = fl["gate_up"]
                qmm(x_h, q, s, z, None, bits, g, out=y_act, activation="silu_mul")
                n, k, q, s, z = fl["down"]
                if allreduce and peer is not None:
                    qmm(x_d, q, s, z, None, bits, g, out=peer.partial(M, n))
                    peer.allreduce(y_h)
                else:
                    y = qmm(x_d, q, s, z, None, bits, g, out=y_h)
                    if allreduce and dist is not None:
                        dist.all_reduce(y)
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        run_step = step
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            run_step = graph.replay
        except Exception:   # noqa: BLE001  (a collective that cannot be captured: eager)
            torch.cuda.synchronize()
        for _ in range(3):
            run_step()
        if dist is not None:
            dist.barrier()
        total = 0.0
        for _ in range(30):
            flush.fill_(1)
            total += time_region(torch, run_step)
        return max_over_ranks(torch, dist, device, total / 30)

    # the all-reduces through peer memory instead of NCCL (bitween_b200/peer.py), plain and fused launches
    peer = None
    if world > 1:
        from bitween_b200.peer import PeerAllReduce
        try:
            peer = PeerAllReduce(64 * HIDDEN70)          # raises on every rank if any rank cannot map its peers
        except RuntimeError as e:
            res["decode64"]["peer_allreduce"] = f"unavailable: {e}"
        if peer is not None:
            ms_p = measure(64, True, True, peer=peer)
            if ms_p is not None:
                res["decode64"]["us_per_layer_peer_allreduce"] = round(ms_p * 1e3 / layers_n, 1)
    ms_f = measure_fused(64, True)
    ms_f_no = measure_fused(64, False) if world > 1 else ms_f
    res["decode64_fused"] = {
        "us_per_layer": round(ms_f * 1e3 / layers_n, 1), "us_per_layer_without_allreduce": round(ms_f_no * 1e3 / layers_n, 1),
        "GBps": round(algo[64] / (ms_f * 1e-3) / 1e9, 1), "launches_per_layer": 4,
        "what": "q/k/v as one GEMM, gate/up as one GEMM with the SiLU * up epilogue, fp16 activations; same weights and all-reduces"}
    if peer is not None:
        res["decode64_fused"]["us_per_layer_peer_allreduce"] = round(measure_fused(64, True, peer=peer) * 1e3 / layers_n, 1)
        peer.close()
    del fused_layers
    # prefill 4096 tokens: plain, and with the row-parallel GEMMs chunked against their all-reduces
    pf = {"plain": measure(4096, True, False)}
    if world > 1:
        pf["overlap4"] = measure(4096, True, False, chunks=4)
        pf_no_ar = measure(4096, False, False)
    else:
        pf_no_ar = pf["plain"]
    bestp = min(pf, key=pf.get)
    res["prefill4096"] = {
        "TFLOPs": round(flops[4096] / (pf[bestp] * 1e-3) / 1e12, 1), "ms_per_layer": round(pf[bestp] / layers_n, 3),
        "ms_per_layer_without_allreduce": round(pf_no_ar / layers_n, 3),
        "allreduce_share": round(max(0.0, 1.0 - pf_no_ar / pf[bestp]), 3), "mode": bestp,
        "ms_per_layer_by_mode": {k: round(v / layers_n, 3) for k, v in pf.items()},
        "allreduce_bytes": 4096 * HIDDEN70 * 2}
    del layers

    # RTN quantize+pack over the weights of 80 decoder layers, layer l on rank l % world, generated
    # layer by layer (never more than one layer of bf16 weights resident), no communication
    total_ms, total_b, mine = 0.0, 0, 0
    for layer in range(args.rtn_layers):
        if layer % world != rank:
            continue
        g2 = torch.Generator(device=device).manual_seed(9000 + layer)
        ws = [(torch.randn(N, K, device=device, generator=g2) * 0.02).to(torch.bfloat16) for (_, N, K, _) in LLAMA70B_LINEARS]
        if mine == 0:
            fn.quantize_rtn_many_to_module_buffers(ws, bits, g)          # warm-up
        total_ms += time_region(torch, lambda: fn.quantize_rtn_many_to_module_buffers(ws, bits, g))
        total_b += sum(N * K * 2 + N * K * bits // 8 + N * (K // g) * 4 for (_, N, K, _) in LLAMA70B_LINEARS)
        mine += 1
        del ws
    total_ms = max_over_ranks(torch, dist, device, total_ms)
    if dist is not None:
        t = torch.tensor([float(total_b)], device=device, dtype=torch.float64)
        dist.all_reduce(t)
        total_b = float(t.item())
    res["rtn80"] = {"GBps": round(total_b / (total_ms * 1e-3) / 1e9, 1), "layers": args.rtn_layers,
                    "ms_slowest_rank": round(total_ms, 2),
                    "what": "bf16 weights in, packed W4 g128 + fp16 scale + fp16 zero point out, the seven linears of a layer "
                            "per batched launch through the Python API; allocation of the outputs inside the timed region"}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=8, help="distinct copies of each layer shape (L2 defeat)")
    ap.add_argument("--graph", type=int, default=1, help="replay each step as one CUDA graph")
    ap.add_argument("--tp-layers", type=int, default=3, help="70B-shaped decoder layers of the tensor-parallel workload")
    ap.add_argument("--rtn-layers", type=int, default=80, help="70B-shaped layers whose weights the sharded RTN run quantizes")
    ap.add_argument("--case", default="", help="kind:shape:tokens[:bits[:group]] -- run one kernel on one shape (for profilers)")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU mode (use --impl reference)")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=device)
        dist = dist_mod

    if args.case:
        if world > 1:
            raise SystemExit("--case runs on one GPU")
        run_case(args, torch, device)
        return

    res = run_decode8b(args, torch, dist, rank, world, device)
    extra = {}
    if not args.no_extra:
        extra["tp70b"] = run_tp70b(args, torch, dist, rank, world, device)
        if rank == 0 and world == 1:
            extra.update(run_single_gpu_extras(args, torch, device, torch.Generator(device=device).manual_seed(77)))

    if rank == 0:
        peaks = read_peaks()
        # the roofline is stated per qmatmul call (one launch of the decode kernel), its duration
        # the call's share of the timed region
        ms_per_launch = res["ms"] / max(res["calls"], 1)
        achieved = res["bytes_per_launch"] / (ms_per_launch * 1e-3) / 1e9
        line = {"metric": "w4g128_qmatmul_decode_GBps", "value": res["value"], "unit": "GB/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": res["ms"] / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": res["config"],
                "clocks": res["clocks"], "e2e": res["e2e"], "gpu_launches": res["launches"],
                "roofline": {"bound": "hbm", "kernel": res["kernel"], "achieved": achieved,
                             "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                             "peak_source": peaks["source"], "traffic": res.get("traffic"),
                             "traffic_source": res.get("traffic_source"),
                             "us_per_launch": ms_per_launch * 1e3,
                             "algorithmic_bytes_per_launch": res["bytes_per_launch"]},
                "breakdown": res.get("breakdown", {}), "extra": extra}
        if world == 1 and not args.no_cpu:
            from oracle import oracle
            oracle.build()
            cores = cpu_threads()
            cpu_decode_sample(LLAMA8B_SHAPES[1:2], [1])
            b, s = cpu_decode_sample(LLAMA8B_SHAPES, DECODE_M, repeats=4)
            line["cpu_baseline"] = {
                "value": b / s / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                "sample": "the whole decode sweep (M in {1,2,4,8,16} x the four Llama-3-8B shapes, W4 g128), "
                          f"4 repeats, one layer copy ({s:.1f} s of CPU time); oracle port of the reference's "
                          "CPU dequantize + matmul, OpenMP over all host threads"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
