"""Tensor-parallel benchmark workload: decode through Llama-3-70B-shaped W4 g128 decoder
linears (hidden 8192, 64 q / 8 kv heads x 128, FFN 28672) sharded over the ranks of one node:
column-parallel q/k/v/gate/up, row-parallel o/down each followed by an NCCL all-reduce.
Used by bench.py; synthetic weights are quantized on the device by the library's own kernel."""
import torch

from . import functional as fn
from .kernels import _lib
from .kernels.cuda_loader import quantized_matmul_cuda

HIDDEN, KV, FFN = 8192, 1024, 28672
# (name, out_features, in_features, parallel mode)
LINEARS = [("q_proj", HIDDEN, HIDDEN, "column"), ("k_proj", KV, HIDDEN, "column"),
           ("v_proj", KV, HIDDEN, "column"), ("o_proj", HIDDEN, HIDDEN, "row"),
           ("gate_proj", FFN, HIDDEN, "column"), ("up_proj", FFN, HIDDEN, "column"),
           ("down_proj", HIDDEN, FFN, "row")]


def shard_shape(N, K, mode, world):
    return (N // world, K) if mode == "column" else (N, K // world)


def run_tp70b(args, torch_mod, dist, rank, world, device, ClockSampler, time_region, decode_bytes):
    bits, g, M = 4, 128, args.tp_tokens
    gen = torch.Generator(device=device).manual_seed(4321 + rank)
    shard_bytes = sum(n * k // 2 for (_, N, K, mode) in LINEARS for (n, k) in [shard_shape(N, K, mode, world)])
    layers_n = max(2, min(args.layers, -(-400_000_000 // shard_bytes)))   # distinct layers: >= 3x L2
    layers = []
    for _ in range(layers_n):
        lay = []
        for (name, N, K, mode) in LINEARS:
            n, k = shard_shape(N, K, mode, world)
            w = (torch.randn(n, k, device=device, generator=gen) * 0.02).to(torch.bfloat16)
            q, s, z = fn.quantize_rtn_to_module_buffers(w, bits, g)
            lay.append((name, mode, n, k, q, s, z))
            del w
        layers.append(lay)
    xs = {k: torch.randn(M, k, device=device, generator=gen).to(torch.bfloat16)
          for k in {kk for lay in layers[:1] for (_, _, _, kk, _, _, _) in lay}}
    outs = {n: torch.empty(M, n, device=device, dtype=torch.float16)
            for n in {nn for lay in layers[:1] for (_, _, nn, _, _, _, _) in lay}}

    def step():
        for lay in layers:
            for (name, mode, n, k, q, s, z) in lay:
                y = quantized_matmul_cuda(xs[k], q, s, z, None, bits, g, out=outs[n])
                if mode == "row" and dist is not None:
                    dist.all_reduce(y)

    # per linear: up to 32 tokens one decode kernel; above, the fp16 cast of the bf16 activations + the GEMM
    kernels_per_call = 1 if M <= 32 else 2
    launches_per_step = layers_n * len(LINEARS) * kernels_per_call
    bytes_per_step_rank = layers_n * sum(decode_bytes(M, n, k, bits, g) for (_, _, n, k, _, _, _) in layers[0])
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    run_step = step
    used_graph = False
    if args.graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            run_step = graph.replay
            used_graph = True
        except Exception:   # noqa: BLE001  (collectives that cannot be captured: run eagerly)
            torch.cuda.synchronize()
            run_step = step
    for _ in range(max(args.warmup, 3)):
        run_step()
    sampler = ClockSampler(device.index)
    if dist is not None:
        dist.barrier()
    sampler.start()
    ms = time_region(torch, lambda: [run_step() for _ in range(args.steps)])
    clocks = sampler.stop()
    if dist is not None:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = bytes_per_step_rank * world * args.steps / (ms * 1e-3) / 1e9

    # end to end: host activations in, host outputs back, every linear
    from .kernels.cuda_loader import quantized_matmul_host
    hx = {k: v.cpu().pin_memory() for k, v in xs.items()}
    hy = {n: torch.empty(M, n, dtype=torch.float16).pin_memory() for n in outs}

    def e2e_step():
        for lay in layers:
            for (name, mode, n, k, q, s, z) in lay:
                quantized_matmul_host(hx[k], q, s, z, None, bits, g, hy[n], xs[k], outs[n])
                if mode == "row" and dist is not None:
                    dist.all_reduce(outs[n])
    e2e_step()
    e2e_steps = max(1, min(args.steps, 3))
    ms_e2e = time_region(torch, lambda: [e2e_step() for _ in range(e2e_steps)])
    if dist is not None:
        t = torch.tensor([ms_e2e], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    h2d = layers_n * sum(2 * M * k for (_, _, n, k, _, _, _) in layers[0])
    d2h = layers_n * sum(2 * M * n for (_, _, n, k, _, _, _) in layers[0])
    return {"value": value, "ms": ms, "launches": launches_per_step * args.steps,
            "calls": layers_n * len(LINEARS) * args.steps, "clocks": clocks,
            "e2e": {"value": bytes_per_step_rank * world * e2e_steps / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": e2e_steps},
            "bytes_per_launch": bytes_per_step_rank / (layers_n * len(LINEARS)),
            "launches_per_step": launches_per_step, "kernel": _lib.last_qmatmul_kernel(),
            "config": {"workload": "tp70b", "shapes": "Llama-3-70B decoder linears, decode batch %d" % M,
                       "bits": bits, "group_size": g, "parallelism": "tp%d" % world,
                       "layer_copies": layers_n, "cuda_graph": used_graph,
                       "l2_policy": "inputs larger than L2: %d distinct layers (%d MB of packed weights per rank per pass)"
                                    % (layers_n, layers_n * shard_bytes // 1_000_000)}}
