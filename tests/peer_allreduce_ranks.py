"""Body of the multi-GPU peer all-reduce test: run under torchrun, one process per GPU.
Checks the kernel against a rank-order fp32 sum of the gathered partials (bit-exact) over many
calls, eager and replayed from a CUDA graph, the row-parallel layer against its NCCL form, and
prints the time of a 1 MiB all-reduce through both."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from bitween_b200 import QuantizedLinear, synth, tp  # noqa: E402
from bitween_b200.kernels import _lib  # noqa: E402
from bitween_b200.peer import PeerAllReduce  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    algo = os.environ.get("BW_PEER_ALGO", "auto")
    peer = PeerAllReduce(64 * 8192, algo=algo)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)

    def reference(part):
        allp = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(allp, part)
        acc = allp[0].float()
        for r in range(1, world):
            acc = acc + allp[r].float()
        return acc.half()

    # many calls, alternating buffers, several sizes
    for it in range(40):
        M, N = [(64, 8192), (1, 1024), (16, 4096), (64, 1024)][it % 4]
        part = torch.randn(M, N, device=dev, generator=gen).half()
        want = reference(part)
        peer.partial(M, N).copy_(part)
        out = torch.empty(M, N, dtype=torch.float16, device=dev)
        peer.allreduce(out)
        torch.cuda.synchronize()
        assert torch.equal(out, want), (rank, it, float((out.float() - want.float()).abs().max()))
    # a prefill-sized message (the two-shot form under "auto" beyond 4 MiB on more than 2 ranks)
    big = PeerAllReduce(2048 * 8192, algo=algo)
    for it in range(3):
        part = torch.randn(2048, 8192, device=dev, generator=gen).half()
        want = reference(part)
        big.partial(2048, 8192).copy_(part)
        out = torch.empty(2048, 8192, dtype=torch.float16, device=dev)
        big.allreduce(out)
        torch.cuda.synchronize()
        assert torch.equal(out, want), (rank, "big", it)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    nb = torch.randn(2048, 8192, device=dev, generator=gen).half()
    dist.all_reduce(nb)
    torch.cuda.synchronize()
    dist.barrier()
    e0.record()
    for _ in range(10):
        big.partial(2048, 8192)
        big.allreduce(out)
    e1.record()
    torch.cuda.synchronize()
    us_big_peer = e0.elapsed_time(e1) / 10 * 1e3
    dist.barrier()
    e0.record()
    for _ in range(10):
        dist.all_reduce(nb)
    e1.record()
    torch.cuda.synchronize()
    us_big_nccl = e0.elapsed_time(e1) / 10 * 1e3
    big.close()
    # replayed from a CUDA graph: the call counter lives on the device
    M, N = 64, 8192
    src = [torch.randn(M, N, device=dev, generator=gen).half() for _ in range(2)]
    outs = [torch.empty(M, N, dtype=torch.float16, device=dev) for _ in range(2)]
    wants = [reference(s) for s in src]
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(2):
            peer.partial(M, N).copy_(src[i])
            peer.allreduce(outs[i])
    for _ in range(5):
        for o in outs:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(outs[0], wants[0]) and torch.equal(outs[1], wants[1])
    # timing: 20 all-reduces of 1 MiB in one graph, peer kernel vs NCCL
    def timed(body):
        body()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(20):
                body()
        g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 200 * 1e3

    buf = torch.randn(M, N, device=dev, generator=gen).half()
    o = torch.empty_like(buf)

    def peer_body():
        peer.partial(M, N)
        peer.allreduce(o)
    us_peer = timed(peer_body)
    us_nccl = timed(lambda: dist.all_reduce(buf))
    # the row-parallel layer: peer collective against NCCL
    torch.manual_seed(0)
    lin = torch.nn.Linear(2048, 1024, bias=False).to(dev)
    full = QuantizedLinear.from_float(lin, bits=4, group_size=128)
    x = torch.from_numpy(synth.normal(7, (64, 2048), 1.0)).to(dev).half()
    xs = x[:, rank * (2048 // world):(rank + 1) * (2048 // world)].contiguous()
    y_nccl = tp.RowParallelQuantizedLinear.from_full(full, rank, world)(xs)
    y_peer = tp.RowParallelQuantizedLinear.from_full(full, rank, world, peer=peer)(xs)
    torch.cuda.synchronize()
    err = float((y_peer.float() - y_nccl.float()).abs().max())
    rms = float(y_nccl.float().pow(2).mean().sqrt())
    assert err <= 4 * 2.0 ** -10 * max(rms, float(y_nccl.float().abs().max())), (err, rms)   # fp16 sums in another order
    assert _lib.lib().bw_device_status() == 0
    two_shot = peer.two_shot
    peer.close()
    if rank == 0:
        print(f"peer all-reduce ok: world={world} two_shot={two_shot} 1 MiB all-reduce {us_peer:.1f} us (peer kernel) vs {us_nccl:.1f} us (NCCL); "
              f"32 MiB {us_big_peer:.0f} us vs {us_big_nccl:.0f} us", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
