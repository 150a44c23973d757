"""Small, self-ending workloads for capturing one of the library's kernels under a profiler.

    python -m bitween_b200.profile_case decode  N K M [--bits 4] [--group 128] [--copies 4]
    python -m bitween_b200.profile_case prefill N K M [--bits 4] [--group 128]
    python -m bitween_b200.profile_case rtn     N K   [--bits 4] [--group 128] [--copies 4]

`decode` / `prefill` quantize `copies` distinct random layers of shape [N, K] (so that every
launch reads weights that are not in L2), then run the QuantizedLinear forward for M tokens over
each copy twice through the public call `quantized_matmul_cuda`; `rtn` runs the fused
quantize-and-pack twice over each copy.  Nothing is timed here: time with CUDA events in
bench.py; a profiler attaches to the few launches this makes, e.g.

    ncu --set full --clock-control none -k regex:qmm_decode -s 4 -c 2 \\
        python -m bitween_b200.profile_case decode 14336 4096 1
"""
import argparse

import torch

from . import functional as fn
from .kernels import _lib
from .kernels.cuda_loader import quantized_matmul_cuda


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("mode", choices=("decode", "prefill", "rtn"))
    ap.add_argument("N", type=int)
    ap.add_argument("K", type=int)
    ap.add_argument("M", type=int, nargs="?", default=1)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--group", type=int, default=128)
    ap.add_argument("--copies", type=int, default=4)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("profile_case needs a CUDA device")
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(1)
    copies = 1 if args.mode == "prefill" else args.copies
    ws = [(torch.randn(args.N, args.K, device=dev, generator=gen) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    if args.mode == "rtn":
        for _ in range(2):
            for w in ws:
                fn.quantize_rtn_to_module_buffers(w, args.bits, args.group)
    else:
        layers = [fn.quantize_rtn_to_module_buffers(w, args.bits, args.group) for w in ws]
        del ws
        xdt = torch.float16 if args.mode == "prefill" else torch.bfloat16
        x = torch.randn(args.M, args.K, device=dev, generator=gen).to(xdt)
        out = torch.empty(args.M, args.N, device=dev, dtype=torch.float16)
        for _ in range(2):
            for (q, s, z) in layers:
                quantized_matmul_cuda(x, q, s, z, None, args.bits, args.group, out=out)
    torch.cuda.synchronize()
    status = _lib.lib().bw_device_status()
    print(f"done: mode={args.mode} kernel={_lib.last_qmatmul_kernel() if args.mode != 'rtn' else 'rtn_quantize_pack_kernel'} "
          f"device_status={status}")
    return 0 if status == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
