"""Generate wrapper_small.npz / wrapper_meta.json by RUNNING THE REFERENCE's WrapperLinear on CPU.

Usage (only where the reference checkout is available; it is not needed to run tests):

    python tests/golden/gen_golden_wrapper.py /path/to/reference

What is imported from the reference: bitween.wrapper.WrapperLinear (bitween/wrapper.py:28-242).
For every case the learnable parameters are set to seeded non-trivial values, then
`_quantize_weight_with_learnable_params` (bitween/wrapper.py:116-172) gives w_dq, w_q, scale and
zero_point, and one backward of sum(w_dq * r) through the reference's own autograd graph gives
the gradients of min_scale / max_scale (value's gradient is identically zero there: round()).
`to_quantized_linear` (bitween/wrapper.py:207-242) gives the packed layer.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
from bitween_b200 import synth  # noqa: E402
from gen_golden import TORCH_DT, to_bits  # noqa: E402


def main(ref_root):
    sys.path.insert(0, ref_root)
    from bitween.wrapper import WrapperLinear

    torch.set_num_threads(4)
    out, meta = {}, []
    case = 0
    specs = []
    for bits in (2, 4, 8):
        for g in (32, 64, 128):
            for dt in ("f32", "f16", "bf16"):
                specs.append((bits, g, dt, True, True, "rand"))
    specs += [(4, 16, "f32", True, True, "rand"), (4, 24, "f32", True, True, "rand"), (8, 8, "f16", True, True, "rand"),
              (4, 256, "f32", True, True, "rand"), (2, 4, "f32", True, True, "rand"),
              (4, 32, "f32", True, False, "rand"), (4, 128, "bf16", True, False, "rand"),
              (8, 64, "f32", False, True, "rand"), (4, 64, "f32", False, False, "rand"),
              (4, 32, "f32", True, True, "constant"), (4, 32, "f16", True, True, "constant"),
              (4, 32, "f32", True, True, "ties"), (2, 32, "f32", True, True, "collapsed"),
              (8, 32, "f32", True, True, "big_value"),
              # every tensor 16-bit (min/max tuning off): each intermediate is rounded to the weight's dtype
              (4, 128, "f16", False, True, "rand"), (8, 32, "bf16", False, True, "rand"), (2, 64, "f16", False, False, "rand"),
              (4, 64, "bf16", False, False, "rand"), (8, 128, "f16", False, True, "big_value")]
    for bits, g, dt, minmax, rnd, kind in specs:
        N = 6
        K = 2 * g if g >= 64 else 4 * g
        w = synth.normal(900 + case, (N, K), 0.02)
        if kind == "constant":          # zero range in some groups: the 1e-8 floor and a huge zero point
            w[0, :g] = 0.5
            w[1, g:2 * g] = 0.0
            w[2, :g] = -0.25
        elif kind == "ties":            # t lands on .5 exactly: half-to-even
            qmax = (1 << bits) - 1
            w = np.tile((np.arange(K, dtype=np.float32) % (qmax + 1)) + 0.5, (N, 1)).astype(np.float32)
            w[:, ::g] = 0.0
            w[:, 1::g] = float(qmax)
        layer = torch.nn.Linear(K, N, bias=True)
        layer.weight.data = torch.from_numpy(w).to(TORCH_DT[dt])
        layer.bias.data = torch.from_numpy(synth.normal(950 + case, (N,), 0.02)).to(TORCH_DT[dt])
        wl = WrapperLinear(layer, bits=bits, group_size=g, enable_minmax_tuning=minmax, enable_round_tuning=rnd)
        G = K // g
        with torch.no_grad():
            if minmax:
                lo, hi = (0.9, 1.1)
                if kind == "collapsed":   # factors that shrink the range past zero: scale hits the floor
                    lo, hi = (-0.2, 0.3)
                wl.min_scale.copy_(torch.from_numpy(synth.uniform(1000 + case, (N, G), lo, hi)))
                wl.max_scale.copy_(torch.from_numpy(synth.uniform(1100 + case, (N, G), lo, hi)))
            if rnd:
                amp = 3.0 if kind == "big_value" else 0.5
                wl.value.copy_(torch.from_numpy(synth.uniform(1200 + case, (N, K), -amp, amp)).to(wl.value.dtype))
        name = f"wl{case}_b{bits}_g{g}_{dt}_{kind}"
        w_dq, w_q, scale, zp = wl._quantize_weight_with_learnable_params()
        r = torch.from_numpy(synth.normal(1300 + case, (N, K), 1.0))
        if w_dq.dtype == torch.float32 and minmax:
            (w_dq * r).sum().backward()
            out[name + "/grad_min_scale"] = to_bits(wl.min_scale.grad)
            out[name + "/grad_max_scale"] = to_bits(wl.max_scale.grad)
            if rnd:
                assert wl.value.grad is None or float(wl.value.grad.abs().max()) == 0.0
        out[name + "/w"] = to_bits(layer.weight.data)
        out[name + "/bias"] = to_bits(layer.bias.data)
        if minmax:
            out[name + "/min_scale"] = to_bits(wl.min_scale.data)
            out[name + "/max_scale"] = to_bits(wl.max_scale.data)
        if rnd:
            out[name + "/value"] = to_bits(wl.value.data)
        out[name + "/r"] = to_bits(r)
        out[name + "/w_dq"] = to_bits(w_dq)
        out[name + "/w_q"] = to_bits(w_q.reshape(N, K))
        out[name + "/scale"] = to_bits(scale)
        out[name + "/zp"] = to_bits(zp)
        ql = wl.to_quantized_linear()
        out[name + "/ql_qweight"] = to_bits(ql.qweight)
        out[name + "/ql_scale"] = to_bits(ql.scale)
        out[name + "/ql_zp"] = to_bits(ql.zero_point)
        meta.append({"name": name, "bits": bits, "g": g, "dtype": dt, "minmax": minmax, "round": rnd, "kind": kind,
                     "shape": [N, K], "out_dtype": str(w_dq.dtype).replace("torch.", ""),
                     "value_dtype": str(wl.value.dtype).replace("torch.", "") if rnd else None})
        case += 1
    np.savez_compressed(os.path.join(HERE, "wrapper_small.npz"), **out)
    with open(os.path.join(HERE, "wrapper_meta.json"), "w") as f:
        json.dump({"torch": torch.__version__, "cases": meta}, f, indent=1)
    print(f"wrote {len(meta)} wrapper cases")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
