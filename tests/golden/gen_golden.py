"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE on CPU.

Usage (only where the reference checkout is available; it is not needed to run tests):

    python tests/golden/gen_golden.py /path/to/reference

What is imported from the reference: bitween.functional.quantize_rtn and dequantize_rtn
(bitween/functional.py:3-71).  The QuantizedLinear forward itself cannot run without a GPU
(bitween/modules.py:88-95 launches a Triton kernel unconditionally), so the forward fixture
is produced the way the reference's own kernel test does it (main.py:446-466): dequantize
with the reference's dequantize_rtn on fp16 scale/zero-point, cast to fp16, F.linear.

Outputs:
  rtn_small.npz      explicit inputs + reference outputs, many small cases incl. edge cases
  forward_small.npz  explicit inputs + reference dequantized weights and linear outputs
  digests.json       sha256 of reference outputs for larger seeded inputs (inputs come from
                     bitween_b200.synth, which is bit-reproducible everywhere)
"""
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
from bitween_b200 import synth  # noqa: E402

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def to_bits(t):
    """torch tensor -> numpy (16-bit floats as uint16 bit patterns)."""
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def edge_weights(kind, N, K, g, bits):
    """Hand-built inputs that hit the numerically interesting branches."""
    w = synth.normal(1234, (N, K), 0.02)
    qmax = (1 << bits) - 1
    if kind == "constant_pos":       # zero range: scale -> 1e-8 floor, codes saturate
        w[:] = 0.5
    elif kind == "constant_zero":
        w[:] = 0.0
    elif kind == "constant_neg":
        w[:] = -0.25
    elif kind == "ties":             # values on exact .5 code boundaries -> half-to-even
        base = np.arange(K, dtype=np.float32) % (qmax + 1)
        w = np.tile(base + 0.5, (N, 1)).astype(np.float32)
        w[:, ::g] = 0.0
        w[:, 1::g] = float(qmax)
    elif kind == "large":
        w = w * 1e6
    elif kind == "tiny":
        w = w * 1e-9
    elif kind == "mixed_groups":     # some groups constant, some not, some all-negative
        w[0, :g] = 1.0
        w[1 % N, :g] = -np.abs(w[1 % N, :g]) - 0.1
        w[2 % N, g:2 * g] = np.abs(w[2 % N, g:2 * g]) + 0.1
    elif kind == "top_code_set":     # max at the last slot of a word -> negative int32 words
        vpi = 32 // bits
        w[:, vpi - 1::vpi] = 1.0
        w[:, 0::vpi] = -1.0
    return np.ascontiguousarray(w, dtype=np.float32)


def main(ref_root):
    sys.path.insert(0, ref_root)
    from bitween.functional import quantize_rtn, dequantize_rtn

    torch.set_num_threads(4)
    rtn = {}
    meta = []

    def add_rtn(name, w_np, dt, bits, g):
        w = torch.from_numpy(w_np).to(TORCH_DT[dt])
        q, s, z, _ = quantize_rtn(w, bits=bits, group_size=g)
        rtn[name + "/w"] = to_bits(w)
        rtn[name + "/q"] = to_bits(q)
        rtn[name + "/scale"] = to_bits(s)
        rtn[name + "/zp"] = to_bits(z)
        # reference dequantize on its own outputs (fp32 scale / int32 zp API dtypes)
        rtn[name + "/deq"] = to_bits(dequantize_rtn(q, s, z, g, bits=bits))
        meta.append({"name": name, "dtype": dt, "bits": bits, "g": g, "shape": list(w_np.shape)})

    case = 0
    for bits in (2, 4, 8):
        for g in (32, 64, 128):
            for dt in ("f32", "f16", "bf16"):
                N, K = 6, 2 * g if g >= 64 else 4 * g
                add_rtn(f"rand_b{bits}_g{g}_{dt}", synth.normal(100 + case, (N, K), 0.02), dt, bits, g)
                case += 1
    # unusual group sizes (any g >= 1 dividing K is legal in the reference)
    for bits, g, K in ((4, 8, 64), (4, 16, 96), (8, 4, 40), (2, 16, 64), (4, 24, 96), (8, 1, 16),
                       (4, 4, 32), (2, 48, 96), (4, 256, 512), (8, 12, 48)):
        add_rtn(f"oddg_b{bits}_g{g}", synth.normal(300 + case, (5, K), 0.05), "f32", bits, g)
        case += 1
    for kind in ("constant_pos", "constant_zero", "constant_neg", "ties", "large", "tiny",
                 "mixed_groups", "top_code_set"):
        for bits in (2, 4, 8):
            for dt in ("f32", "f16", "bf16"):
                if kind == "constant_zero" and dt == "f16":
                    continue  # 0/0 -> NaN -> int32: platform-defined in the reference
                if kind == "tiny" and dt == "f16":
                    continue  # everything flushes to zero: same NaN path
                add_rtn(f"edge_{kind}_b{bits}_{dt}", edge_weights(kind, 4, 128, 32, bits), dt, bits, 32)
    np.savez_compressed(os.path.join(HERE, "rtn_small.npz"), **rtn)

    # ---- forward fixtures (main.py:446-466 recipe) ------------------------------------
    fwd = {}
    fmeta = []
    fcase = 0
    for bits, g, (M, N, K), use_bias in ((4, 128, (16, 48, 256), True), (8, 128, (5, 32, 256), True),
                                         (2, 64, (9, 40, 128), False), (4, 32, (1, 24, 96), False),
                                         (8, 32, (33, 16, 64), True), (2, 32, (3, 8, 64), True),
                                         (4, 64, (70, 20, 192), False)):
        w = torch.from_numpy(synth.normal(500 + fcase, (N, K), 0.02))
        b = torch.from_numpy(synth.normal(600 + fcase, (N,), 0.02)) if use_bias else None
        x = torch.from_numpy(synth.normal(700 + fcase, (M, K), 1.0))
        q, s, z, _ = quantize_rtn(w, bits=bits, group_size=g)
        s_h, z_h = s.half(), z.half()                       # modules.py:207-209 copy_ casts
        w_h = dequantize_rtn(q, s_h, z_h, g, bits=bits).half()
        x_h = x.half()                                      # modules.py:74
        b_h = b.half() if b is not None else None
        y = torch.nn.functional.linear(x_h, w_h, b_h)       # main.py:466
        y32 = x_h.double() @ w_h.double().T                 # fp64 accumulate of the fp16 operands
        name = f"fwd{fcase}_b{bits}_g{g}"
        fwd[name + "/x"] = to_bits(x)
        fwd[name + "/q"] = to_bits(q)
        fwd[name + "/scale_h"] = to_bits(s_h)
        fwd[name + "/zp_h"] = to_bits(z_h)
        if b is not None:
            fwd[name + "/bias"] = to_bits(b)
        fwd[name + "/w_h"] = to_bits(w_h)
        fwd[name + "/y_h"] = to_bits(y)
        fwd[name + "/y_acc64"] = y32.numpy()
        fmeta.append({"name": name, "bits": bits, "g": g, "M": M, "N": N, "K": K, "bias": use_bias})
        fcase += 1
    np.savez_compressed(os.path.join(HERE, "forward_small.npz"), **fwd)

    # ---- digests of larger seeded cases --------------------------------------------------
    dig = {}

    def sha(*arrs):
        h = hashlib.sha256()
        for a in arrs:
            h.update(np.ascontiguousarray(a).tobytes())
        return h.hexdigest()

    for name, seed, (N, K), std, dt, bits, g in (
            ("cfg1_opt125m_qproj_w4g128", 1, (768, 768), 0.02, "f32", 4, 128),
            ("opt_fc1_w8g32", 2, (3072, 768), 0.02, "f32", 8, 32),
            ("opt_fc2_w2g64", 3, (768, 3072), 0.02, "f32", 2, 64),
            ("llama_kv_w4g128_bf16round", 4, (1024, 4096), 0.02, "bf16->f32", 4, 128),
            ("llama_kv_w8g128_bf16round", 5, (1024, 4096), 0.02, "bf16->f32", 8, 128),
            ("llama_kv_w2g64_f16native", 6, (256, 4096), 0.02, "f16", 2, 64),
            ("llama_kv_w4g128_bf16native", 7, (256, 4096), 0.02, "bf16", 4, 128)):
        w = torch.from_numpy(synth.normal(seed, (N, K), std))
        if dt == "bf16->f32":       # bf16 checkpoint weights up-cast to fp32 (modules.py:191)
            w = w.to(torch.bfloat16).to(torch.float32)
        elif dt != "f32":
            w = w.to(TORCH_DT[dt])
        q, s, z, _ = quantize_rtn(w, bits=bits, group_size=g)
        dig[name] = {"seed": seed, "shape": [N, K], "std": std, "dtype": dt, "bits": bits, "g": g,
                     "w_sha256": sha(to_bits(w)), "q_sha256": sha(to_bits(q)),
                     "scale_sha256": sha(to_bits(s)), "zp_sha256": sha(to_bits(z)),
                     "scale_h_sha256": sha(to_bits(s.half())), "zp_h_sha256": sha(to_bits(z.half()))}
    with open(os.path.join(HERE, "digests.json"), "w") as f:
        json.dump({"torch": torch.__version__, "rtn_meta": meta, "fwd_meta": fmeta, "digests": dig},
                  f, indent=1)
    print(f"wrote {len(meta)} rtn cases, {len(fmeta)} forward cases, {len(dig)} digests")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
