"""GPU parity: the CUDA kernels, called through the C ABI (ctypes), against the golden
fixtures produced by the reference and against the CPU oracle on identical seeded inputs.

Bars: bit-exact for packed codes, zero-points, scales and dequantized weights; for matmul
outputs max|err| <= 1e-2 * RMS(output) in 16-bit and <= 1e-5 relative in the fp32-accumulate
checks (the tolerances the task states).
"""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from bitween_b200 import QuantizedLinear, dequantize_rtn, quantize_rtn, synth
from bitween_b200.functional import _rtn_launch, quantize_rtn_to_module_buffers
from bitween_b200.kernels import _lib
from bitween_b200.kernels.cuda_loader import quantized_matmul_cuda, quantized_matmul_grad_input
from helpers import ORACLE_DT, as_f32, assert_close_rms, from_bits, oracle_forward, rms, to_np
from oracle import oracle

pytestmark = pytest.mark.gpu

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
DEV = "cuda"


def _golden(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def _meta(golden_dir):
    with open(os.path.join(golden_dir, "digests.json")) as f:
        return json.load(f)


def _w_tensor(arr, dt):
    if dt == "f32":
        return torch.from_numpy(arr.copy())
    return from_bits(arr, TORCH_DT[dt])


def _bits_equal(t, ref_np):
    got, ref = to_np(t), np.ascontiguousarray(ref_np)
    if got.dtype == np.float32 and np.isnan(ref).any():
        # NaN payload/sign is not defined by IEEE 754 (x86 yields the negative default NaN for
        # inf*0, the GPU the positive one): NaNs must sit in the same places, all else bit-equal
        nan = np.isnan(ref)
        return bool(np.array_equal(np.isnan(got), nan) and
                    np.array_equal(got.view(np.uint32)[~nan], ref.view(np.uint32)[~nan]))
    return got.tobytes() == ref.tobytes()


# --------------------------------------------------------------------------- RTN quantize

def test_rtn_matches_reference_golden_bit_exact(golden_dir):
    meta, gold = _meta(golden_dir), _golden(golden_dir, "rtn_small.npz")
    for c in meta["rtn_meta"]:
        n = c["name"]
        w = _w_tensor(gold[n + "/w"], c["dtype"]).to(DEV)
        q, s, z, g = quantize_rtn(w, bits=c["bits"], group_size=c["g"])
        assert g == c["g"] and q.dtype == torch.int32 and z.dtype == torch.int32 and s.dtype == w.dtype
        assert _bits_equal(q, gold[n + "/q"]), f"{n}: packed codes differ"
        assert _bits_equal(z, gold[n + "/zp"]), f"{n}: zero points differ"
        assert _bits_equal(s, gold[n + "/scale"]), f"{n}: scales differ"


def test_rtn_cpu_tensor_round_trips_through_the_gpu(golden_dir):
    gold = _golden(golden_dir, "rtn_small.npz")
    w = torch.from_numpy(gold["rand_b4_g128_f32/w"].copy())
    q, s, z, _ = quantize_rtn(w, bits=4, group_size=128)
    assert q.device.type == "cpu" and _bits_equal(q, gold["rand_b4_g128_f32/q"])


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_rtn_seeded_layers_match_reference_digests(golden_dir):
    for name, c in _meta(golden_dir)["digests"].items():
        w = torch.from_numpy(synth.normal(c["seed"], tuple(c["shape"]), c["std"]))
        if c["dtype"] == "bf16->f32":
            w = w.to(torch.bfloat16).to(torch.float32)
        elif c["dtype"] != "f32":
            w = w.to(TORCH_DT[c["dtype"]])
        assert _sha(to_np(w)) == c["w_sha256"], name
        q, s, z, _ = quantize_rtn(w.to(DEV), bits=c["bits"], group_size=c["g"])
        assert _sha(to_np(q)) == c["q_sha256"], name
        assert _sha(to_np(s)) == c["scale_sha256"], name
        assert _sha(to_np(z)) == c["zp_sha256"], name
        if c["dtype"] in ("f32", "bf16->f32"):
            q2, s_h, z_h = quantize_rtn_to_module_buffers(w.to(DEV), c["bits"], c["g"])
            assert _sha(to_np(q2)) == c["q_sha256"], name
            assert _sha(to_np(s_h)) == c["scale_h_sha256"], name
            assert _sha(to_np(z_h)) == c["zp_h_sha256"], name


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_rtn_vs_oracle_shapes_and_group_sizes(bits, dt):
    vpi = 32 // bits
    cases = [(1, 32, 32), (3, 64, 32), (7, 256, 64), (33, 384, 128), (130, 1024, 128), (257, 512, 256),
             (5, 96, 16), (5, 96, 48), (9, 80, 8), (4, 64, 4), (3, 48, 24), (2, 2048, 2048), (2, 4096, 512),
             (6, 32, 1), (1000, 128, 32)]
    seed = 1000 * bits
    for (N, K, g) in cases:
        if K % vpi or K % g:
            continue
        seed += 1
        w = torch.from_numpy(synth.normal(seed, (N, K), 0.05)).to(TORCH_DT[dt])
        q, s, z, _ = quantize_rtn(w.to(DEV), bits=bits, group_size=g)
        qo, so, zo = oracle.quantize_rtn(to_np(w), ORACLE_DT[w.dtype], bits, g)
        assert _bits_equal(q, qo), (N, K, g, "codes")
        assert _bits_equal(z, zo), (N, K, g, "zp")
        assert _bits_equal(s, so), (N, K, g, "scale")


def test_rtn_upcast_mode_equals_fp32_path():
    w16 = torch.from_numpy(synth.normal(77, (64, 512), 0.02)).to(torch.bfloat16)
    q, s_h, z_h = quantize_rtn_to_module_buffers(w16.to(DEV), 4, 128)
    qo, so, zo = oracle.quantize_rtn(to_np(w16.float()), oracle.F32, 4, 128)
    assert _bits_equal(q, qo)
    assert _bits_equal(s_h, oracle.f16_bits(so))
    assert _bits_equal(z_h, oracle.f16_bits(zo.astype(np.float32)))


def test_rtn_division_by_reciprocal_is_correctly_rounded():
    # the RTN kernel divides by one correctly rounded reciprocal per group plus four FMAs per
    # element; on 2^28 operand pairs (random and adversarial significands, the whole exponent
    # range of the fast path) the result must equal IEEE division bit for bit
    L = _lib.lib()
    for seed in (1, 2):
        assert L.bw_selftest_division(1 << 27, seed) == 0


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_rtn_streaming_kernel_equals_register_kernel(dt):
    # the opt-in bulk-async (TMA 1-D) pipeline must give the same bits as the default
    # register-load kernel, ragged last tile included, and no bounded wait may run out
    L = _lib.lib()
    N, K = 2051, 4096                      # not a multiple of the 16 KB tile
    gen = torch.Generator(device=DEV).manual_seed(5)
    w = (torch.randn(N, K, device=DEV, generator=gen) * 0.02).to(TORCH_DT[dt])
    w[7, 128:256] = 0.25                   # a constant group
    if dt == "f32":
        w[11, 5] = float("inf")            # sends one group down the NaN/Inf-propagating path
    for bits, g in ((4, 128), (8, 32), (2, 64)):
        ref = quantize_rtn(w, bits=bits, group_size=g)
        got = _rtn_launch(w, bits, g, w.dtype, torch.int32, upcast=False, flags=_lib.RTN_TMA_STREAM)
        assert L.bw_device_status() == 0
        for a, b in zip(got[:3], ref[:3]):
            assert _bits_equal(a, to_np(b)), (dt, bits, g)
    # and the oracle agrees on a slice (rows are independent)
    qo, so, zo = oracle.quantize_rtn(to_np(w[:16].cpu()), ORACLE_DT[w.dtype], 2, 64)
    assert _bits_equal(got[0][:16], qo) and _bits_equal(got[1][:16], so) and _bits_equal(got[2][:16], zo)


def test_rtn_error_bound_full_size_layer():
    # size-independent property at a full Llama-3-8B shape: |w - dequant| <= scale/2 per element
    torch.manual_seed(0)
    w = (torch.randn(4096, 14336, device=DEV) * 0.02).to(torch.bfloat16).float()
    for bits, g in ((4, 128), (8, 128), (2, 64)):
        q, s, z, _ = quantize_rtn(w, bits=bits, group_size=g)
        assert int(z.min()) >= 0 and int(z.max()) <= (1 << bits) - 1
        d = dequantize_rtn(q, s, z, g, bits=bits)
        err = (d - w).abs().view(4096, -1, g)
        bound = s.view(4096, -1, 1) * 0.5 * (1 + 1e-5) + 1e-12
        # elements clipped by the zero-point rounding may exceed scale/2 by at most one more half step
        assert bool((err <= 2 * bound).all())
        assert float((err <= bound).float().mean()) > 0.99
        # idempotence: quantizing the dequantized weights reproduces (nearly) every packed word;
        # a 1-ulp change of the recomputed scale may flip a code that sits on a rounding boundary
        q2, s2, z2, _ = quantize_rtn(d, bits=bits, group_size=g)
        assert float((q2 == q).float().mean()) > 0.99


# --------------------------------------------------------------------------- dequantize

def test_dequantize_matches_reference_golden_bit_exact(golden_dir):
    meta, gold = _meta(golden_dir), _golden(golden_dir, "rtn_small.npz")
    for c in meta["rtn_meta"]:
        n = c["name"]
        q = torch.from_numpy(gold[n + "/q"].copy()).to(DEV)
        s = _w_tensor(gold[n + "/scale"], c["dtype"]).to(DEV)
        z = torch.from_numpy(gold[n + "/zp"].copy()).to(DEV)
        d = dequantize_rtn(q, s, z, c["g"], bits=c["bits"])
        assert d.dtype == torch.float32
        assert _bits_equal(d, gold[n + "/deq"]), n


def test_dequantize_module_dtypes_match_golden_fp16_weights(golden_dir):
    meta, gold = _meta(golden_dir), _golden(golden_dir, "forward_small.npz")
    for c in meta["fwd_meta"]:
        n = c["name"]
        q = torch.from_numpy(gold[n + "/q"].copy()).to(DEV)
        s_h = from_bits(gold[n + "/scale_h"], torch.float16).to(DEV)
        z_h = from_bits(gold[n + "/zp_h"], torch.float16).to(DEV)
        w_h = dequantize_rtn(q, s_h, z_h, c["g"], bits=c["bits"], out_dtype=torch.float16)
        assert _bits_equal(w_h, gold[n + "/w_h"]), n


# --------------------------------------------------------------------------- qmatmul forward

def test_forward_matches_reference_golden(golden_dir):
    meta, gold = _meta(golden_dir), _golden(golden_dir, "forward_small.npz")
    for c in meta["fwd_meta"]:
        n = c["name"]
        x = torch.from_numpy(gold[n + "/x"].copy()).to(DEV)              # fp32 in, cast inside
        q = torch.from_numpy(gold[n + "/q"].copy()).to(DEV)
        s_h = from_bits(gold[n + "/scale_h"], torch.float16).to(DEV)
        z_h = from_bits(gold[n + "/zp_h"], torch.float16).to(DEV)
        b_h = torch.from_numpy(gold[n + "/bias"].copy()).half().to(DEV) if c["bias"] else None
        y = quantized_matmul_cuda(x, q, s_h, z_h, b_h, c["bits"], c["g"])
        assert y.dtype == torch.float16 and tuple(y.shape) == (c["M"], c["N"])
        ref = oracle.bits_to_f32(gold[n + "/y_h"], oracle.F16)
        assert_close_rms(as_f32(y), ref, 1e-2, n)
        # fp32-accumulate check against the fp64 sum of the same fp16 operands
        acc = quantized_matmul_cuda(x, q, s_h, z_h, None, c["bits"], c["g"], out_dtype=torch.float32)
        ref64 = gold[n + "/y_acc64"]
        assert np.abs(as_f32(acc) - ref64).max() <= 1e-5 * np.abs(ref64).max(), n


def _make_layer(seed, N, K, bits, g, bias):
    w = torch.from_numpy(synth.normal(seed, (N, K), 0.02))
    q, s, z = oracle.quantize_rtn(to_np(w), oracle.F32, bits, g)
    q = torch.from_numpy(q)
    s_h = torch.from_numpy(s).half()
    z_h = torch.from_numpy(z).half()
    b_h = torch.from_numpy(synth.normal(seed + 1, (N,), 0.02)).half() if bias else None
    return q, s_h, z_h, b_h


FWD_CASES = [
    # bits, g, M, N, K, bias
    (4, 128, 1, 256, 512, False), (4, 128, 2, 130, 384, True), (4, 128, 8, 64, 128, True),
    (4, 128, 16, 768, 768, True), (4, 64, 5, 48, 192, False), (4, 32, 16, 100, 96, True),
    (4, 16, 3, 40, 64, True), (4, 256, 9, 96, 1024, False), (4, 128, 16, 512, 4096, False),
    (8, 128, 1, 128, 256, True), (8, 32, 16, 72, 160, False), (8, 8, 4, 24, 48, True),
    (8, 64, 7, 200, 576, True), (8, 128, 16, 256, 2048, False),
    (2, 64, 1, 64, 256, False), (2, 32, 16, 136, 192, True), (2, 128, 12, 80, 768, True),
    (2, 64, 16, 256, 2048, False),
    (4, 128, 17, 96, 256, True), (4, 128, 33, 64, 384, False), (8, 64, 64, 48, 256, True),
    (2, 64, 50, 40, 512, True), (4, 64, 70, 20, 192, False), (4, 128, 200, 32, 256, True),
    # layouts the streaming kernel cannot take -> general kernel
    (4, 24, 4, 16, 96, True), (8, 12, 9, 8, 48, False), (2, 48, 3, 8, 96, True), (4, 8, 5, 12, 40, True),
    (8, 4, 2, 6, 20, False), (4, 128, 3, 16, 128 * 3 + 0, True),
]


@pytest.mark.parametrize("case", FWD_CASES, ids=lambda c: "b%d_g%d_M%d_N%d_K%d_%s" % c)
def test_forward_vs_oracle(case):
    bits, g, M, N, K, bias = case
    q, s_h, z_h, b_h = _make_layer(hash(case) % 100000, N, K, bits, g, bias)
    x = torch.from_numpy(synth.normal(4242 + M, (M, K), 1.0)).half()
    ref, ref_acc = oracle_forward(x, q, s_h, z_h, b_h, bits, g, want_acc=True)
    dev = [t.to(DEV) if t is not None else None for t in (x, q, s_h, z_h, b_h)]
    y = quantized_matmul_cuda(*dev, bits, g)
    assert_close_rms(as_f32(y), as_f32(ref), 1e-2, str(case))
    acc = quantized_matmul_cuda(dev[0], dev[1], dev[2], dev[3], None, bits, g, out_dtype=torch.float32)
    denom = max(float(ref_acc.abs().max()), 1e-30)
    assert float((acc.cpu() - ref_acc).abs().max()) <= 1e-5 * denom, case


TC_CASES = [
    # bits, g, M, N, K, bias  -- token counts above 32 run on the tcgen05 tensor-core kernel
    (4, 128, 128, 128, 256, True), (4, 64, 33, 256, 512, False), (4, 32, 300, 200, 384, True),
    (8, 128, 256, 384, 1024, True), (8, 16, 100, 72, 160, False), (2, 64, 512, 256, 2048, True),
    (2, 32, 65, 40, 192, False), (4, 32, 1000, 130, 96, True), (4, 256, 129, 64, 1024, False),
]


@pytest.mark.parametrize("case", TC_CASES, ids=lambda c: "b%d_g%d_M%d_N%d_K%d_%s" % c)
def test_tensor_core_forward_vs_oracle(case):
    bits, g, M, N, K, bias = case
    q, s_h, z_h, b_h = _make_layer(hash(case) % 100000, N, K, bits, g, bias)
    x = torch.from_numpy(synth.normal(777 + M, (M, K), 1.0)).half()
    ref, ref_acc = oracle_forward(x, q, s_h, z_h, b_h, bits, g, want_acc=True)
    dev = [t.to(DEV) if t is not None else None for t in (x, q, s_h, z_h, b_h)]
    y = quantized_matmul_cuda(*dev, bits, g)
    assert _lib.last_qmatmul_kernel() == "qmm_tc_kernel"
    assert _lib.lib().bw_device_status() == 0, "a bounded wait of the tensor-core pipeline ran out"
    assert_close_rms(as_f32(y), as_f32(ref), 1e-2, str(case))
    acc = quantized_matmul_cuda(dev[0], dev[1], dev[2], dev[3], None, bits, g, out_dtype=torch.float32)
    denom = max(float(ref_acc.abs().max()), 1e-30)
    assert float((acc.cpu() - ref_acc).abs().max()) <= 1e-5 * denom, case
    # bf16 / fp32 activations are cast to fp16 first, like the reference (modules.py:74)
    yb = quantized_matmul_cuda(dev[0].to(torch.bfloat16), dev[1], dev[2], dev[3], dev[4], bits, g)
    refb = oracle_forward(x.to(torch.bfloat16), q, s_h, z_h, b_h, bits, g)
    assert_close_rms(as_f32(yb), as_f32(refb), 1e-2, str(case))


@pytest.mark.parametrize("M", [512, 2048])
@pytest.mark.parametrize("bits,g", [(4, 128), (2, 64)])
def test_prefill_full_size_shape_against_gpu_dequant_matmul(M, bits, g):
    # Llama-3-8B gate/up shape: the tensor-core kernel against "dequantize (bit-exact kernel)
    # then matmul in fp32" on the same device
    N, K = 14336, 4096
    gen = torch.Generator(device=DEV).manual_seed(M + bits)
    w = (torch.randn(N, K, device=DEV, generator=gen) * 0.02).to(torch.bfloat16)
    q, s_h, z_h = quantize_rtn_to_module_buffers(w, bits, g)
    w_h = dequantize_rtn(q, s_h, z_h, g, bits=bits, out_dtype=torch.float16)
    x = torch.randn(M, K, device=DEV, generator=gen).half()
    y = quantized_matmul_cuda(x, q, s_h, z_h, None, bits, g)
    assert _lib.last_qmatmul_kernel() == "qmm_tc_kernel" and _lib.lib().bw_device_status() == 0
    ref = x.float() @ w_h.float().T
    assert_close_rms(as_f32(y), as_f32(ref), 1e-2)
    acc = quantized_matmul_cuda(x, q, s_h, z_h, None, bits, g, out_dtype=torch.float32)
    assert float((acc - ref).abs().max()) <= 2e-5 * float(ref.abs().max())   # both sides accumulate in fp32


@pytest.mark.parametrize("bits,g", [(8, 32), (4, 32), (2, 32), (4, 64)])
def test_tensor_core_long_k_many_tiles_is_race_free(bits, g):
    # 6 row tiles x 16 token tiles over 48 k-stages: the packed-word ring is refilled by TMA many
    # times while other warps still expand earlier stages (a missing proxy fence between the
    # generic reads of a ring slot and the TMA write that refills it once corrupted random rows
    # here, differently on every run)
    N, K, M = 768, 3072, 4096
    gen = torch.Generator(device=DEV).manual_seed(bits * 100 + g)
    w = (torch.randn(N, K, device=DEV, generator=gen) * 0.02).to(torch.bfloat16)
    q, s_h, z_h = quantize_rtn_to_module_buffers(w, bits, g)
    w_h = dequantize_rtn(q, s_h, z_h, g, bits=bits, out_dtype=torch.float16)
    x = torch.randn(M, K, device=DEV, generator=gen).half()
    ref = x.float() @ w_h.float().T
    first = None
    for _ in range(4):
        acc = quantized_matmul_cuda(x, q, s_h, z_h, None, bits, g, out_dtype=torch.float32)
        assert _lib.last_qmatmul_kernel() == "qmm_tc_kernel"
        assert float((acc - ref).abs().max()) <= 2e-5 * float(ref.abs().max())
        first = acc if first is None else first
        assert torch.equal(acc, first)
    assert _lib.lib().bw_device_status() == 0


def test_forward_kernel_selection():
    q, s_h, z_h, b_h = _make_layer(5, 64, 256, 4, 128, False)
    x = torch.zeros(4, 256, dtype=torch.float16, device=DEV)
    quantized_matmul_cuda(x, q.to(DEV), s_h.to(DEV), z_h.to(DEV), None, 4, 128)
    assert _lib.last_qmatmul_kernel() == "qmm_smallm_kernel"
    q, s_h, z_h, b_h = _make_layer(6, 16, 96, 4, 24, False)
    x = torch.zeros(4, 96, dtype=torch.float16, device=DEV)
    quantized_matmul_cuda(x, q.to(DEV), s_h.to(DEV), z_h.to(DEV), None, 4, 24)
    assert _lib.last_qmatmul_kernel() == "qmm_general_kernel"
    q, s_h, z_h, b_h = _make_layer(7, 256, 1024, 4, 128, False)
    x = torch.zeros(4, 1024, dtype=torch.float16, device=DEV)
    quantized_matmul_cuda(x, q.to(DEV), s_h.to(DEV), z_h.to(DEV), None, 4, 128)
    assert _lib.last_qmatmul_kernel() == "qmm_decode_kernel"


@pytest.mark.parametrize("xdt", [torch.float32, torch.bfloat16])
def test_forward_input_dtypes_are_cast_to_fp16_like_the_reference(xdt):
    q, s_h, z_h, b_h = _make_layer(11, 96, 256, 4, 128, True)
    x = torch.from_numpy(synth.normal(12, (6, 256), 1.0)).to(xdt)
    ref = oracle_forward(x, q, s_h, z_h, b_h, 4, 128)            # casts x to fp16 (modules.py:74)
    y = quantized_matmul_cuda(x.to(DEV), q.to(DEV), s_h.to(DEV), z_h.to(DEV), b_h.to(DEV), 4, 128)
    assert y.dtype == torch.float16                               # always fp16 out (modules.py:106)
    assert_close_rms(as_f32(y), as_f32(ref), 1e-2)


def test_forward_bf16_output_extension():
    q, s_h, z_h, b_h = _make_layer(13, 128, 512, 4, 128, False)
    x = torch.from_numpy(synth.normal(14, (16, 512), 1.0)).to(torch.bfloat16)
    # bf16 restatement of the reference: dequantize -> bf16 -> matmul, bf16 activations
    ref = oracle_forward(x, q, s_h, z_h, None, 4, 128, act=torch.bfloat16)
    y = quantized_matmul_cuda(x.to(DEV), q.to(DEV), s_h.to(DEV), z_h.to(DEV), None, 4, 128,
                              out_dtype=torch.bfloat16)
    assert y.dtype == torch.bfloat16
    # Tolerance for bf16 OUTPUT: 1e-2 * RMS(out) plus one bf16 ulp of the value.  The final
    # rounding to bf16 alone moves a value by up to 2^-8 * |y|, and two correctly computed
    # results can land on neighbouring bf16 numbers (2^-7 * |y| apart), which exceeds
    # 1e-2 * RMS for every |y| > 1.3 * RMS; the ulp term accounts for exactly that.
    got, want = as_f32(y).astype(np.float64), as_f32(ref).astype(np.float64)
    bound = 1e-2 * rms(want) + np.abs(want) * 2.0 ** -7
    assert np.all(np.abs(got - want) <= bound)
    # and before the output rounding the stated bar holds as is
    acc = quantized_matmul_cuda(x.to(DEV), q.to(DEV), s_h.to(DEV), z_h.to(DEV), None, 4, 128,
                                out_dtype=torch.float32)
    _, ref_acc = oracle_forward(x, q, s_h, z_h, None, 4, 128, act=torch.bfloat16, want_acc=True)
    assert_close_rms(as_f32(acc), ref_acc.numpy(), 1e-2)


def test_leading_dims_and_empty_batch():
    q, s_h, z_h, b_h = _make_layer(15, 32, 128, 8, 32, True)
    d = [t.to(DEV) for t in (q, s_h, z_h, b_h)]
    x = torch.from_numpy(synth.normal(16, (2, 3, 128), 1.0)).half()
    y = quantized_matmul_cuda(x.to(DEV), *d, 8, 32)
    assert tuple(y.shape) == (2, 3, 32)
    ref = oracle_forward(x.reshape(6, 128), q, s_h, z_h, b_h, 8, 32)
    assert_close_rms(as_f32(y).reshape(6, 32), as_f32(ref), 1e-2)
    y0 = quantized_matmul_cuda(torch.zeros(0, 128, dtype=torch.float16, device=DEV), *d, 8, 32)
    assert tuple(y0.shape) == (0, 32)


def test_config1_opt125m_qproj_end_to_end():
    # 768 -> 768 with bias, fp32 weights, W4 g128, activations [16, 768] fp32
    lin = torch.nn.Linear(768, 768, bias=True)
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(synth.normal(1, (768, 768), 0.02)))
        lin.bias.copy_(torch.from_numpy(synth.normal(2, (768,), 0.02)))
    x = torch.from_numpy(synth.normal(3, (16, 768), 1.0))
    ql = QuantizedLinear.from_float(lin.to(DEV), bits=4, group_size=128)
    qo, so, zo = oracle.quantize_rtn(to_np(lin.weight.data.cpu()), oracle.F32, 4, 128)
    assert _bits_equal(ql.qweight, qo)
    assert _bits_equal(ql.scale, oracle.f16_bits(so))
    assert _bits_equal(ql.zero_point, oracle.f16_bits(zo.astype(np.float32)))
    assert _bits_equal(ql.bias, oracle.f16_bits(to_np(lin.bias.data.cpu())))
    y = ql(x.to(DEV))
    ref = oracle_forward(x, ql.qweight.cpu(), ql.scale.cpu(), ql.zero_point.cpu(), ql.bias.cpu(), 4, 128)
    assert y.dtype == torch.float16 and tuple(y.shape) == (16, 768)
    assert_close_rms(as_f32(y), as_f32(ref), 1e-2)


@pytest.mark.parametrize("bits,g", [(4, 128), (8, 128)])
@pytest.mark.parametrize("shape", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
def test_decode_full_size_shapes_against_gpu_dequant_matmul(bits, g, shape):
    # Llama-3-8B shapes: the fused kernel must agree with "dequantize (bit-exact kernel) then
    # matmul" on the same device, and sampled rows must agree with the CPU oracle.
    N, K = shape
    gen = torch.Generator(device=DEV).manual_seed(N + K + bits)
    w = (torch.randn(N, K, device=DEV, generator=gen) * 0.02).to(torch.bfloat16)
    q, s_h, z_h = quantize_rtn_to_module_buffers(w, bits, g)
    w_h = dequantize_rtn(q, s_h, z_h, g, bits=bits, out_dtype=torch.float16)
    for M in (1, 2, 4, 8, 16):
        x = torch.randn(M, K, device=DEV, generator=gen).to(torch.bfloat16)
        y = quantized_matmul_cuda(x, q, s_h, z_h, None, bits, g)
        ref = (x.half().float() @ w_h.float().T)
        assert_close_rms(as_f32(y), as_f32(ref), 1e-2, f"{shape} M={M}")
        acc = quantized_matmul_cuda(x, q, s_h, z_h, None, bits, g, out_dtype=torch.float32)
        ref64 = x.half().double() @ w_h.double().T
        assert float((acc.double() - ref64).abs().max()) <= 1e-5 * float(ref64.abs().max())
    rows = torch.tensor([0, 1, 15, 16, N // 2 + 3, N - 1])
    x = torch.randn(16, K, device=DEV, generator=gen).half()
    y = quantized_matmul_cuda(x, q, s_h, z_h, None, bits, g)
    ref = oracle_forward(x.cpu(), q[rows].cpu(), s_h[rows].cpu(), z_h[rows].cpu(), None, bits, g)
    assert_close_rms(as_f32(y[:, rows]), as_f32(ref), 1e-2)


DECODE_CASES = [
    # bits, g, M, N, K, bias -- shapes the persistent TMA-fed decode kernel takes (M <= 32, K/g a
    # multiple of 8): cluster splits of a row block (few row blocks), whole row blocks, stream-K
    # splits with shares in the global scratch (more row blocks than SMs), ragged N and K tails
    (4, 128, 1, 1024, 4096, True), (4, 128, 8, 512, 2048, False), (4, 128, 13, 1000, 1024, True),
    (4, 64, 32, 300, 1536, True), (4, 32, 5, 130, 768, False), (4, 128, 16, 14336, 1024, False),
    (4, 128, 3, 20000, 1024, True), (4, 128, 24, 19100, 2048, False),
    (8, 128, 1, 640, 2048, True), (8, 16, 9, 96, 384, False), (8, 64, 32, 20480, 512, True),
    (2, 64, 2, 256, 4096, False), (2, 128, 16, 1100, 2048, True), (2, 64, 30, 19300, 1024, False),
]


@pytest.mark.parametrize("case", DECODE_CASES, ids=lambda c: "b%d_g%d_M%d_N%d_K%d_%s" % c)
def test_persistent_decode_kernel_vs_oracle(case):
    bits, g, M, N, K, bias = case
    q, s_h, z_h, b_h = _make_layer(hash(case) % 100000, N, K, bits, g, bias)
    x = torch.from_numpy(synth.normal(99 + M, (M, K), 1.0)).half()
    ref, ref_acc = oracle_forward(x, q, s_h, z_h, b_h, bits, g, want_acc=True)
    dev = [t.to(DEV) if t is not None else None for t in (x, q, s_h, z_h, b_h)]
    y = quantized_matmul_cuda(*dev, bits, g)
    assert _lib.last_qmatmul_kernel() == "qmm_decode_kernel"
    assert _lib.lib().bw_device_status() == 0, "a bounded wait of the decode pipeline ran out"
    assert_close_rms(as_f32(y), as_f32(ref), 1e-2, str(case))
    acc = quantized_matmul_cuda(dev[0], dev[1], dev[2], dev[3], None, bits, g, out_dtype=torch.float32)
    denom = max(float(ref_acc.abs().max()), 1e-30)
    assert float((acc.cpu() - ref_acc).abs().max()) <= 1e-5 * denom, case
    # the summation order is fixed: a second run gives the same bits
    assert torch.equal(acc, quantized_matmul_cuda(dev[0], dev[1], dev[2], dev[3], None, bits, g, out_dtype=torch.float32))
    # bf16 / fp32 activations are cast to fp16 inside the kernel, like the reference (modules.py:74)
    for xdt in (torch.bfloat16, torch.float32):
        xs = torch.from_numpy(synth.normal(7 + M, (M, K), 1.0)).to(xdt)
        yb = quantized_matmul_cuda(xs.to(DEV), dev[1], dev[2], dev[3], dev[4], bits, g)
        # (32 tokens of fp32 activations at 2 bits need more shared memory per stage than a ring
        # of two stages leaves: that one combination runs on the cluster split-K kernel)
        assert _lib.last_qmatmul_kernel() in ("qmm_decode_kernel", "qmm_smallm_kernel")
        refb = oracle_forward(xs, q, s_h, z_h, b_h, bits, g)
        assert_close_rms(as_f32(yb), as_f32(refb), 1e-2, str(case))


# --------------------------------------------------------------------------- backward

@pytest.mark.parametrize("bits,g,gdt", [(4, 128, torch.float16), (8, 32, torch.float32), (2, 64, torch.bfloat16),
                                        (4, 24, torch.float32)])
def test_grad_input_vs_oracle(bits, g, gdt):
    N, K, M = 40, 384 if g != 24 else 96, 11
    q, s_h, z_h, _ = _make_layer(900 + bits, N, K, bits, g, False)
    go = torch.from_numpy(synth.normal(901, (M, N), 1.0)).to(gdt)
    ref = oracle.qlinear_grad_input(to_np(go), ORACLE_DT[gdt], to_np(q), to_np(s_h), to_np(z_h), bits, g)
    ref = torch.from_numpy(ref) if gdt == torch.float32 else from_bits(ref, gdt)
    gi = quantized_matmul_grad_input(go.to(DEV), q.to(DEV), s_h.to(DEV), z_h.to(DEV), bits, g)
    assert gi.dtype == gdt and tuple(gi.shape) == (M, K)
    assert_close_rms(as_f32(gi), as_f32(ref), 1e-2 if gdt != torch.float32 else 1e-5)


def test_autograd_through_quantized_linear():
    lin = torch.nn.Linear(256, 64, bias=True).to(DEV)
    ql = QuantizedLinear.from_float(lin, bits=4, group_size=64)
    x = torch.randn(5, 256, device=DEV, dtype=torch.float16, requires_grad=True)
    y = ql(x)
    y.float().pow(2).sum().backward()
    w = dequantize_rtn(ql.qweight, ql.scale, ql.zero_point, 64, bits=4)
    ref = (2 * y.detach().float()).half().float() @ w
    assert x.grad is not None and x.grad.dtype == torch.float16
    assert_close_rms(as_f32(x.grad), as_f32(ref), 1e-2)


def test_rtn_batched_call_equals_single_calls_bit_for_bit():
    # bw_rtn_quantize_pack_batch: the linears of a block in one launch (shapes differ, one dtype /
    # bits / group); a batch that cannot take the vector path falls back to one launch per matrix
    from bitween_b200.functional import quantize_rtn_many_to_module_buffers
    gen = torch.Generator(device=DEV).manual_seed(21)
    shapes = [(768, 768), (3072, 768), (768, 3072), (130, 256), (1, 128)]
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        ws = [(torch.randn(n, k, device=DEV, generator=gen) * 0.02).to(dt) for n, k in shapes]
        ws[1][5, 128:256] = 0.125            # a constant group
        for bits, g in ((4, 128), (2, 64), (8, 32), (4, 24 if dt == torch.float32 else 128)):
            if any(k % g for _, k in shapes):
                ws_use = [w for w in ws if w.shape[1] % g == 0]
            else:
                ws_use = ws
            many = quantize_rtn_many_to_module_buffers(ws_use, bits, g)
            for w, (q, s, z) in zip(ws_use, many):
                q1, s1, z1 = quantize_rtn_to_module_buffers(w, bits, g)
                assert torch.equal(q, q1) and torch.equal(s, s1) and torch.equal(z, z1), (dt, bits, g, tuple(w.shape))
    assert _lib.lib().bw_device_status() == 0


@pytest.mark.parametrize("case", [
    # bits, g, M, N, K -- one case per kernel: decode (clusters, whole row blocks, stream-K),
    # cluster split-K streaming kernel, general kernel, tensor-core GEMM (plain and split-K)
    (4, 128, 4, 1024, 4096), (4, 128, 16, 14336, 1024), (4, 128, 3, 20000, 1024), (4, 16, 5, 320, 512),
    (4, 24, 7, 64, 96), (4, 128, 64, 1024, 2048), (4, 128, 300, 512, 1024), (2, 64, 4096, 256, 512),
], ids=lambda c: "b%d_g%d_M%d_N%d_K%d" % c)
def test_fused_relu_and_residual_equal_the_separate_ops(case):
    # bw_qmatmul_fused: relu(linear) + residual inside the kernel's output stage must give the
    # bits of the unfused sequence (fp16 op by op) for fp16 outputs
    bits, g, M, N, K = case
    q, s_h, z_h, b_h = _make_layer(hash(case) % 100000, N, K, bits, g, True)
    x = torch.from_numpy(synth.normal(5 + M, (M, K), 1.0)).half().to(DEV)
    res = torch.from_numpy(synth.normal(6 + M, (M, N), 1.0)).half().to(DEV)
    dev = [t.to(DEV) for t in (q, s_h, z_h, b_h)]
    plain = quantized_matmul_cuda(x, *dev, bits, g)
    kern = _lib.last_qmatmul_kernel()
    fused = quantized_matmul_cuda(x, *dev, bits, g, activation="relu", residual=res)
    assert _lib.last_qmatmul_kernel() == kern
    assert torch.equal(fused, torch.relu(plain) + res), (case, kern)
    only_relu = quantized_matmul_cuda(x, *dev, bits, g, activation="relu")
    assert torch.equal(only_relu, torch.relu(plain))
    # in place on the residual buffer (the usual `h = h + mlp(h)`)
    buf = res.clone()
    quantized_matmul_cuda(x, *dev, bits, g, residual=buf, out=buf)
    assert torch.equal(buf, plain + res)
    # fp32 output: one rounding at the end
    f32 = quantized_matmul_cuda(x, *dev, bits, g, out_dtype=torch.float32, activation="relu", residual=res)
    ref = torch.relu(quantized_matmul_cuda(x, *dev, bits, g, out_dtype=torch.float32)) + res.float()
    assert torch.allclose(f32, ref, rtol=0, atol=1e-6 * float(ref.abs().max()))
    assert _lib.lib().bw_device_status() == 0


@pytest.mark.parametrize("bits,g,gdt,shape", [
    (4, 128, torch.float16, (300, 200, 384)), (4, 64, torch.bfloat16, (129, 48, 192)),
    (8, 32, torch.float16, (16, 130, 96)), (2, 64, torch.bfloat16, (257, 64, 1024)), (4, 24, torch.float16, (33, 18, 96)),
], ids=lambda v: str(v).replace(" ", ""))
def test_grad_input_tensor_core_kernel_vs_oracle(bits, g, gdt, shape):
    # 16-bit gradients run on mma.sync tiles of 128 tokens x 64 k over steps of 16 weight rows:
    # ragged M, N and K tails, every bit width, groups that split a packed word (g = 24)
    M, N, K = shape
    q, s_h, z_h, _ = _make_layer(950 + bits + M, N, K, bits, g, False)
    go = torch.from_numpy(synth.normal(951, (M, N), 1.0)).to(gdt)
    ref = from_bits(oracle.qlinear_grad_input(to_np(go), ORACLE_DT[gdt], to_np(q), to_np(s_h), to_np(z_h), bits, g), gdt)
    gi = quantized_matmul_grad_input(go.to(DEV), q.to(DEV), s_h.to(DEV), z_h.to(DEV), bits, g)
    assert gi.dtype == gdt and tuple(gi.shape) == (M, K)
    if gdt == torch.bfloat16:
        # one bf16 ulp of the value on top of the bar: the final rounding alone moves a value by
        # up to 2^-8 |y|, more than 1e-2 * RMS for |y| > 2.6 RMS, whenever the fp32 sums differ
        # in their last bits (other summation order)
        err = np.abs(as_f32(gi) - as_f32(ref))
        assert (err <= 1e-2 * rms(as_f32(ref)) + 2.0 ** -8 * np.abs(as_f32(ref))).all(), shape
    else:
        assert_close_rms(as_f32(gi), as_f32(ref), 1e-2, str(shape))
    # and the same numbers as the CUDA-core kernel gives on fp32 copies of the same operands
    # (W is rounded to the gradient dtype in both, products are exact, sums are fp32)
    w = dequantize_rtn(q.to(DEV), s_h.to(DEV), z_h.to(DEV), g, bits=bits).to(gdt).float()
    full = go.to(DEV).float() @ w
    slack = 2.0 ** -8 * full.abs() if gdt == torch.bfloat16 else 0.0
    assert bool(((gi.float() - full).abs() <= 1e-2 * rms(as_f32(full)) + slack).all())


@pytest.mark.parametrize("pinned", [True, False])
@pytest.mark.parametrize("M,N,K,bits,g", [(1, 1024, 4096, 4, 128), (16, 4096, 4096, 4, 128), (5, 72, 256, 8, 32),
                                          (200, 512, 1024, 2, 64)])
def test_host_buffer_call_equals_device_call(pinned, M, N, K, bits, g):
    """bw_qmatmul_host (pinned buffers staged by the copy kernel, pageable ones by the copy engine)
    returns exactly what the device-buffer call returns, also when replayed from a CUDA graph."""
    from bitween_b200.kernels.cuda_loader import quantized_matmul_cuda, quantized_matmul_host
    w = torch.from_numpy(synth.normal(31, (N, K), 0.02)).to(DEV)
    q, s, z = _rtn_launch(w, bits, g, torch.float16, torch.float16, True)
    bias = torch.from_numpy(synth.normal(32, (N,), 0.02)).to(DEV).half()
    x = torch.from_numpy(synth.normal(33, (M, K), 1.0)).to(torch.bfloat16)
    hx = x.clone().pin_memory() if pinned else x.clone()
    hy = torch.zeros(M, N, dtype=torch.float16)
    hy = hy.pin_memory() if pinned else hy
    x_dev = torch.empty(M, K, dtype=torch.bfloat16, device=DEV)
    out_dev = torch.empty(M, N, dtype=torch.float16, device=DEV)
    want = quantized_matmul_cuda(x.to(DEV), q, s, z, bias, bits, g).cpu()
    quantized_matmul_host(hx, q, s, z, bias, bits, g, hy, x_dev, out_dev)
    torch.cuda.synchronize()
    assert torch.equal(hy, want)
    if pinned:
        # new inputs through the same pinned buffer, the calls replayed from a graph
        x2 = torch.from_numpy(synth.normal(34, (M, K), 1.0)).to(torch.bfloat16)
        want2 = quantized_matmul_cuda(x2.to(DEV), q, s, z, bias, bits, g).cpu()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            quantized_matmul_host(hx, q, s, z, bias, bits, g, hy, x_dev, out_dev)
        hx.copy_(x2)
        hy.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(hy, want2)
    assert _lib.lib().bw_device_status() == 0


@pytest.mark.parametrize("M", [1, 8, 16, 32, 64, 300])
@pytest.mark.parametrize("bits,g,F,K,bias,res", [(4, 128, 1024, 2048, False, False), (8, 64, 256, 1024, True, True),
                                                  (2, 64, 384, 512, True, False), (4, 128, 14336 // 8, 4096, False, True)])
def test_fused_silu_mul_equals_the_separate_ops(M, bits, g, F, K, bias, res):
    """The gated feed-forward as one [2F, K] GEMM with the SiLU * up epilogue against two plain calls
    followed by torch's own silu and mul on fp16 tensors (and the residual add)."""
    from bitween_b200.kernels.cuda_loader import interleave_gate_up
    wg = torch.from_numpy(synth.normal(41, (F, K), 0.02)).to(DEV)
    wu = torch.from_numpy(synth.normal(42, (F, K), 0.02)).to(DEV)
    qg, sg, zg = _rtn_launch(wg, bits, g, torch.float16, torch.float16, True)
    qu, su, zu = _rtn_launch(wu, bits, g, torch.float16, torch.float16, True)
    bg = torch.from_numpy(synth.normal(43, (F,), 0.5)).to(DEV).half() if bias else None
    bu = torch.from_numpy(synth.normal(44, (F,), 0.5)).to(DEV).half() if bias else None
    x = torch.from_numpy(synth.normal(45, (M, K), 1.0)).to(DEV).to(torch.bfloat16)
    r = torch.from_numpy(synth.normal(46, (M, F), 1.0)).to(DEV).half() if res else None
    gate = quantized_matmul_cuda(x, qg, sg, zg, bg, bits, g)
    up = quantized_matmul_cuda(x, qu, su, zu, bu, bits, g)
    want = torch.nn.functional.silu(gate) * up
    if res:
        want = want + r
    got = quantized_matmul_cuda(x, interleave_gate_up(qg, qu), interleave_gate_up(sg, su), interleave_gate_up(zg, zu),
                                None if not bias else interleave_gate_up(bg, bu), bits, g, activation="silu_mul", residual=r)
    assert tuple(got.shape) == (M, F) and got.dtype == torch.float16
    assert _lib.last_qmatmul_kernel() == ("qmm_decode_kernel" if M <= 32 else "qmm_tc_kernel")
    # the sums may be added in another order than in the two plain calls (other tiling of the rows), and
    # expf may differ from torch's in the last place: a few fp16 ulps of the largest factor
    a, b = as_f32(got), as_f32(want)
    scale_ = np.maximum(np.abs(as_f32(up)), 1.0) * np.maximum(np.abs(as_f32(gate)), 1.0)
    assert np.all(np.abs(a - b) <= 4 * 2.0 ** -10 * scale_ + (np.abs(as_f32(r)) * 2.0 ** -10 if res else 0.0))
    # fp32 output: one rounding at the end
    got32 = quantized_matmul_cuda(x, interleave_gate_up(qg, qu), interleave_gate_up(sg, su), interleave_gate_up(zg, zu),
                                  None if not bias else interleave_gate_up(bg, bu), bits, g, activation="silu_mul",
                                  out_dtype=torch.float32)
    g32 = quantized_matmul_cuda(x, qg, sg, zg, bg, bits, g, out_dtype=torch.float32)
    u32 = quantized_matmul_cuda(x, qu, su, zu, bu, bits, g, out_dtype=torch.float32)
    want32 = torch.nn.functional.silu(g32) * u32
    assert torch.allclose(got32, want32, rtol=1e-4, atol=1e-5 * float(want32.abs().max()) + 1e-7)
    assert _lib.lib().bw_device_status() == 0
