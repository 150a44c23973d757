"""ctypes/numpy front end of the CPU oracle (oracle/bw_oracle.c).

TEST INFRASTRUCTURE ONLY.  Only tests/, __graft_entry__.smoke() and bench.py's CPU
baseline legs may import this module; the shipped package never does.

Parity status: pinned -- tests/test_oracle_golden.py compares every function below with
fixtures produced by the reference's own bitween/functional.py (tests/golden/gen_golden.py).

16-bit floats cross this boundary as numpy uint16 bit patterns (numpy has no bfloat16);
`f16_bits` / `bf16_bits` / `bits_to_f32` convert.
"""
import ctypes
import os
import subprocess

import numpy as np

F32, F16, BF16, I32 = 0, 1, 2, 3

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libbw_oracle.so")
_lib = None


def build(force=False):
    """Compile oracle/bw_oracle.c with the committed Makefile (gcc, OpenMP, no fast-math)."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(
            os.path.join(_HERE, "bw_oracle.c")):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.bwo_quantize_rtn.argtypes = [vp, i32, i64, i64, i32, i32, vp, vp, vp]
        L.bwo_dequantize_rtn.argtypes = [vp, vp, i32, vp, i32, i64, i64, i32, i32, vp]
        L.bwo_dequantize_module.argtypes = [vp, vp, vp, i64, i64, i32, i32, vp, i32]
        L.bwo_qlinear_forward.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp, vp, i32, i32, vp, vp]
        L.bwo_qlinear_grad_input.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp, i32, i32, vp]
        L.bwo_set_num_threads.argtypes = [i32]
        for f in (L.bwo_quantize_rtn, L.bwo_dequantize_rtn, L.bwo_dequantize_module,
                  L.bwo_qlinear_forward, L.bwo_qlinear_grad_input, L.bwo_num_threads, L.bwo_set_num_threads):
            f.restype = ctypes.c_int
        _lib = L
    return _lib


def num_threads():
    return int(lib().bwo_num_threads())


def set_num_threads(n):
    """OpenMP threads used by the later calls (overrides OMP_NUM_THREADS of the environment)."""
    lib().bwo_set_num_threads(int(n))


# ---- 16-bit float helpers (bit patterns in uint16) ---------------------------------

def f16_bits(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32).astype(np.float16)).view(np.uint16)


def bf16_bits(a):
    u = np.ascontiguousarray(np.asarray(a, dtype=np.float32)).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bits_to_f32(bits, dtype):
    bits = np.ascontiguousarray(bits)
    if dtype == F16:
        return bits.view(np.float16).astype(np.float32)
    if dtype == BF16:
        return (bits.astype(np.uint32) << 16).view(np.float32)
    raise ValueError(dtype)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _np_dtype(code):
    return {F32: np.float32, F16: np.uint16, BF16: np.uint16, I32: np.int32}[code]


def _check(rc, what):
    if rc == -1:
        raise AssertionError("Only 2, 4, or 8-bit quantization supported.")
    if rc == -2:
        raise ValueError(f"{what}: in_features is not a multiple of group_size")
    if rc == -3:
        raise RuntimeError(f"{what}: in_features is not a multiple of 32/bits")
    if rc != 0:
        raise RuntimeError(f"{what}: oracle error {rc}")


# ---- the oracle functions --------------------------------------------------------------

def quantize_rtn(w, dtype=F32, bits=8, group_size=32):
    """bitween/functional.py:3-45.  `w` is float32 (dtype=F32) or uint16 bit patterns.

    Returns (q_packed int32 [N, K*bits/32], scale [N, K/g] float32 or uint16 bits,
    zero_point int32 [N, K/g]).
    """
    w = np.ascontiguousarray(w, dtype=_np_dtype(dtype))
    N, K = w.shape
    vpi = 32 // bits if bits in (2, 4, 8) else 1
    G = K // group_size if group_size >= 1 else 0
    q = np.empty((N, K // vpi), dtype=np.int32)
    scale = np.empty((N, G), dtype=_np_dtype(dtype))
    zp = np.empty((N, G), dtype=np.int32)
    rc = lib().bwo_quantize_rtn(_p(w), dtype, N, K, bits, group_size, _p(q), _p(scale), _p(zp))
    _check(rc, "quantize_rtn")
    return q, scale, zp


def dequantize_rtn(q, scale, zp, group_size, bits=8, scale_dtype=F32, zp_dtype=I32):
    """bitween/functional.py:47-71 -> float32 [N, K]."""
    q = np.ascontiguousarray(q, dtype=np.int32)
    scale = np.ascontiguousarray(scale, dtype=_np_dtype(scale_dtype))
    zp = np.ascontiguousarray(zp, dtype=_np_dtype(zp_dtype))
    N = q.shape[0]
    K = q.shape[1] * (32 // bits)
    out = np.empty((N, K), dtype=np.float32)
    rc = lib().bwo_dequantize_rtn(_p(q), _p(scale), scale_dtype, _p(zp), zp_dtype, N, K, bits,
                                  group_size, _p(out))
    _check(rc, "dequantize_rtn")
    return out


def dequantize_module(q, scale_h, zp_h, group_size, bits, out_dtype=F16):
    """bitween/modules.py:10-58 (fp16 scale / zero_point buffers) -> [N, K] in out_dtype."""
    q = np.ascontiguousarray(q, dtype=np.int32)
    scale_h = np.ascontiguousarray(scale_h, dtype=np.uint16)
    zp_h = np.ascontiguousarray(zp_h, dtype=np.uint16)
    N = q.shape[0]
    K = q.shape[1] * (32 // bits)
    out = np.empty((N, K), dtype=_np_dtype(out_dtype))
    rc = lib().bwo_dequantize_module(_p(q), _p(scale_h), _p(zp_h), N, K, bits, group_size, _p(out),
                                     out_dtype)
    _check(rc, "dequantize_module")
    return out


def qlinear_forward(x_bits, q, scale_h, zp_h, bias_bits, bits, group_size, act_dtype=F16,
                    want_acc=False):
    """bitween/modules.py:61-106.  x_bits [M,K] uint16 (already in act_dtype).

    Returns out uint16 [M,N] (and, with want_acc, the float32 pre-rounding accumulator).
    """
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    q = np.ascontiguousarray(q, dtype=np.int32)
    scale_h = np.ascontiguousarray(scale_h, dtype=np.uint16)
    zp_h = np.ascontiguousarray(zp_h, dtype=np.uint16)
    if bias_bits is not None:
        bias_bits = np.ascontiguousarray(bias_bits, dtype=np.uint16)
    M, K = x_bits.shape
    N = q.shape[0]
    assert q.shape[1] * (32 // bits) == K, "x / qweight shape mismatch"
    out = np.empty((M, N), dtype=np.uint16)
    acc = np.empty((M, N), dtype=np.float32) if want_acc else None
    rc = lib().bwo_qlinear_forward(_p(x_bits), act_dtype, M, N, K, _p(q), _p(scale_h), _p(zp_h),
                                   _p(bias_bits), bits, group_size, _p(out), _p(acc))
    _check(rc, "qlinear_forward")
    return (out, acc) if want_acc else out


def qlinear_grad_input(grad_out, grad_dtype, q, scale_h, zp_h, bits, group_size):
    """grad_input of bitween/modules.py:108-141; grad_out [M,N] float32 or uint16 bits."""
    grad_out = np.ascontiguousarray(grad_out, dtype=_np_dtype(grad_dtype))
    q = np.ascontiguousarray(q, dtype=np.int32)
    scale_h = np.ascontiguousarray(scale_h, dtype=np.uint16)
    zp_h = np.ascontiguousarray(zp_h, dtype=np.uint16)
    M, N = grad_out.shape
    K = q.shape[1] * (32 // bits)
    out = np.empty((M, K), dtype=_np_dtype(grad_dtype))
    rc = lib().bwo_qlinear_grad_input(_p(grad_out), grad_dtype, M, N, K, _p(q), _p(scale_h),
                                      _p(zp_h), bits, group_size, _p(out))
    _check(rc, "qlinear_grad_input")
    return out


def wrapper_group_params(w32, bits, group_size, min_scale=None, max_scale=None):
    """scale, zero_point [N,G] fp32 of bitween/wrapper.py:127-140 for weights already up-cast to
    fp32 (exact for 16-bit weights; the products below are fp32 there because the factors are)."""
    w32 = np.asarray(w32, dtype=np.float32)
    N, K = w32.shape
    grouped = w32.reshape(N, K // group_size, group_size)
    w_min, w_max = grouped.min(-1), grouped.max(-1)
    if min_scale is not None and max_scale is not None:
        w_min = w_min * np.asarray(min_scale, dtype=np.float32)
        w_max = w_max * np.asarray(max_scale, dtype=np.float32)
    with np.errstate(all="ignore"):
        scale = (w_max - w_min) / np.float32((1 << bits) - 1)
        scale = np.where(scale < np.float32(1e-8), np.float32(1e-8), scale).astype(np.float32)   # clamp(min=): NaN stays
        zp = (-w_min / scale).astype(np.float32)
    return scale, zp


def wrapper_fake_quant(w32, scale, zp, value32, bits, group_size):
    """w_dq, w_q [N,K] fp32 of bitween/wrapper.py:143-155: one fp32 rounding per operation."""
    w32 = np.asarray(w32, dtype=np.float32)
    N, K = w32.shape
    s3 = np.asarray(scale, dtype=np.float32)[:, :, None]
    z3 = np.asarray(zp, dtype=np.float32)[:, :, None]
    with np.errstate(all="ignore"):
        t = w32.reshape(N, K // group_size, group_size) / s3 + z3
        if value32 is not None:
            t = t + np.asarray(value32, dtype=np.float32).reshape(t.shape)
        r = np.rint(t)
        q = np.where(np.isnan(r), r, np.minimum(np.maximum(r, np.float32(0)), np.float32((1 << bits) - 1))).astype(np.float32)
        dq = (s3 * (q - z3)).astype(np.float32)
    return dq.reshape(N, K), q.reshape(N, K)


def wrapper_param_grads(w32, scale, zp, value32, grad, bits, group_size):
    """d/d scale and d/d zero_point of sum(w_dq * grad) as the reference's autograd graph gives
    them (round has zero gradient), accumulated in float64."""
    _, q = wrapper_fake_quant(w32, scale, zp, value32, bits, group_size)
    N, K = q.shape
    g3 = np.asarray(grad, dtype=np.float64).reshape(N, K // group_size, group_size)
    q3 = q.astype(np.float64).reshape(g3.shape)
    z = np.asarray(zp, dtype=np.float64)
    return (g3 * (q3 - z[:, :, None])).sum(-1), -np.asarray(scale, dtype=np.float64) * g3.sum(-1)


def _round_to(a, dtype):
    """fp32 values rounded to the 16-bit format `dtype` (and back to fp32)."""
    return bits_to_f32(f16_bits(a) if dtype == F16 else bf16_bits(a), dtype).reshape(np.shape(a))


def wrapper_fake_quant_native(w_bits, value_bits, dtype, bits, group_size):
    """bitween/wrapper.py:127-155 when every tensor has the 16-bit `dtype` (16-bit weights, min/max
    tuning off): each operation is an fp32 operation on 16-bit values rounded back to 16 bits, which is
    how torch evaluates it.  Inputs are uint16 bit patterns [N,K]; returns (w_dq, w_q [N,K], scale,
    zero_point [N,G]) as fp32 arrays holding 16-bit-representable values."""
    w = bits_to_f32(np.asarray(w_bits), dtype)
    N, K = w.shape
    g3 = w.reshape(N, K // group_size, group_size)
    rd = lambda a: _round_to(a, dtype)   # noqa: E731
    with np.errstate(all="ignore"):
        w_min, w_max = g3.min(-1, keepdims=True), g3.max(-1, keepdims=True)
        scale = rd(rd(w_max - w_min) / np.float32((1 << bits) - 1))
        floor = rd(np.float32(1e-8))                       # 1e-8 in the 16-bit format (0 in fp16)
        scale = np.where(scale < floor, floor, scale).astype(np.float32)
        zp = rd(-w_min / scale)
        t = rd(rd(g3 / scale) + zp)
        if value_bits is not None:
            t = rd(t + bits_to_f32(np.asarray(value_bits), dtype).reshape(g3.shape))
        r = np.rint(t)
        q = np.where(np.isnan(r), r, np.minimum(np.maximum(r, np.float32(0)), np.float32((1 << bits) - 1))).astype(np.float32)
        dq = rd(scale * rd(q - zp))
    return dq.reshape(N, K), q.reshape(N, K), scale[:, :, 0], zp[:, :, 0]
