"""ctypes binding of the C ABI declared in include/bitween_b200.h.

This is the only place the Python host code crosses into native code.  There is no
fallback of any kind: if the shared library is missing (and cannot be built because nvcc
is absent) or no CUDA device is present, the calls raise.
"""
import ctypes
import os
import threading

import torch

F32, F16, BF16, I32 = 0, 1, 2, 3
RTN_UPCAST_F32 = 1
RTN_TMA_STREAM = 2

_DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int32: I32}

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "_C", "libbitween_b200.so")

_lib = None
_lock = threading.Lock()


class BitweenKernelError(RuntimeError):
    """A C-ABI call returned a non-zero bw_status."""

    def __init__(self, status, text):
        super().__init__(f"libbitween_b200: {text} (status {status})")
        self.status = status


def dtype_code(dt):
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"bitween_b200: unsupported dtype {dt}") from None


ACT_NONE, ACT_RELU, ACT_SILU_MUL = 0, 1, 2


class Epilogue(ctypes.Structure):
    """bw_epilogue of include/bitween_b200.h."""
    _fields_ = [("activation", ctypes.c_int), ("residual", ctypes.c_void_p)]


class RtnJob(ctypes.Structure):
    """bw_rtn_job of include/bitween_b200.h."""
    _fields_ = [("w", ctypes.c_void_p), ("qweight", ctypes.c_void_p), ("scale", ctypes.c_void_p),
                ("zero_point", ctypes.c_void_p), ("N", ctypes.c_int64), ("K", ctypes.c_int64)]


def _declare(L):
    i64, i32, vp, u32, sz = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_uint, ctypes.c_size_t
    L.bw_rtn_quantize_pack.argtypes = [vp, i32, i64, i64, i32, i32, vp, vp, i32, vp, i32, u32, vp]
    L.bw_rtn_quantize_pack.restype = i32
    L.bw_rtn_batch_table_bytes.argtypes = [i32]
    L.bw_rtn_batch_table_bytes.restype = sz
    L.bw_rtn_quantize_pack_batch.argtypes = [ctypes.POINTER(RtnJob), i32, i32, i32, i32, i32, i32, u32, vp, sz, vp]
    L.bw_rtn_quantize_pack_batch.restype = i32
    L.bw_peer_alloc.argtypes = [sz, ctypes.POINTER(vp), ctypes.c_char_p]
    L.bw_peer_alloc.restype = i32
    L.bw_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    L.bw_peer_open.restype = i32
    L.bw_peer_close.argtypes = [vp]
    L.bw_peer_close.restype = i32
    L.bw_peer_free.argtypes = [vp]
    L.bw_peer_free.restype = i32
    L.bw_peer_flag_bytes.restype = sz
    L.bw_peer_state_bytes.restype = sz
    L.bw_peer_allreduce_f16.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(vp), i32, i32, vp, i64, vp, vp]
    L.bw_peer_allreduce_f16.restype = i32
    L.bw_peer_allreduce2_f16.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(vp), i32, i32, vp, i64, vp, vp]
    L.bw_peer_allreduce2_f16.restype = i32
    L.bw_fake_quant.argtypes = [vp, i32, i64, i64, i32, i32, vp, vp, vp, i32, vp, vp, vp]
    L.bw_fake_quant.restype = i32
    L.bw_fake_quant_native16.argtypes = [vp, i32, i64, i64, i32, i32, vp, vp, vp, vp, vp, vp]
    L.bw_fake_quant_native16.restype = i32
    L.bw_fake_quant_backward.argtypes = [vp, i32, i64, i64, i32, i32, vp, vp, vp, i32, vp, vp, vp, vp]
    L.bw_fake_quant_backward.restype = i32
    L.bw_dequantize.argtypes = [vp, vp, i32, vp, i32, i64, i64, i32, i32, vp, i32, vp]
    L.bw_dequantize.restype = i32
    L.bw_qmatmul_workspace_bytes.argtypes = [i64, i64, i64, i32, i32]
    L.bw_qmatmul_workspace_bytes.restype = sz
    L.bw_qmatmul_workspace_bytes_for.argtypes = [i64, i64, i64, i32, i32, i32, i32]
    L.bw_qmatmul_workspace_bytes_for.restype = sz
    L.bw_qmatmul.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp, vp, vp, i32, i32, i32, vp, sz, vp]
    L.bw_qmatmul.restype = i32
    L.bw_qmatmul_fused.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp, vp, vp, i32, i32, i32, ctypes.POINTER(Epilogue), vp, sz, vp]
    L.bw_qmatmul_fused.restype = i32
    L.bw_qmatmul_noalloc.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp, vp, vp, i32, i32, i32, vp]
    L.bw_qmatmul_noalloc.restype = i32
    L.bw_qmatmul_noalloc_max_scratch_bytes.argtypes = []
    L.bw_qmatmul_noalloc_max_scratch_bytes.restype = sz
    L.bw_qmatmul_host.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, vp,
                                  sz, vp]
    L.bw_qmatmul_host.restype = i32
    L.bw_qmatmul_grad_input.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp, vp, i32, i32, vp]
    L.bw_qmatmul_grad_input.restype = i32
    L.bw_status_string.argtypes = [i32]
    L.bw_status_string.restype = ctypes.c_char_p
    L.bw_last_cuda_error.argtypes = []
    L.bw_last_cuda_error.restype = ctypes.c_char_p
    L.bw_last_qmatmul_kernel.argtypes = []
    L.bw_last_qmatmul_kernel.restype = ctypes.c_char_p
    L.bw_version.argtypes = []
    L.bw_version.restype = i32
    L.bw_device_status.argtypes = []
    L.bw_device_status.restype = i32
    L.bw_selftest_division.argtypes = [ctypes.c_ulonglong, ctypes.c_ulonglong]
    L.bw_selftest_division.restype = ctypes.c_longlong


def lib():
    """Loads (building first if the .so is absent and nvcc is present) the native library."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    try:
                        from ..csrc.build import build
                        build()
                    except Exception as e:  # noqa: BLE001
                        raise RuntimeError(
                            "bitween_b200: the CUDA extension libbitween_b200.so is not built and could "
                            f"not be built here ({e}). Run `python -m bitween_b200.csrc.build`. "
                            "There is no CPU fallback.") from e
                L = ctypes.CDLL(LIB_PATH)
                _declare(L)
                _lib = L
    return _lib


def check(status):
    if status != 0:
        L = lib()
        text = L.bw_status_string(status).decode()
        if status == 8:
            text += ": " + L.bw_last_cuda_error().decode()
        raise BitweenKernelError(status, text)


def require_cuda(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"bitween_b200: `{name}` must be a CUDA tensor; this library has no CPU path")
    return t


def stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


_workspaces = {}
_retired = []


def workspace(device, nbytes):
    """Caller-owned scratch for bw_qmatmul, cached per (device, stream): calls that may overlap on
    the GPU must not share scratch, and calls on one stream are ordered.  The buffer only grows;
    it is never freed while the process lives, so pointers captured in CUDA graphs stay valid
    as long as the first capture already saw the largest size it needs."""
    if nbytes == 0:
        return None
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _retired.append(buf)   # a captured CUDA graph may still hold its address
        buf = torch.empty(max(nbytes, 1 << 21), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def last_qmatmul_kernel():
    return lib().bw_last_qmatmul_kernel().decode()
