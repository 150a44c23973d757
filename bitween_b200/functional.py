"""RTN group-wise quantize/pack and dequantize -- same signatures, return values and packed
layout as the reference's bitween/functional.py, computed by the sm_100a kernels behind the
C ABI (bw_rtn_quantize_pack / bw_dequantize) instead of eager tensor ops.

CPU tensors are accepted the way the reference accepts them (results come back on the
tensor's device), but the arithmetic always runs on a CUDA device; without one the calls
raise -- there is no CPU implementation in this package.
"""
import torch

from .kernels import _lib

_FLOAT_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


def _compute_device(t):
    if t.is_cuda:
        return t.device
    if not torch.cuda.is_available():
        raise RuntimeError("bitween_b200: no CUDA device available and this library has no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


def _rtn_launch(weight, bits, group_size, scale_dtype, zp_dtype, upcast, flags=0):
    """weight: contiguous CUDA [N,K] float tensor.  Returns (q, scale, zp) on that device."""
    N, K = weight.shape
    vpi = 32 // bits
    G = K // group_size
    q = torch.empty((N, K // vpi), dtype=torch.int32, device=weight.device)
    scale = torch.empty((N, G), dtype=scale_dtype, device=weight.device)
    zp = torch.empty((N, G), dtype=zp_dtype, device=weight.device)
    L = _lib.lib()
    with torch.cuda.device(weight.device):
        rc = L.bw_rtn_quantize_pack(_lib.ptr(weight), _lib.dtype_code(weight.dtype), N, K, bits, group_size,
                                    _lib.ptr(q), _lib.ptr(scale), _lib.dtype_code(scale_dtype),
                                    _lib.ptr(zp), _lib.dtype_code(zp_dtype),
                                    (_lib.RTN_UPCAST_F32 if upcast else 0) | flags, _lib.stream_ptr(weight.device))
    _lib.check(rc)
    return q, scale, zp


def _validate(weight, bits, group_size):
    assert bits in [2, 4, 8], "Only 2, 4, or 8-bit quantization supported."
    if weight.dim() != 2:
        raise ValueError("weight must be 2-D [out_features, in_features]")
    if group_size < 1:
        raise ValueError("Group size must be at least 1.")
    out_features, in_features = weight.shape
    pad = (group_size - in_features % group_size) % group_size
    if pad > 0:
        raise ValueError(f"Padding {pad} columns to {in_features} to make it a multiple of {group_size}")
    if in_features % (32 // bits) != 0:
        # the reference fails here too (shape mismatch in its packing loop / final view)
        raise RuntimeError(f"in_features={in_features} is not a multiple of {32 // bits} codes per int32")


@torch.no_grad()
def quantize_rtn(weight: torch.Tensor, bits: int = 8, group_size: int = 32):
    """Drop-in for bitween/functional.py:3-45.

    Returns `(q_packed int32 [N, K*bits/32], scale [N, K/g] in weight.dtype,
    zero_point int32 [N, K/g], group_size)`; bit-identical to the reference run on CPU for
    float32, float16 and bfloat16 weights (arithmetic in the weight's own dtype, as torch does).
    """
    _validate(weight, bits, group_size)
    if weight.dtype not in _FLOAT_DTYPES:
        raise TypeError(f"quantize_rtn: unsupported weight dtype {weight.dtype} (float32/float16/bfloat16)")
    src_device = weight.device
    w = weight.detach().to(_compute_device(weight)).contiguous()
    q, scale, zp = _rtn_launch(w, bits, group_size, weight.dtype, torch.int32, upcast=False)
    if not src_device.type == "cuda":
        q, scale, zp = q.to(src_device), scale.to(src_device), zp.to(src_device)
    return q, scale, zp, group_size


@torch.no_grad()
def quantize_rtn_to_module_buffers(weight: torch.Tensor, bits: int, group_size: int):
    """The fused form of what QuantizedLinear.from_float needs (bitween/modules.py:189-213):
    fp32 arithmetic on the up-cast weight, packed codes, and scale / zero_point already in the
    fp16 module-buffer dtypes -- one kernel, no fp32 copy of the layer, no temporaries.
    Results equal `quantize_rtn(weight.float())` followed by the reference's `.copy_()` casts.
    """
    _validate(weight, bits, group_size)
    if weight.dtype not in _FLOAT_DTYPES:
        weight = weight.to(torch.float32)          # e.g. float64 layers: same cast the reference does
    w = weight.detach().to(_compute_device(weight)).contiguous()
    return _rtn_launch(w, bits, group_size, torch.float16, torch.float16, upcast=True)


@torch.no_grad()
def quantize_rtn_many_to_module_buffers(weights, bits: int, group_size: int):
    """`quantize_rtn_to_module_buffers` for a list of weight matrices (the linears of a decoder
    block, or of a whole model) with ONE kernel launch per (device, dtype) instead of one per
    layer (C ABI: bw_rtn_quantize_pack_batch).  Returns a list of (qweight, scale, zero_point)
    in the order of `weights`; every result equals the single-layer call's bit for bit."""
    prepared = []
    for weight in weights:
        _validate(weight, bits, group_size)
        if weight.dtype not in _FLOAT_DTYPES:
            weight = weight.to(torch.float32)
        prepared.append(weight.detach().to(_compute_device(weight)).contiguous())
    results = [None] * len(prepared)
    groups = {}
    for i, w in enumerate(prepared):
        groups.setdefault((w.device, w.dtype), []).append(i)
    vpi = 32 // bits
    L = _lib.lib()
    for (device, dtype), idx in groups.items():
        jobs = (_lib.RtnJob * len(idx))()
        for j, i in enumerate(idx):
            w = prepared[i]
            N, K = w.shape
            q = torch.empty((N, K // vpi), dtype=torch.int32, device=device)
            s = torch.empty((N, K // group_size), dtype=torch.float16, device=device)
            z = torch.empty((N, K // group_size), dtype=torch.float16, device=device)
            results[i] = (q, s, z)
            jobs[j] = _lib.RtnJob(w.data_ptr(), q.data_ptr(), s.data_ptr(), z.data_ptr(), N, K)
        with torch.cuda.device(device):
            nbytes = L.bw_rtn_batch_table_bytes(len(idx))
            table = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=device)
            rc = L.bw_rtn_quantize_pack_batch(jobs, len(idx), _lib.dtype_code(dtype), bits, group_size, _lib.F16, _lib.F16,
                                              _lib.RTN_UPCAST_F32, _lib.ptr(table), table.numel(), _lib.stream_ptr(device))
        _lib.check(rc)
        # the kernel reads `table` and the weights asynchronously: keep them alive until it has run
        table.record_stream(torch.cuda.current_stream(device))
        for i in idx:
            prepared[i].record_stream(torch.cuda.current_stream(device))
    return results


@torch.no_grad()
def dequantize_rtn(q_packed: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor, group_size: int,
                   bits: int = 8, out_dtype: torch.dtype = torch.float32):
    """Drop-in for bitween/functional.py:47-71: float32 [N, K] = scale * (code - zero_point).
    `out_dtype` (fp16/bf16) is an extension; fp16 scale/zero_point with fp16 output reproduces
    the reference module's device kernel (bitween/modules.py:10-58) bit for bit."""
    assert bits in [2, 4, 8], "Only 2, 4, or 8-bit quantization supported."
    if q_packed.dim() != 2 or q_packed.dtype != torch.int32:
        raise ValueError("q_packed must be a 2-D int32 tensor")
    vpi = 32 // bits
    N, packed = q_packed.shape
    K = packed * vpi
    if group_size < 1 or K % group_size != 0:
        raise ValueError(f"in_features={K} is not a multiple of group_size={group_size}")
    G = K // group_size
    src_device = q_packed.device
    dev = _compute_device(q_packed)
    q = q_packed.detach().to(dev).contiguous()
    s = scale.detach().to(dev).reshape(N, G).contiguous()
    z = zero_point.detach().to(dev).reshape(N, G).contiguous()
    if s.dtype not in _FLOAT_DTYPES:
        s = s.to(torch.float32)
    if z.dtype not in _FLOAT_DTYPES and z.dtype != torch.int32:
        z = z.to(torch.int32) if not z.dtype.is_floating_point else z.to(torch.float32)
    out = torch.empty((N, K), dtype=out_dtype, device=dev)
    L = _lib.lib()
    with torch.cuda.device(dev):
        rc = L.bw_dequantize(_lib.ptr(q), _lib.ptr(s), _lib.dtype_code(s.dtype), _lib.ptr(z),
                             _lib.dtype_code(z.dtype), N, K, bits, group_size, _lib.ptr(out),
                             _lib.dtype_code(out_dtype), _lib.stream_ptr(dev))
    _lib.check(rc)
    return out if src_device.type == "cuda" else out.to(src_device)
