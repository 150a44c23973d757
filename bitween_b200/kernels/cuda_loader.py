"""`quantized_matmul_cuda` -- the fused dequantize+matmul entry point.

The reference's scripts import this symbol from `bitween.kernels.cuda_loader`
(main.py:401, README.md:347) and call it as
`quantized_matmul_cuda(x, qweight, scale, zero_point, bias, bits, group_size)`
(main.py:433); the module itself is missing from the reference snapshot.  Here it is a
thin wrapper over the C-ABI call `bw_qmatmul`.
"""
import torch

from . import _lib

_OUT_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


def _as_half(t, name):
    _lib.require_cuda(t, name)
    if t.dtype != torch.float16:
        t = t.to(torch.float16)
    return t.contiguous()


def quantized_matmul_cuda(x, qweight, scale, zero_point, bias, bits, group_size, out_dtype=None,
                          out=None, activation=None, residual=None):
    """x [..., K] (fp16/bf16/fp32, cast to fp16 as bitween/modules.py:74 does) times the packed
    weight [N, K*bits/32] with fp16 per-group scale / zero_point [N, K/group_size] and an
    optional fp16 bias [N].  Returns fp16 [..., N] exactly as the reference forward does
    (bitween/modules.py:106); `out_dtype` (bf16 / fp32) is an extension of this library.

    `activation="relu"` and `residual` (fp16 [..., N], added last) fuse what follows the linear in
    a decoder block into the kernel's output stage (C ABI: bw_qmatmul_fused): the result equals
    `torch.relu(linear) + residual` computed op by op in fp16.  `activation="silu_mul"` is the
    gated feed-forward as one GEMM: the packed weight holds (gate, up) row pairs (see
    `interleave_gate_up`) and the result is `silu(gate) * up` of shape [..., N/2].
    """
    if bits not in (2, 4, 8):
        raise ValueError("Only 2, 4, or 8 bits are supported.")
    _lib.require_cuda(x, "x")
    _lib.require_cuda(qweight, "qweight")
    if qweight.dtype != torch.int32:
        raise TypeError("qweight must be int32")
    out_dtype = torch.float16 if out_dtype is None else out_dtype
    if out_dtype not in _OUT_DTYPES:
        raise TypeError(f"unsupported out_dtype {out_dtype}")
    if x.dtype not in _OUT_DTYPES:
        x = x.to(torch.float16)
    K = x.shape[-1]
    N = qweight.shape[0]
    vpi = 32 // bits
    if qweight.shape[1] * vpi != K:
        raise ValueError(f"x has {K} input features but qweight packs {qweight.shape[1] * vpi}")
    if group_size < 1 or K % group_size != 0:
        raise ValueError("Group size must be at least 1 and divide in_features.")
    G = K // group_size
    if tuple(scale.shape) != (N, G) or tuple(zero_point.shape) != (N, G):
        raise ValueError(f"scale / zero_point must have shape {(N, G)}")
    x2 = x.reshape(-1, K).contiguous()
    M = x2.shape[0]
    qweight = qweight.contiguous()
    scale = _as_half(scale, "scale")
    zero_point = _as_half(zero_point, "zero_point")
    if bias is not None:
        bias = _as_half(bias, "bias")
        if bias.numel() != N:
            raise ValueError("bias must have out_features elements")
    dev = x2.device
    for name, t in (("qweight", qweight), ("scale", scale), ("zero_point", zero_point), ("bias", bias)):
        if t is not None and t.device != dev:
            raise RuntimeError(f"`{name}` is on {t.device} but x is on {dev}")
    if activation not in (None, "relu", "silu_mul"):
        raise ValueError("activation must be None, 'relu' or 'silu_mul'")
    if activation == "silu_mul" and N % 4 != 0:
        raise ValueError("'silu_mul' pairs adjacent weight rows (gate, up): out_features must be a multiple of 4")
    N_out = N // 2 if activation == "silu_mul" else N
    if out is None:
        out = torch.empty((M, N_out), dtype=out_dtype, device=dev)
    else:
        if out.dtype != out_dtype or tuple(out.shape) != (M, N_out) or not out.is_contiguous() or out.device != dev:
            raise ValueError("`out` must be a contiguous [M, N] tensor of out_dtype on x's device ([M, N/2] for 'silu_mul')")
    ep = None
    if activation is not None or residual is not None:
        if residual is not None:
            _lib.require_cuda(residual, "residual")
            if residual.dtype != torch.float16 or residual.numel() != M * N_out or residual.device != dev:
                raise ValueError("`residual` must be an fp16 tensor of the output's shape on x's device")
            residual = residual.contiguous()
        act = {None: _lib.ACT_NONE, "relu": _lib.ACT_RELU, "silu_mul": _lib.ACT_SILU_MUL}[activation]
        ep = _lib.Epilogue(act, None if residual is None else residual.data_ptr())
    L = _lib.lib()
    with torch.cuda.device(dev):
        ws_bytes = L.bw_qmatmul_workspace_bytes_for(M, N, K, bits, group_size, _lib.dtype_code(x2.dtype),
                                                    16 if x2.data_ptr() % 16 == 0 else 2)
        ws = _lib.workspace(dev, ws_bytes)
        args = (_lib.ptr(x2), _lib.dtype_code(x2.dtype), M, N, K, _lib.ptr(qweight),
                _lib.ptr(scale), _lib.ptr(zero_point), _lib.ptr(bias), _lib.ptr(out),
                _lib.dtype_code(out_dtype), bits, group_size)
        tail = (_lib.ptr(ws), 0 if ws is None else ws.numel(), _lib.stream_ptr(dev))
        rc = L.bw_qmatmul(*args, *tail) if ep is None else L.bw_qmatmul_fused(*args, ep, *tail)
    _lib.check(rc)
    return out.reshape(*x.shape[:-1], N_out)


def interleave_gate_up(gate, up):
    """Row-interleaves the tensors of a gate and an up projection (packed words, scales, zero points or
    biases of equal shape): row 2i = gate row i, row 2i+1 = up row i -- the [2*ffn, K] layout that
    `activation="silu_mul"` expects."""
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("gate and up must have the same shape and dtype")
    return torch.stack((gate, up), dim=1).reshape(2 * gate.shape[0], *gate.shape[1:]).contiguous()


def quantized_matmul_grad_input(grad_output, qweight, scale, zero_point, bits, group_size):
    """grad_input of the backward pass (bitween/modules.py:108-141): grad_output [..., N] times
    the dequantized weight [N, K] -> [..., K] in grad_output's dtype."""
    _lib.require_cuda(grad_output, "grad_output")
    if grad_output.dtype not in _OUT_DTYPES:
        grad_output = grad_output.to(torch.float32)
    N = qweight.shape[0]
    K = qweight.shape[1] * (32 // bits)
    g2 = grad_output.reshape(-1, N).contiguous()
    M = g2.shape[0]
    scale = _as_half(scale, "scale")
    zero_point = _as_half(zero_point, "zero_point")
    out = torch.empty((M, K), dtype=g2.dtype, device=g2.device)
    L = _lib.lib()
    with torch.cuda.device(g2.device):
        rc = L.bw_qmatmul_grad_input(_lib.ptr(g2), _lib.dtype_code(g2.dtype), M, N, K,
                                     _lib.ptr(qweight.contiguous()), _lib.ptr(scale), _lib.ptr(zero_point),
                                     _lib.ptr(out), bits, group_size, _lib.stream_ptr(g2.device))
    _lib.check(rc)
    return out.reshape(*grad_output.shape[:-1], K)


def quantized_matmul_host(x_host, qweight, scale, zero_point, bias, bits, group_size, out_host, x_dev,
                          out_dev):
    """End-to-end form for callers whose activations live in host memory: copies `x_host`
    (pinned) into `x_dev`, runs the fused kernel into `out_dev` and copies the result to
    `out_host` (pinned), all asynchronously on the current stream (C ABI: bw_qmatmul_host).
    The packed weights stay resident on the device.  All buffers are caller-owned:
    x_host/x_dev [M,K] of one dtype, out_host/out_dev [M,N] of one dtype."""
    if x_host.is_cuda or out_host.is_cuda:
        raise RuntimeError("x_host / out_host must be host tensors")
    _lib.require_cuda(x_dev, "x_dev")
    _lib.require_cuda(out_dev, "out_dev")
    M, K = x_host.shape
    N = qweight.shape[0]
    if tuple(x_dev.shape) != (M, K) or x_dev.dtype != x_host.dtype or tuple(out_dev.shape) != (M, N) \
            or tuple(out_host.shape) != (M, N) or out_host.dtype != out_dev.dtype:
        raise ValueError("host/device staging buffers do not match")
    if qweight.shape[1] * (32 // bits) != K:
        raise ValueError("x / qweight shape mismatch")
    if scale.dtype != torch.float16 or zero_point.dtype != torch.float16:
        raise TypeError("scale / zero_point must be fp16 module buffers")
    for t in (x_host, out_host, x_dev, out_dev, qweight, scale, zero_point):
        if not t.is_contiguous():
            raise ValueError("all buffers must be contiguous")
    dev = x_dev.device
    L = _lib.lib()
    with torch.cuda.device(dev):
        ws = _lib.workspace(dev, L.bw_qmatmul_workspace_bytes(M, N, K, bits, group_size))
        rc = L.bw_qmatmul_host(_lib.ptr(x_host), _lib.dtype_code(x_host.dtype), M, N, K, _lib.ptr(qweight),
                               _lib.ptr(scale), _lib.ptr(zero_point), _lib.ptr(bias), _lib.ptr(out_host),
                               _lib.dtype_code(out_host.dtype), bits, group_size, _lib.ptr(x_dev),
                               _lib.ptr(out_dev), _lib.ptr(ws), 0 if ws is None else ws.numel(),
                               _lib.stream_ptr(dev))
    _lib.check(rc)
    return out_host


def quantized_matmul_noalloc(x, qweight, scale, zero_point, bias, bits, group_size, out):
    """Fused dequantize+matmul for callers that must not allocate device memory (inside a CUDA
    graph capture, in an allocation-free serving loop, in a plugin that only receives buffers).

    Same result as `quantized_matmul_cuda`, but nothing is allocated here or in the library: the
    caller passes the output tensor, every tensor must already be a contiguous CUDA tensor of
    its final dtype (fp16 scale / zero_point / bias), and the kernel's scratch is a fixed 2 MiB
    array inside the library (C ABI: bw_qmatmul_noalloc).  Requests that need more scratch raise
    BitweenKernelError (status 11).  All calls on one device share that array: issue them on
    one stream.  Make the first call on a device outside stream capture."""
    for name, t in (("x", x), ("qweight", qweight), ("scale", scale), ("zero_point", zero_point), ("out", out)):
        _lib.require_cuda(t, name)
        if not t.is_contiguous():
            raise ValueError(f"`{name}` must be contiguous (this call may not make copies)")
    if bias is not None and (not bias.is_cuda or not bias.is_contiguous() or bias.dtype != torch.float16):
        raise ValueError("`bias` must be a contiguous fp16 CUDA tensor")
    if scale.dtype != torch.float16 or zero_point.dtype != torch.float16 or qweight.dtype != torch.int32:
        raise TypeError("qweight must be int32 and scale / zero_point fp16")
    if x.dtype not in _OUT_DTYPES or out.dtype not in _OUT_DTYPES:
        raise TypeError("x / out must be fp16, bf16 or fp32")
    K = x.shape[-1]
    N = qweight.shape[0]
    M = x.numel() // K if K else 0
    if qweight.shape[1] * (32 // bits) != K or out.numel() != M * N:
        raise ValueError("shape mismatch between x, qweight and out")
    if group_size < 1 or K % group_size != 0:
        raise ValueError("Group size must be at least 1 and divide in_features.")
    G = K // group_size
    if tuple(scale.shape) != (N, G) or tuple(zero_point.shape) != (N, G):
        raise ValueError(f"scale / zero_point must have shape {(N, G)}")
    if bias is not None and bias.numel() != N:
        raise ValueError("bias must have out_features elements")
    dev = x.device
    L = _lib.lib()
    with torch.cuda.device(dev):
        rc = L.bw_qmatmul_noalloc(_lib.ptr(x), _lib.dtype_code(x.dtype), M, N, K, _lib.ptr(qweight),
                                  _lib.ptr(scale), _lib.ptr(zero_point), _lib.ptr(bias), _lib.ptr(out),
                                  _lib.dtype_code(out.dtype), bits, group_size, _lib.stream_ptr(dev))
    _lib.check(rc)
    return out
