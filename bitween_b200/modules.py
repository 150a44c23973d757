"""QuantizedLinear -- same class surface, buffers, dtypes and pickled state as the reference's
bitween/modules.py:143-217; the forward calls the fused sm_100a dequantize+matmul behind the
C ABI instead of `Triton dequantize -> temporary fp16 [N,K] -> torch.matmul -> bias add`.
"""
import torch
import torch.nn as nn

from .functional import quantize_rtn_to_module_buffers
from .kernels.cuda_loader import quantized_matmul_cuda, quantized_matmul_grad_input


class QuantizedLinearFunction(torch.autograd.Function):
    """Drop-in for bitween/modules.py:60-141.  `apply(x, qweight, scale, zero_point, bias, bits,
    group_size)`; an optional 8th argument selects a non-fp16 output dtype (extension)."""

    @staticmethod
    def forward(ctx, x, qweight, scale, zero_point, bias, bits, group_size, out_dtype=None):
        ctx.save_for_backward(x, qweight, scale, zero_point, bias)
        ctx.bits = bits
        ctx.group_size = group_size
        ctx.nargs = 7 if out_dtype is None else 8
        return quantized_matmul_cuda(x, qweight, scale, zero_point, bias, bits, group_size,
                                     out_dtype=out_dtype)

    @staticmethod
    def backward(ctx, grad_output):
        x, qweight, scale, zero_point, bias = ctx.saved_tensors
        grad_input = None
        # the packed weight is frozen: only the activation gradient exists (modules.py:138-141)
        if ctx.needs_input_grad[0]:
            grad_input = quantized_matmul_grad_input(grad_output, qweight, scale, zero_point,
                                                     ctx.bits, ctx.group_size)
        return (grad_input,) + (None,) * (ctx.nargs - 1)


class QuantizedLinear(nn.Module):
    """A linear layer with 2/4/8-bit group-wise quantized weights (bitween/modules.py:143-217).

    Buffers: `qweight` int32 [out, in*bits/32], `scale` fp16 [out, in/group], `zero_point` fp16
    [out, in/group], `bias` fp16 [out] (or attribute None).  No native handles live on the
    module, so `torch.save(model)` / `state_dict()` round-trip exactly like the reference's.
    """

    def __init__(self, in_features, out_features, bits=8, group_size=32, bias=True, dtype=torch.float16):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.bits = bits
        self.group_size = group_size
        self.requires_grad = False

        if self.bits not in [2, 4, 8]:
            raise ValueError("Only 2, 4, or 8 bits are supported.")
        if group_size < 1:
            raise ValueError("Group size must be at least 1.")

        # The reference ignores `dtype` and always stores / returns fp16 (modules.py:163-167).
        self.dtype = torch.float16

        values_per_int32 = 32 // self.bits
        self.register_buffer("qweight", torch.zeros((out_features, in_features // values_per_int32),
                                                    dtype=torch.int32))
        num_groups = in_features // group_size
        self.register_buffer("scale", torch.zeros((out_features, num_groups), dtype=self.dtype))
        self.register_buffer("zero_point", torch.zeros((out_features, num_groups), dtype=self.dtype))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=self.dtype))
        else:
            self.bias = None

    def forward(self, x):
        out_dtype = getattr(self, "out_dtype", None)   # extension: set layer.out_dtype = torch.bfloat16
        if out_dtype is None:
            return QuantizedLinearFunction.apply(x, self.qweight, self.scale, self.zero_point, self.bias,
                                                 self.bits, self.group_size)
        return QuantizedLinearFunction.apply(x, self.qweight, self.scale, self.zero_point, self.bias,
                                             self.bits, self.group_size, out_dtype)

    @classmethod
    def from_buffers(cls, float_layer: nn.Linear, bits, group_size, qweight, scale, zero_point):
        """A QuantizedLinear for `float_layer` around already computed RTN buffers (the results
        of `quantize_rtn_to_module_buffers`, e.g. from the batched call or a cache).  The buffers
        are adopted, not copied; the bias is cast to fp16 as bitween/modules.py:210-211 does."""
        device = float_layer.weight.device
        q_layer = cls(float_layer.in_features, float_layer.out_features, bits, group_size,
                      bias=float_layer.bias is not None, dtype=torch.float16)
        q_layer = q_layer.to(device)
        q_layer.qweight = qweight.to(device)
        q_layer.scale = scale.to(device)
        q_layer.zero_point = zero_point.to(device)
        if float_layer.bias is not None:
            q_layer.bias.data.copy_(float_layer.bias.data)
        return q_layer

    @classmethod
    def from_float(cls, float_layer: nn.Linear, bits=8, group_size=32):
        """RTN-quantize an nn.Linear.  Results are bit-identical to the reference's
        `deepcopy(layer).to(float32)` -> `quantize_rtn` -> `.copy_()` casts (modules.py:189-213),
        but the weight is read once in its own dtype by one kernel that writes the packed codes
        and the fp16 scale / zero_point directly: no fp32 copy of the layer, no temporaries."""
        buffers = quantize_rtn_to_module_buffers(float_layer.weight.data, bits, group_size)
        return cls.from_buffers(float_layer, bits, group_size, *buffers)

    def __repr__(self):
        return (f"QuantizedLinear(in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}, bits={self.bits}, group_size={self.group_size})")
