"""`WrapperLinear` -- the trainable stand-in for a linear layer of the reference's trainable and
gradual modes (bitween/wrapper.py:28-242), with its fake-quantized weight computed by one fused
sm_100a kernel instead of about ten eager passes over [N,K].

Same constructor, buffers (`orig_weight`, `orig_bias`, `base_qweight`, `base_scale`,
`base_zero_point`), parameters (`value`, `min_scale`, `max_scale`) and methods as the reference
class, so `unified_wrapper` / `unified_unwrapper` / `wrap_model_for_training`
(bitween/wrapper.py:245-372) work on it unchanged; they are mirrored below.

What runs where on every training step (bitween/wrapper.py:116-172):
  * the per-group minima / maxima of the frozen weight are taken once at construction, not on
    every call (they cannot change: `orig_weight` is a buffer);
  * scale and float zero point come from them and the learnable factors on [N, K/group_size]
    tensors with torch ops, so autograd tracks `min_scale` / `max_scale` exactly as in the
    reference (clamp included);
  * the [N,K] part -- divide, add, perturb, round, clamp, dequantize -- is `bw_fake_quant`, and
    its backward for (scale, zero_point) is `bw_fake_quant_backward`.
The fused kernels compute in fp32, which is what the reference computes whenever an fp32
parameter takes part (fp32 weights, or min/max tuning on: `torch.ones` factors are fp32 and
promote everything).  With 16-bit weights AND min/max tuning off the reference rounds every
intermediate to 16 bits; `bw_fake_quant_native16` does the same, rounding after each operation.
"""
from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as F

from .functional import quantize_rtn
from .kernels import _lib
from .modules import QuantizedLinear

_BWD_GROUPS = (4, 8, 16, 32, 64, 128, 256)
_ERR_GROUP, _ERR_ALIGN = 2, 5


def _value_args(value):
    if value is None:
        return None, 0
    return _lib.ptr(value), _lib.dtype_code(value.dtype)


class _FakeQuant(torch.autograd.Function):
    """(w, scale[N,G], zero_point[N,G], value) -> (w_dq [N,K] fp32, w_q [N,K] fp32)."""

    @staticmethod
    def forward(ctx, w, scale, zero_point, value, bits, group_size, want_q):
        N, K = w.shape
        scale = scale.contiguous()
        zero_point = zero_point.contiguous()
        v = None if value is None else value.detach().contiguous()
        dq = torch.empty((N, K), dtype=torch.float32, device=w.device)
        wq = torch.empty((N, K), dtype=torch.float32, device=w.device) if want_q else None
        vptr, vdt = _value_args(v)
        with torch.cuda.device(w.device):
            rc = _lib.lib().bw_fake_quant(_lib.ptr(w), _lib.dtype_code(w.dtype), N, K, bits, group_size,
                                          _lib.ptr(scale), _lib.ptr(zero_point), vptr, vdt, _lib.ptr(dq),
                                          None if wq is None else _lib.ptr(wq), _lib.stream_ptr(w.device))
        _lib.check(rc)
        ctx.save_for_backward(w, scale, zero_point, v)
        ctx.bits, ctx.group_size = bits, group_size
        if wq is None:
            wq = dq.new_empty(0)
        ctx.mark_non_differentiable(wq)
        return dq, wq

    @staticmethod
    def backward(ctx, grad_dq, _grad_q):
        w, scale, zero_point, v = ctx.saved_tensors
        N, K = w.shape
        g = ctx.group_size
        grad = grad_dq.to(torch.float32).contiguous()
        rc = _ERR_GROUP
        if g in _BWD_GROUPS:
            gs = torch.empty_like(scale)
            gz = torch.empty_like(zero_point)
            vptr, vdt = _value_args(v)
            with torch.cuda.device(w.device):
                rc = _lib.lib().bw_fake_quant_backward(_lib.ptr(w), _lib.dtype_code(w.dtype), N, K, ctx.bits, g,
                                                       _lib.ptr(scale), _lib.ptr(zero_point), vptr, vdt,
                                                       _lib.ptr(grad), _lib.ptr(gs), _lib.ptr(gz),
                                                       _lib.stream_ptr(w.device))
        if rc not in (_ERR_GROUP, _ERR_ALIGN):
            _lib.check(rc)
        else:
            # group sizes / alignments the shuffle reduction does not cover: same sums with torch reductions
            s3, z3 = scale.unsqueeze(-1), zero_point.unsqueeze(-1)
            t = w.view(N, -1, g).to(torch.float32) / s3 + z3
            if v is not None:
                t = t + v.view(N, -1, g)
            q = torch.clamp(torch.round(t), 0, (1 << ctx.bits) - 1)
            g3 = grad.view(N, -1, g)
            gs = (g3 * (q - z3)).sum(-1)
            gz = -scale * g3.sum(-1)
        # round() passes no gradient (bitween/wrapper.py:152): nothing for w or value
        return None, gs, gz, None, None, None, None


def fake_quantize(weight, scale, zero_point, value, bits, group_size, want_q=True):
    """w_dq, w_q of bitween/wrapper.py:143-155 from per-group fp32 scale / zero point [N,G]."""
    _lib.require_cuda(weight, "weight")
    if scale.dtype != torch.float32 or zero_point.dtype != torch.float32:
        raise TypeError("fake_quantize computes in fp32: scale and zero_point must be fp32")
    if weight.dim() != 2 or weight.shape[1] % group_size != 0:
        raise ValueError("weight must be [N,K] with K a multiple of group_size")
    G = weight.shape[1] // group_size
    if tuple(scale.shape) != (weight.shape[0], G) or tuple(zero_point.shape) != (weight.shape[0], G):
        raise ValueError(f"scale / zero_point must have shape {(weight.shape[0], G)}")
    if value is not None and value.shape != weight.shape:
        raise ValueError("value must have the weight's shape")
    return _FakeQuant.apply(weight.contiguous(), scale, zero_point, value, bits, group_size, want_q)


class WrapperLinear(nn.Module):
    """Drop-in for bitween/wrapper.py:28-242."""

    def __init__(self, orig_layer, bits=8, group_size=32, enable_minmax_tuning=True, enable_round_tuning=True,
                 device="cpu"):
        super().__init__()
        self.orig_layer = orig_layer
        self.bits = bits
        self.group_size = group_size
        self.enable_minmax_tuning = enable_minmax_tuning
        self.enable_round_tuning = enable_round_tuning
        # the layer's own device wins over the argument, as in bitween/wrapper.py:53-54
        self.device = orig_layer.weight.device
        self.register_buffer("orig_weight", orig_layer.weight.data.clone())
        if orig_layer.bias is not None:
            self.register_buffer("orig_bias", orig_layer.bias.data.clone())
        else:
            self.orig_bias = None
        self._init_quantization_params()
        self._init_learnable_params()
        self.to(self.device)
        self.best_params = {}
        self.best_loss = float("inf")

    def _init_quantization_params(self):
        """RTN codes of the frozen weight (bitween/wrapper.py:77-91) and its group extrema."""
        with torch.no_grad():
            qweight, scale, zero_point, _ = quantize_rtn(self.orig_weight, bits=self.bits, group_size=self.group_size)
            self.register_buffer("base_qweight", qweight)
            self.register_buffer("base_scale", scale)
            self.register_buffer("base_zero_point", zero_point)
            N, K = self.orig_weight.shape
            grouped = self.orig_weight.view(N, K // self.group_size, self.group_size)
            # not in the reference's state dict: derived from orig_weight
            self.register_buffer("_w_min", grouped.amin(dim=-1), persistent=False)
            self.register_buffer("_w_max", grouped.amax(dim=-1), persistent=False)

    def _init_learnable_params(self):
        """bitween/wrapper.py:93-114: `value` zeros like the weight, min/max factors fp32 ones."""
        shape = self.orig_weight.shape
        self.value = nn.Parameter(torch.zeros_like(self.orig_weight)) if self.enable_round_tuning else None
        if self.enable_minmax_tuning:
            groups = (shape[0], shape[1] // self.group_size)
            self.min_scale = nn.Parameter(torch.ones(groups) * 1.0)
            self.max_scale = nn.Parameter(torch.ones(groups) * 1.0)
        else:
            self.min_scale = None
            self.max_scale = None

    def _group_params(self):
        """scale, zero_point [N,G] of bitween/wrapper.py:131-140."""
        max_val = (1 << self.bits) - 1
        w_min, w_max = self._w_min, self._w_max
        if self.min_scale is not None and self.max_scale is not None:
            w_min = w_min * self.min_scale
            w_max = w_max * self.max_scale
        # A tensor divisor: torch's CUDA kernel turns division by a Python scalar into a multiplication
        # by its reciprocal (one ulp off on some groups); the correctly rounded quotient is what the
        # reference computes on the CPU and what the golden vectors hold.
        span = w_max - w_min
        scale = torch.clamp(span / torch.full((), max_val, dtype=span.dtype, device=span.device), min=1e-8)
        return scale, -w_min / scale

    def _quantize_weight_with_learnable_params(self):
        """Returns (w_dq [N,K], w_q [N,G,g], scale [N,G], zero_point [N,G]) like bitween/wrapper.py:116-172."""
        N, K = self.orig_weight.shape
        G = K // self.group_size
        scale, zero_point = self._group_params()
        if scale.dtype != torch.float32:
            return self._all_16bit_path(scale, zero_point)
        w_dq, w_q = fake_quantize(self.orig_weight, scale, zero_point, self.value, self.bits, self.group_size)
        return w_dq, w_q.view(N, G, self.group_size), scale, zero_point

    def _all_16bit_path(self, scale, zero_point):
        # 16-bit weights with min/max tuning off: every intermediate is rounded to the weight's dtype in
        # the reference (no fp32 tensor takes part); bw_fake_quant_native16 rounds after every operation.
        N, K = self.orig_weight.shape
        w = self.orig_weight
        _lib.require_cuda(w, "orig_weight")
        scale, zero_point = scale.contiguous(), zero_point.contiguous()
        v = None if self.value is None else self.value.detach().contiguous()
        dq = torch.empty_like(w)
        wq = torch.empty_like(w)
        with torch.cuda.device(w.device):
            rc = _lib.lib().bw_fake_quant_native16(_lib.ptr(w), _lib.dtype_code(w.dtype), N, K, self.bits, self.group_size,
                                                   _lib.ptr(scale), _lib.ptr(zero_point), None if v is None else _lib.ptr(v),
                                                   _lib.ptr(dq), _lib.ptr(wq), _lib.stream_ptr(w.device))
        _lib.check(rc)
        # (nothing here has a gradient in the reference either: round() cuts `value` off, and there are no
        # min/max factors in this mode)
        return dq, wq.view(N, K // self.group_size, self.group_size), scale, zero_point

    def forward(self, x):
        scale, zero_point = self._group_params()
        if scale.dtype != torch.float32:
            weight_dq = self._all_16bit_path(scale, zero_point)[0]
        else:
            weight_dq, _ = fake_quantize(self.orig_weight, scale, zero_point, self.value, self.bits, self.group_size,
                                         want_q=False)
        return F.linear(x, weight_dq, self.orig_bias)

    def update_best_params(self, loss_value):
        """bitween/wrapper.py:183-194."""
        if loss_value < self.best_loss:
            self.best_loss = loss_value
            self.best_params = {}
            for name in ("value", "min_scale", "max_scale"):
                p = getattr(self, name)
                if p is not None:
                    self.best_params[name] = p.data.clone()

    def apply_best_params(self):
        """bitween/wrapper.py:196-205."""
        for name, saved in self.best_params.items():
            p = getattr(self, name)
            if p is not None:
                p.data.copy_(saved)

    def to_quantized_linear(self) -> QuantizedLinear:
        """bitween/wrapper.py:207-242: RTN of (orig_weight + value), i.e. the min/max factors do
        not reach the packed layer -- kept, since the packed result is what parity is judged on."""
        with torch.no_grad():
            self.apply_best_params()
            adjusted = self.orig_weight if self.value is None else self.orig_weight + self.value
            qweight, scale, zero_point, _ = quantize_rtn(adjusted, bits=self.bits, group_size=self.group_size)
            q_layer = QuantizedLinear(self.orig_layer.in_features, self.orig_layer.out_features, bits=self.bits,
                                      group_size=self.group_size, bias=self.orig_layer.bias is not None)
            q_layer.qweight.copy_(qweight)
            q_layer.scale.copy_(scale)
            q_layer.zero_point.copy_(zero_point)
            if self.orig_layer.bias is not None:
                q_layer.bias.copy_(self.orig_layer.bias)
            return q_layer


def _get_module(model, module_name: str):
    cur = model
    for token in module_name.split("."):
        cur = getattr(cur, token)
    return cur


def _set_module(model, module_name: str, new_module):
    tokens = module_name.split(".")
    cur = model
    for token in tokens[:-1]:
        cur = getattr(cur, token)
    setattr(cur, tokens[-1], new_module)


def unified_wrapper(module, enable_minmax_tuning=True, enable_round_tuning=True, bits=8, group_size=32,
                    device="cpu", ignore_layers=None, module_prefix=""):
    """A single nn.Linear or every nn.Linear of a block becomes a WrapperLinear; returns
    (module, names of the wrapped layers) like bitween/wrapper.py:245-316."""
    ignore_layers = ignore_layers or set()
    if isinstance(module, WrapperLinear):
        print(f"Module already wrapped, skipping: {module_prefix}")
        return module, []
    kw = dict(bits=bits, group_size=group_size, enable_minmax_tuning=enable_minmax_tuning,
              enable_round_tuning=enable_round_tuning, device=device)
    if isinstance(module, nn.Linear):
        if module_prefix in ignore_layers:
            print(f"  Skipping ignored layer: {module_prefix}")
            return module, []
        return WrapperLinear(module, **kw), ["single_layer"]
    names = []
    for name, sub in list(module.named_modules()):
        if not isinstance(sub, nn.Linear) or ".orig_layer" in f".{name}":
            continue
        full = f"{module_prefix}.{name}" if module_prefix and name else (module_prefix or name)
        if full in ignore_layers:
            print(f"  Skipping ignored layer: {full}")
            continue
        _set_module(module, name, WrapperLinear(sub, **kw))
        names.append(name)
    return module, names


def unified_unwrapper(module, apply_quantization=True):
    """bitween/wrapper.py:319-346: wrappers become QuantizedLinear, or the original layers again."""
    if isinstance(module, WrapperLinear):
        return module.to_quantized_linear() if apply_quantization else module.orig_layer
    for name, sub in list(module.named_modules()):
        if isinstance(sub, WrapperLinear):
            _set_module(module, name, sub.to_quantized_linear() if apply_quantization else sub.orig_layer)
    return module


def wrapper_block(block, enable_minmax_tuning=True, enable_round_tuning=True, bits=8, group_size=32, device="cpu",
                  ignore_layers=None, block_prefix=""):
    """bitween/wrapper.py:350-355."""
    _, quantized = unified_wrapper(block, enable_minmax_tuning, enable_round_tuning, bits, group_size, device,
                                   ignore_layers, block_prefix)
    unquantized = [n for n, m in block.named_modules() if not isinstance(m, WrapperLinear)]
    return quantized, unquantized


def unwrapper_block(block, apply_quantization=True):
    """bitween/wrapper.py:358-360."""
    unified_unwrapper(block, apply_quantization)


def wrap_model_for_training(model, block_names: List[str], enable_minmax_tuning: bool, bits: int, group_size: int,
                            ignore_layers: set):
    """bitween/wrapper.py:362-405: wraps the named blocks, returns {name: info}.  Single layers
    are returned, not installed, exactly as there."""
    info = {}
    for module_name in block_names:
        module = _get_module(model, module_name)
        wrapped, names = unified_wrapper(module, enable_minmax_tuning=enable_minmax_tuning, enable_round_tuning=True,
                                         bits=bits, group_size=group_size, device=next(module.parameters()).device,
                                         ignore_layers=ignore_layers, module_prefix=module_name)
        if names:
            info[module_name] = {"wrapped_module": wrapped, "quantized_names": names,
                                 "is_single_layer": isinstance(wrapped, WrapperLinear), "original_module": module}
        else:
            print(f"  No layers to wrap in {module_name}")
    return info
