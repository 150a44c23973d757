"""Block wrappers of the gradual flow: `BaseBlockWrapper` and `RTNWrapper` with the constructor
arguments, attributes and methods of the reference's bitween/gradual/base_wrapper.py:10-119 and
:242-370, plus `quantize_block`, the per-block RTN loop itself (base_wrapper.py:289-315).

What differs from the reference is how the loop runs, not what it returns: the block's linears
are quantized by ONE batched kernel launch (no per-layer launches, no fp32 copy of each layer),
the nn.Linear weights are not deep-copied on the way (only the rest of the block is), and the
results are cached across the search's repeated (bits, group_size) trials.  The quantized
block's buffers are bit-identical to the reference's.
"""
import copy

import torch
import torch.nn as nn

from ..functional import quantize_rtn_many_to_module_buffers
from ..modules import QuantizedLinear
from .rtn_cache import default_cache


class _LinearPlaceholder(nn.Module):
    """Stands in for an nn.Linear while the rest of a block is deep-copied."""

    def __init__(self, source):
        super().__init__()
        self.__dict__["source"] = source      # not a submodule: invisible to parameters() / state_dict()


def copy_without_linears(module, skip=None):
    """Deep copy of `module` in which every nn.Linear (except those `skip(name, layer)` accepts,
    which are copied normally) is replaced by a placeholder that still points at the ORIGINAL
    layer: the weights that are about to be quantized are never copied.  Returns the copy and
    the list of (dotted name, original layer)."""
    memo, taken = {}, []
    for name, layer in module.named_modules():
        if isinstance(layer, nn.Linear) and not (skip is not None and skip(name, layer)):
            memo[id(layer)] = _LinearPlaceholder(layer)
            taken.append((name, layer))
    if isinstance(module, nn.Linear) and taken and taken[0][1] is module:
        return memo[id(module)], taken
    return copy.deepcopy(module, memo), taken


def replace_leftover_placeholders(module):
    """A layer that the tree references under several names is replaced under its first name only
    (named_modules lists it once -- the reference's loops behave the same way); its other
    references get a float copy, as the reference's deep copy of the whole tree would."""
    for parent in module.modules():
        for key, child in list(parent._modules.items()):
            if isinstance(child, _LinearPlaceholder):
                parent._modules[key] = copy.deepcopy(child.source)


def set_submodule(parent, dotted_name, new_module):
    """Same walk as the reference's RTNWrapper._set_submodule (base_wrapper.py:337-350)."""
    if not dotted_name:
        return
    parts = dotted_name.split(".")
    current = parent
    for part in parts[:-1]:
        current = getattr(current, part)
    setattr(current, parts[-1], new_module)


def quantized_linears(layers, bits, group_size, cache=None):
    """QuantizedLinear for each nn.Linear of `layers`, all cache misses quantized by one batched
    launch per (device, dtype)."""
    out = [None] * len(layers)
    todo = []
    for i, layer in enumerate(layers):
        hit = cache.get(layer.weight, bits, group_size) if cache is not None else None
        if hit is not None:
            out[i] = QuantizedLinear.from_buffers(layer, bits, group_size, *hit)
        else:
            todo.append(i)
    if todo:
        fresh = quantize_rtn_many_to_module_buffers([layers[i].weight.data for i in todo], bits, group_size)
        for i, buffers in zip(todo, fresh):
            if cache is not None:
                cache.put(layers[i].weight, bits, group_size, buffers)
            out[i] = QuantizedLinear.from_buffers(layers[i], bits, group_size, *buffers)
    return out


def quantize_block(block, bits=8, group_size=32, cache=None):
    """The reference's per-block RTN loop (base_wrapper.py:289-315): returns a copy of `block`
    in which every nn.Linear is a QuantizedLinear of the given bits / group_size; `block` itself
    is left untouched."""
    quantized, taken = copy_without_linears(block)
    q_layers = quantized_linears([layer for _, layer in taken], bits, group_size, cache)
    if isinstance(quantized, _LinearPlaceholder):
        return q_layers[0]
    for (name, _), q_layer in zip(taken, q_layers):
        set_submodule(quantized, name, q_layer)
    replace_leftover_placeholders(quantized)
    return quantized


class BaseBlockWrapper(nn.Module):
    """Transparent wrapper around a block with pre/post forward hooks and an on/off switch
    (bitween/gradual/base_wrapper.py:10-119)."""

    def __init__(self, wrapped_block, storage_device="cpu", block_name=None):
        super().__init__()
        self.wrapped_block = wrapped_block
        self.storage_device = storage_device
        self.block_name = block_name or "unnamed_block"
        self.enabled = True
        self._original_device = next(wrapped_block.parameters()).device

    def forward(self, x, *args, **kwargs):
        if not self.enabled:
            return self.wrapped_block(x, *args, **kwargs)
        x = self._pre_forward_hook(x)
        output = self.wrapped_block(x, *args, **kwargs)
        return self._post_forward_hook(output)

    def _pre_forward_hook(self, x):
        return x

    def _post_forward_hook(self, output):
        return output

    def enable(self):
        self.enabled = True

    def disable(self):
        self.enabled = False

    def to_device(self, device):
        self.storage_device = device
        if device != "cpu":
            self.wrapped_block.to(device)

    def get_wrapped_block(self):
        return self.wrapped_block

    def __repr__(self):
        return f"{self.__class__.__name__}({self.block_name}, storage={self.storage_device}, enabled={self.enabled})"


class RTNWrapper(BaseBlockWrapper):
    """Applies RTN quantization to all linear layers of a block on the first forward pass, when
    the device is known (bitween/gradual/base_wrapper.py:242-370).  `cache` (extension): the
    RTNCache consulted for the block's (weight, bits, group_size) triples; the process-wide one
    by default, `False` for none."""

    def __init__(self, wrapped_block, bits=8, group_size=32, storage_device="cpu", block_name=None, cache=None):
        super().__init__(wrapped_block, storage_device, block_name)
        self.bits = bits
        self.group_size = group_size
        self.original_block = wrapped_block
        self.quantized_block = None
        self.quantization_applied = False
        self._cache = None if cache is False else (cache if cache is not None else default_cache())

    def _pre_forward_hook(self, x):
        if not self.quantization_applied:
            if next(self.original_block.parameters()).device != x.device:
                self.original_block = self.original_block.to(x.device)
            self._apply_rtn_quantization()
        return x

    def _apply_rtn_quantization(self):
        if self.quantization_applied:
            return
        self.quantized_block = quantize_block(self.original_block, self.bits, self.group_size, self._cache)
        self.wrapped_block = self.quantized_block
        self.quantization_applied = True

    def _remove_rtn_quantization(self):
        if not self.quantization_applied:
            return
        self.wrapped_block = self.original_block
        self.quantized_block = None
        self.quantization_applied = False

    def _set_submodule(self, parent_module, module_name, new_module):
        set_submodule(parent_module, module_name, new_module)

    def enable(self):
        super().enable()

    def disable(self):
        super().disable()
        self._remove_rtn_quantization()

    def cleanup(self):
        self._remove_rtn_quantization()

    def get_wrapped_block(self):
        return self.original_block
