"""`Bitween(model, ...).quantize(rtn=True)` -- the RTN per-layer loop of the reference
(bitween/quantizer/quantizer.py:11-118), with each layer quantized by the fused sm_100a kernel.

Only the RTN branch is part of this library.  Trainable quantization, calibration data and the
perplexity / KL evaluation of the reference are outside its scope: asking for them raises or
prints a notice instead of silently doing something else.
"""
import copy

import torch
import torch.nn as nn

from ..modules import QuantizedLinear
from .func import _set_module


class Bitween:
    """Same constructor and `quantize` signature as the reference class (quantizer.py:15-39)."""

    def __init__(self, model, tokenizer=None, bits=8, group_size=32, iters=1, lr=0.005,
                 enable_minmax_tuning=True, seqlen=2048, cache_to_disk=False, max_memory_mb=512,
                 ignore_layers=None, batch_size=32):
        self.model = model
        self.tokenizer = tokenizer
        self.bits = bits
        self.group_size = group_size
        self.iters = iters
        self.lr = lr
        self.enable_minmax_tuning = enable_minmax_tuning
        self.seqlen = seqlen
        self.cache_to_disk = cache_to_disk
        self.max_memory_mb = max_memory_mb
        self.ignore_layers = set(ignore_layers) if ignore_layers else set()
        self.batch_size = batch_size
        assert group_size > 0, "Group size must be greater than 0."

    def quantize(self, evaluate_perplexity=False, eval_samples=100, rtn=False, trainable=False,
                 calib_dataset="pile-10k", nsamples=None, cache_to_disk=None, max_memory_mb=None,
                 ignore_layers=None, batch_size=None, layer_filter=None, **eval_kwargs):
        """Returns a deep copy of the model with every non-ignored nn.Linear replaced by a
        QuantizedLinear (quantizer.py:67-84).  As in the reference the branch is keyed on
        `trainable`; `rtn` is accepted for signature compatibility.

        `layer_filter` (extension): optional callable `(index, name) -> bool`; layers it rejects
        are left as nn.Linear.  `bitween_b200.tp.layer_shard_filter(rank, world)` uses it to
        spread the layers of one model over several GPUs with no communication.
        """
        if trainable:
            raise NotImplementedError(
                "bitween_b200 implements the RTN path only; trainable quantization "
                "(reference quantizer.py:86-97,120-291) is outside this library")
        original_ignore_layers = self.ignore_layers
        if ignore_layers is not None:
            self.ignore_layers = set(ignore_layers)
        if batch_size is not None:
            self.batch_size = batch_size
        try:
            quantized_model = copy.deepcopy(self.model)
            index = 0
            for name, module in list(quantized_model.named_modules()):
                if not isinstance(module, nn.Linear):
                    continue
                if name in self.ignore_layers:
                    print(f"  - Skipping ignored layer: {name}")
                    continue
                take = layer_filter is None or layer_filter(index, name)
                index += 1
                if not take:
                    continue
                print(f"  - Quantizing layer: {name}")
                q_module = QuantizedLinear.from_float(module, self.bits, self.group_size)
                _set_module(quantized_model, name, q_module)
            print("--- Quantization complete ---")
            if evaluate_perplexity:
                print("bitween_b200: perplexity / KL evaluation is not part of this library; skipped")
        finally:
            self.ignore_layers = original_ignore_layers
        return quantized_model
