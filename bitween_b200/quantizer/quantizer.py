"""`Bitween(model, ...).quantize(rtn=True)` -- the RTN per-layer loop of the reference
(bitween/quantizer/quantizer.py:11-118), with each layer quantized by the fused sm_100a kernel.

Only the RTN branch is part of this library.  Trainable quantization, calibration data and the
perplexity / KL evaluation of the reference are outside its scope: asking for them raises or
prints a notice instead of silently doing something else.
"""
import torch
import torch.nn as nn

from ..gradual.base_wrapper import copy_without_linears, quantized_linears, replace_leftover_placeholders
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
        """Returns a copy of the model with every non-ignored nn.Linear replaced by a
        QuantizedLinear (quantizer.py:67-84); the input model is left untouched.  As in the reference the branch is keyed on
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
            # Which layers are quantized is decided first, in module order and with the reference's
            # printed lines (quantizer.py:72-80); their weights are then NOT deep-copied with the
            # rest of the model (the reference copies the whole model, quantizer.py:69, and every
            # layer once more, modules.py:191) and all of them are quantized by one batched launch
            # per (device, dtype) instead of one launch per layer.
            state = {"index": 0}

            def keep_as_linear(name, layer):
                if name in self.ignore_layers:
                    print(f"  - Skipping ignored layer: {name}")
                    return True
                take = layer_filter is None or layer_filter(state["index"], name)
                state["index"] += 1
                if take:
                    print(f"  - Quantizing layer: {name}")
                return not take

            quantized_model, taken = copy_without_linears(self.model, skip=keep_as_linear)
            q_layers = quantized_linears([layer for _, layer in taken], self.bits, self.group_size)
            if taken and taken[0][0] == "":
                quantized_model = q_layers[0]        # the model is a single nn.Linear
            else:
                for (name, _), q_module in zip(taken, q_layers):
                    _set_module(quantized_model, name, q_module)
                replace_leftover_placeholders(quantized_model)
            print("--- Quantization complete ---")
            if evaluate_perplexity:
                print("bitween_b200: perplexity / KL evaluation is not part of this library; skipped")
        finally:
            self.ignore_layers = original_ignore_layers
        return quantized_model
