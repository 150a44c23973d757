"""Host-side mirror of the reference interface: argument rules, module state, the per-layer
loop and the drop-in aliasing -- everything that needs no GPU."""
import io
import pickle
from contextlib import redirect_stdout

import pytest
import torch
import torch.nn as nn

import bitween_b200
from bitween_b200 import Bitween, QuantizedLinear, quantize_rtn
from bitween_b200 import functional, modules
from helpers import to_np
from oracle import oracle


def test_quantize_rtn_argument_errors_match_reference():
    w = torch.zeros(4, 48)
    with pytest.raises(ValueError, match="Padding 16 columns"):
        quantize_rtn(w, bits=4, group_size=32)                 # functional.py:12-17
    with pytest.raises(AssertionError, match="Only 2, 4, or 8-bit"):
        quantize_rtn(w, bits=3, group_size=16)                 # functional.py:6
    with pytest.raises(RuntimeError):
        quantize_rtn(torch.zeros(4, 12), bits=4, group_size=4)  # 12 % 8 != 0: reference fails too


def test_no_cpu_fallback():
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError, match="no CPU path"):
        quantize_rtn(torch.zeros(4, 64), bits=4, group_size=32)
    layer = QuantizedLinear(64, 8, bits=4, group_size=32)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        layer(torch.zeros(2, 64))


def test_quantized_linear_state_matches_reference_layout():
    m = QuantizedLinear(768, 256, bits=4, group_size=128, bias=True, dtype=torch.bfloat16)
    sd = m.state_dict()
    assert list(sd) == ["qweight", "scale", "zero_point", "bias"]
    assert sd["qweight"].dtype == torch.int32 and tuple(sd["qweight"].shape) == (256, 96)
    assert sd["scale"].dtype == torch.float16 and tuple(sd["scale"].shape) == (256, 6)
    assert sd["zero_point"].dtype == torch.float16 and tuple(sd["zero_point"].shape) == (256, 6)
    assert sd["bias"].dtype == torch.float16 and tuple(sd["bias"].shape) == (256,)
    assert m.dtype == torch.float16                          # dtype arg is ignored (modules.py:167)
    assert (m.in_features, m.out_features, m.bits, m.group_size, m.requires_grad) == (768, 256, 4, 128, False)
    assert repr(m) == "QuantizedLinear(in_features=768, out_features=256, bias=True, bits=4, group_size=128)"
    nb = QuantizedLinear(64, 8, bits=2, group_size=32, bias=False)
    assert nb.bias is None and "bias" not in nb.state_dict()
    assert tuple(nb.qweight.shape) == (8, 4)
    with pytest.raises(ValueError, match="Only 2, 4, or 8 bits"):
        QuantizedLinear(64, 8, bits=3)
    with pytest.raises(ValueError, match="Group size"):
        QuantizedLinear(64, 8, bits=4, group_size=0)


def test_pickle_round_trip_and_bitween_alias():
    m = QuantizedLinear(64, 8, bits=8, group_size=32)
    m.qweight.fill_(7)
    m2 = pickle.loads(pickle.dumps(m))
    assert torch.equal(m2.qweight, m.qweight) and m2.bits == 8 and m2.group_size == 32
    me = bitween_b200.install_as_bitween()
    import bitween
    import bitween.modules
    from bitween.kernels.cuda_loader import quantized_matmul_cuda  # noqa: F401  (main.py:401)
    from bitween.functional import quantize_rtn as q2, dequantize_rtn  # noqa: F401
    assert bitween is me and bitween.modules.QuantizedLinear is QuantizedLinear and q2 is quantize_rtn


def _oracle_many(weights, bits, group_size):
    """quantize_rtn_many_to_module_buffers with the oracle doing the arithmetic (test double for
    the batched CUDA call): fp32 arithmetic, fp16 scale / zero-point buffers."""
    out = []
    for w in weights:
        q, s, z = oracle.quantize_rtn(to_np(w.float()), oracle.F32, bits, group_size)
        out.append((torch.from_numpy(q), torch.from_numpy(s).half(), torch.from_numpy(z).half()))
    return out


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(64, 128)
        self.fc2 = nn.Linear(128, 64, bias=False)


class _Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed_tokens = nn.Embedding(10, 64)
        self.layers = nn.ModuleList([_Block(), _Block()])
        self.lm_head = nn.Linear(64, 10, bias=False)


def test_bitween_rtn_loop_replaces_linears(monkeypatch):
    from bitween_b200.gradual import base_wrapper
    monkeypatch.setattr(base_wrapper, "quantize_rtn_many_to_module_buffers", _oracle_many)
    model = _Tiny()
    buf = io.StringIO()
    with redirect_stdout(buf):
        qm = Bitween(model, bits=4, group_size=32).quantize(rtn=True, ignore_layers=["lm_head"])
    out = buf.getvalue()
    assert "  - Quantizing layer: layers.0.fc1" in out and "  - Skipping ignored layer: lm_head" in out
    assert "--- Quantization complete ---" in out
    assert isinstance(qm.layers[0].fc1, QuantizedLinear) and isinstance(qm.layers[1].fc2, QuantizedLinear)
    assert isinstance(qm.lm_head, nn.Linear)
    assert isinstance(model.layers[0].fc1, nn.Linear), "the original model must stay untouched"
    assert qm.layers[1].fc2.bias is None and qm.layers[0].fc1.bias.dtype == torch.float16
    assert tuple(qm.layers[0].fc1.qweight.shape) == (128, 8)
    # layer_filter keeps only every second layer (multi-GPU layer sharding hook)
    with redirect_stdout(io.StringIO()):
        half = Bitween(model, bits=4, group_size=32).quantize(
            rtn=True, ignore_layers=["lm_head"], layer_filter=lambda i, name: i % 2 == 0)
    kinds = [type(m).__name__ for m in (half.layers[0].fc1, half.layers[0].fc2, half.layers[1].fc1, half.layers[1].fc2)]
    assert kinds == ["QuantizedLinear", "Linear", "QuantizedLinear", "Linear"]
    # the weights that get quantized are not copied on the way; everything else is
    assert qm.embed_tokens.weight.data_ptr() != model.embed_tokens.weight.data_ptr()
    assert qm.lm_head.weight.data_ptr() != model.lm_head.weight.data_ptr()
    with pytest.raises(NotImplementedError):
        Bitween(model).quantize(trainable=True)
    with pytest.raises(AssertionError):
        Bitween(model, group_size=0)


def test_qmatmul_wrapper_validates_before_crossing_abi():
    from bitween_b200.kernels.cuda_loader import quantized_matmul_cuda
    x = torch.zeros(2, 64, dtype=torch.float16)
    with pytest.raises(ValueError):
        quantized_matmul_cuda(x, torch.zeros(8, 8, dtype=torch.int32), None, None, None, 3, 32)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        quantized_matmul_cuda(x, torch.zeros(8, 8, dtype=torch.int32), torch.zeros(8, 2), torch.zeros(8, 2),
                              None, 4, 32)
    assert functional.quantize_rtn is quantize_rtn and modules.QuantizedLinear is QuantizedLinear


def test_rtn_wrapper_quantizes_a_block_once_per_config_and_restores_it(monkeypatch):
    """The per-block RTN loop of the gradual flow (reference bitween/gradual/base_wrapper.py:
    242-370): first forward quantizes a copy of the block, disable() restores the original, and
    a repeated (bits, group_size) trial on unchanged weights is served from the cache."""
    from bitween_b200.gradual import RTNCache, RTNWrapper, base_wrapper, quantize_block
    calls = []

    def counting(weights, bits, group_size):
        calls.append(len(weights))
        return _oracle_many(weights, bits, group_size)

    monkeypatch.setattr(base_wrapper, "quantize_rtn_many_to_module_buffers", counting)

    class _Fwd(_Block):
        def forward(self, x):
            return x                                     # the wrapped block's own forward is not under test

    block = _Fwd()
    cache = RTNCache()
    wrap = RTNWrapper(block, bits=4, group_size=32, block_name="layers.0", cache=cache)
    assert (wrap.bits, wrap.group_size, wrap.quantization_applied, wrap.quantized_block) == (4, 32, False, None)
    x = torch.zeros(1, 64)
    wrap(x)
    assert wrap.quantization_applied and calls == [2], "both linears of the block in ONE batched call"
    assert isinstance(wrap.wrapped_block.fc1, QuantizedLinear) and isinstance(block.fc1, nn.Linear)
    assert wrap.get_wrapped_block() is block
    assert repr(wrap) == "RTNWrapper(layers.0, storage=cpu, enabled=True)"
    wrap.disable()
    assert wrap.wrapped_block is block and not wrap.quantization_applied and not wrap.enabled
    # the same trial again: no kernel work, same buffers
    first = quantize_block(block, 4, 32, cache)
    again = quantize_block(block, 4, 32, cache)
    assert calls == [2] and cache.hits >= 4
    assert again.fc1.qweight.data_ptr() == first.fc1.qweight.data_ptr()
    # another group size, or a modified weight, is a new entry
    quantize_block(block, 4, 64, cache)
    with torch.no_grad():
        block.fc1.weight.add_(1.0)
    quantize_block(block, 4, 32, cache)
    assert calls == [2, 2, 1]
    # a tiny cache evicts the oldest entries instead of growing
    small = RTNCache(max_bytes=1)
    quantize_block(block, 8, 32, small)
    assert len(small) == 1


def test_wrapper_linear_host_logic_with_oracle_doubles(monkeypatch):
    """WrapperLinear's bookkeeping (buffers, parameters, wrap / unwrap, best-parameter tracking)
    with the two CUDA calls replaced by the oracle: no GPU needed."""
    import numpy as np
    from bitween_b200 import wrapper

    def rtn_double(weight, bits=8, group_size=32):
        q, s, z = oracle.quantize_rtn(to_np(weight.float()), oracle.F32, bits, group_size)
        return torch.from_numpy(q), torch.from_numpy(s), torch.from_numpy(z), weight.shape

    def fq_double(weight, scale, zero_point, value, bits, group_size, want_q=True):
        dq, q = oracle.wrapper_fake_quant(weight.detach().float().numpy(), scale.detach().numpy(),
                                          zero_point.detach().numpy(),
                                          None if value is None else value.detach().float().numpy(), bits, group_size)
        return torch.from_numpy(dq), torch.from_numpy(q)

    monkeypatch.setattr(wrapper, "quantize_rtn", rtn_double)
    monkeypatch.setattr(wrapper, "fake_quantize", fq_double)
    torch.manual_seed(0)
    block = nn.Sequential(nn.Linear(64, 32), nn.ReLU(), nn.Linear(32, 64, bias=False))
    buf = io.StringIO()
    with redirect_stdout(buf):
        _, names = wrapper.unified_wrapper(block, bits=4, group_size=32, ignore_layers={"blk.2"}, module_prefix="blk")
    assert names == ["0"] and "Skipping ignored layer: blk.2" in buf.getvalue()
    wl = block[0]
    assert isinstance(wl, wrapper.WrapperLinear) and isinstance(block[2], nn.Linear)
    assert list(wl.state_dict()) == ["value", "min_scale", "max_scale", "orig_weight", "orig_bias", "base_qweight",
                                     "base_scale", "base_zero_point", "orig_layer.weight", "orig_layer.bias"]
    assert tuple(wl.min_scale.shape) == (32, 2) and wl.value.shape == wl.orig_weight.shape
    w_dq, w_q, scale, zp = wl._quantize_weight_with_learnable_params()
    assert tuple(w_q.shape) == (32, 2, 32) and tuple(scale.shape) == (32, 2)
    # untouched parameters: fake quantization is plain RTN with a float zero point
    assert float((w_dq - wl.orig_weight).abs().max()) <= float(scale.detach().max()) * 0.5 + 1e-7
    assert block(torch.randn(3, 64)).shape == (3, 64)
    off = wrapper.WrapperLinear(nn.Linear(64, 8), bits=2, group_size=64, enable_minmax_tuning=False,
                                enable_round_tuning=False)
    assert off.value is None and off.min_scale is None and off.max_scale is None
    assert list(off.state_dict())[:2] == ["orig_weight", "orig_bias"]
    wl.update_best_params(3.0)
    with torch.no_grad():
        wl.value.add_(0.25)
    wl.update_best_params(5.0)
    assert wl.best_loss == 3.0 and float(wl.best_params["value"].abs().max()) == 0.0
    q, un = wrapper.wrapper_block(nn.Sequential(nn.Linear(32, 32)), bits=8, group_size=32)
    assert q == ["0"] and "" in un
    ql = wrapper.unified_unwrapper(wl, apply_quantization=True)
    assert isinstance(ql, QuantizedLinear) and float(wl.value.abs().max()) == 0.0    # best parameters applied
    want_q, want_s, want_z = oracle.quantize_rtn(to_np(wl.orig_weight), oracle.F32, 4, 32)
    assert np.array_equal(to_np(ql.qweight), want_q)
    assert wrapper.unified_unwrapper(wl, apply_quantization=False) is wl.orig_layer
