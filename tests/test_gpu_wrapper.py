"""WrapperLinear (trainable mode) on the GPU: the fused fake-quantization kernels against outputs
of the reference class itself (tests/golden/wrapper_small.npz), against the numpy oracle on
larger seeded inputs, and against the reference's sequence of torch ops at full layer size."""
import json
import os

import numpy as np
import pytest
import torch

from bitween_b200 import QuantizedLinear, synth
from bitween_b200.kernels import _lib
from bitween_b200.wrapper import (WrapperLinear, fake_quantize, unified_unwrapper, unified_wrapper,
                                  wrap_model_for_training)
from helpers import from_bits, to_np
from oracle import oracle
from test_oracle_wrapper import same_numbers

pytestmark = pytest.mark.gpu
DEV = "cuda"
TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "float32": torch.float32,
       "float16": torch.float16, "bfloat16": torch.bfloat16}


def _t(gold, key, dt):
    a = gold[key]
    return torch.from_numpy(a.copy()) if a.dtype == np.float32 else from_bits(a, TDT[dt])


def _build(gold, c):
    n = c["name"]
    N, K = c["shape"]
    layer = torch.nn.Linear(K, N, bias=True)
    layer.weight.data = _t(gold, n + "/w", c["dtype"])
    layer.bias.data = _t(gold, n + "/bias", c["dtype"])
    layer = layer.to(DEV)
    wl = WrapperLinear(layer, bits=c["bits"], group_size=c["g"], enable_minmax_tuning=c["minmax"],
                       enable_round_tuning=c["round"])
    with torch.no_grad():
        if c["minmax"]:
            wl.min_scale.copy_(torch.from_numpy(gold[n + "/min_scale"]))
            wl.max_scale.copy_(torch.from_numpy(gold[n + "/max_scale"]))
        if c["round"]:
            wl.value.copy_(_t(gold, n + "/value", c["value_dtype"]))
    return wl


def test_wrapper_matches_reference_class_outputs(golden_dir):
    with open(os.path.join(golden_dir, "wrapper_meta.json")) as f:
        cases = json.load(f)["cases"]
    gold = np.load(os.path.join(golden_dir, "wrapper_small.npz"))
    grads = 0
    for c in cases:
        n = c["name"]
        wl = _build(gold, c)
        assert wl.orig_weight.is_cuda and (wl.value is None or wl.value.dtype == TDT[c["value_dtype"]])
        w_dq, w_q, scale, zp = wl._quantize_weight_with_learnable_params()
        N, K = c["shape"]
        assert tuple(w_q.shape) == (N, K // c["g"], c["g"]) and tuple(w_dq.shape) == (N, K)
        if c["out_dtype"] != "float32":
            # every tensor 16-bit (min/max tuning off): the kernel that rounds after each operation
            dt16 = TDT[c["dtype"]]
            assert w_dq.dtype == dt16 and w_q.dtype == dt16 and scale.dtype == dt16
            f = lambda key: _t(gold, n + key, c["dtype"]).float().numpy()   # noqa: E731
            assert same_numbers(scale.float().cpu().numpy(), f("/scale")), n
            assert same_numbers(zp.float().cpu().numpy(), f("/zp")), n
            assert same_numbers(w_q.float().cpu().numpy().reshape(N, K), f("/w_q")), n
            assert same_numbers(w_dq.float().cpu().numpy(), f("/w_dq")), n
        else:
            assert w_dq.dtype == torch.float32
            assert np.array_equal(to_np(scale).view(np.uint32), gold[n + "/scale"].view(np.uint32)), n
            assert np.array_equal(to_np(zp).view(np.uint32), gold[n + "/zp"].view(np.uint32)), n
            assert same_numbers(to_np(w_q).reshape(N, K), gold[n + "/w_q"]), n
            assert same_numbers(to_np(w_dq), gold[n + "/w_dq"]), n
        if n + "/grad_min_scale" in gold.files:
            r = torch.from_numpy(gold[n + "/r"]).to(DEV)
            (w_dq * r).sum().backward()
            for name in ("min_scale", "max_scale"):
                want = gold[f"{n}/grad_{name}"].astype(np.float64)
                got = getattr(wl, name).grad.double().cpu().numpy()
                # same graph, other summation order: fp32 sums of <= 256 terms
                assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max()), (n, name)
            assert wl.value is None or wl.value.grad is None
            grads += 1
        # forward = F.linear with the fake-quantized weight (bitween/wrapper.py:174-181)
        # (fp32 layers only: with a 16-bit bias beside the fp32 w_dq F.linear refuses in the reference too)
        if c["dtype"] == "f32":
            x = torch.from_numpy(synth.normal(5, (3, K), 1.0)).to(DEV)
            y = wl(x)
            want_y = torch.nn.functional.linear(x, torch.from_numpy(gold[n + "/w_dq"]).to(DEV), wl.orig_bias)
            assert torch.allclose(y, want_y, rtol=1e-5, atol=1e-6), n
        ql = wl.to_quantized_linear()
        assert isinstance(ql, QuantizedLinear)
        assert np.array_equal(to_np(ql.qweight), gold[n + "/ql_qweight"]), n
        assert np.array_equal(to_np(ql.scale), gold[n + "/ql_scale"]), n
        assert np.array_equal(to_np(ql.zero_point), gold[n + "/ql_zp"]), n
    assert grads >= 30 and _lib.lib().bw_device_status() == 0


@pytest.mark.parametrize("dt,bits,g", [(torch.float16, 4, 128), (torch.bfloat16, 2, 64), (torch.float32, 8, 32),
                                       (torch.float16, 4, 24)])
def test_fake_quant_kernels_vs_oracle(dt, bits, g):
    N, K = 384, 3072
    w = torch.from_numpy(synth.normal(11, (N, K), 0.02)).to(dt)
    value = torch.from_numpy(synth.uniform(12, (N, K), -0.5, 0.5)).to(dt)
    mn = synth.uniform(13, (N, K // g), 0.9, 1.1)
    mx = synth.uniform(14, (N, K // g), 0.9, 1.1)
    w32 = w.float().numpy()
    scale, zp = oracle.wrapper_group_params(w32, bits, g, mn, mx)
    dq_ref, q_ref = oracle.wrapper_fake_quant(w32, scale, zp, value.float().numpy(), bits, g)
    s_d = torch.from_numpy(scale).to(DEV).requires_grad_()
    z_d = torch.from_numpy(zp).to(DEV).requires_grad_()
    dq, q = fake_quantize(w.to(DEV), s_d, z_d, value.to(DEV), bits, g)
    assert same_numbers(to_np(q), q_ref) and same_numbers(to_np(dq), dq_ref)
    grad = synth.normal(15, (N, K), 1.0)
    dq.backward(torch.from_numpy(grad).to(DEV))
    gs_ref, gz_ref = oracle.wrapper_param_grads(w32, scale, zp, value.float().numpy(), grad, bits, g)
    # fp32 sums of g terms against float64
    for got, want in ((s_d.grad, gs_ref), (z_d.grad, gz_ref)):
        err = np.abs(got.double().cpu().numpy() - want).max()
        assert err <= 1e-5 * np.sqrt(g) * max(1.0, np.abs(want).max()), (err, np.abs(want).max())
    # without the perturbation and without w_q
    dq2, q2 = fake_quantize(w.to(DEV), s_d.detach(), z_d.detach(), None, bits, g, want_q=False)
    assert q2.numel() == 0
    assert same_numbers(to_np(dq2), oracle.wrapper_fake_quant(w32, scale, zp, None, bits, g)[0])


def _torch_ops_restatement(wl):
    """The reference's own op sequence (bitween/wrapper.py:116-172) with torch ops on the GPU."""
    weight = wl.orig_weight
    N, K = weight.shape
    G = K // wl.group_size
    wg = weight.view(N, G, wl.group_size)
    max_val = (1 << wl.bits) - 1
    w_min = wg.min(dim=-1, keepdim=True)[0] * wl.min_scale.unsqueeze(-1)
    w_max = wg.max(dim=-1, keepdim=True)[0] * wl.max_scale.unsqueeze(-1)
    # (a tensor divisor: division by a Python scalar is a reciprocal multiplication on CUDA, not the
    # correctly rounded quotient of the CPU run)
    scale = torch.clamp((w_max - w_min) / torch.full((), max_val, dtype=torch.float32, device=DEV), min=1e-8)
    zero_point = -w_min / scale
    t = wg / scale + zero_point + wl.value.view(N, G, wl.group_size)
    wq = torch.clamp(torch.round(t), 0, max_val)
    return (scale * (wq - zero_point)).view(N, K), wq


def test_full_size_layer_equals_torch_op_sequence_and_trains():
    # Llama-3-8B gate/up projection shape, bf16 checkpoint weights, W4 g128
    N, K, bits, g = 14336, 4096, 4, 128
    torch.manual_seed(0)
    layer = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16, device=DEV)
    with torch.no_grad():
        layer.weight.normal_(0, 0.02)
    wl = WrapperLinear(layer, bits=bits, group_size=g)
    with torch.no_grad():
        wl.min_scale.uniform_(0.9, 1.1)
        wl.max_scale.uniform_(0.9, 1.1)
        wl.value.uniform_(-0.5, 0.5)
    w_dq, w_q, scale, zp = wl._quantize_weight_with_learnable_params()
    ref_dq, ref_q = _torch_ops_restatement(wl)
    assert torch.equal(w_q, ref_q) and torch.equal(w_dq, ref_dq)     # == treats -0.0 and 0.0 alike
    assert float(w_q.min()) >= 0 and float(w_q.max()) <= 15
    # gradients of the factors against autograd through the torch op sequence
    r = torch.randn(N, K, device=DEV)
    (w_dq * r).sum().backward()
    got = wl.min_scale.grad.clone(), wl.max_scale.grad.clone()
    wl.min_scale.grad = wl.max_scale.grad = None
    (ref_dq * r).sum().backward()
    for a, b in zip(got, (wl.min_scale.grad, wl.max_scale.grad)):
        assert float((a - b).abs().max()) <= 1e-4 * max(1.0, float(b.abs().max()))
    del r, ref_dq, ref_q, w_dq, w_q
    # a few signed-gradient steps on the factors lower the output error against the float layer
    x = torch.randn(64, K, device=DEV)
    with torch.no_grad():
        target = torch.nn.functional.linear(x, layer.weight.float())
    with torch.no_grad():
        wl.min_scale.fill_(1.0)
        wl.max_scale.fill_(1.0)
        wl.value.zero_()
    losses = []
    for _ in range(6):
        for p in (wl.min_scale, wl.max_scale):
            p.grad = None
        loss = torch.nn.functional.mse_loss(wl(x), target)
        loss.backward()
        losses.append(float(loss.detach()))
        with torch.no_grad():
            wl.min_scale -= 2e-3 * wl.min_scale.grad.sign()
            wl.max_scale -= 2e-3 * wl.max_scale.grad.sign()
    assert losses[-1] < losses[0]
    assert _lib.lib().bw_device_status() == 0


class _Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = torch.nn.Linear(64, 128)
        self.fc2 = torch.nn.Linear(128, 64)
        self.norm = torch.nn.LayerNorm(64)

    def forward(self, x):
        return self.norm(self.fc2(torch.relu(self.fc1(x))))


def test_wrap_train_unwrap_block():
    torch.manual_seed(1)
    model = torch.nn.ModuleDict({"blk": _Block(), "head": torch.nn.Linear(64, 10)}).to(DEV)
    info = wrap_model_for_training(model, ["blk", "head"], True, 4, 32, {"blk.fc2"})
    assert info["blk"]["quantized_names"] == ["fc1"] and not info["blk"]["is_single_layer"]
    assert info["head"]["is_single_layer"] and isinstance(info["head"]["wrapped_module"], WrapperLinear)
    assert isinstance(model["blk"].fc1, WrapperLinear) and isinstance(model["blk"].fc2, torch.nn.Linear)
    again, names = unified_wrapper(model["blk"].fc1)
    assert names == [] and again is model["blk"].fc1
    y = model["blk"](torch.randn(5, 64, device=DEV))
    assert y.shape == (5, 64)
    sd = model["blk"].fc1.state_dict()
    assert {"orig_weight", "orig_bias", "base_qweight", "base_scale", "base_zero_point", "value", "min_scale",
            "max_scale", "orig_layer.weight", "orig_layer.bias"} == set(sd)
    wl = model["blk"].fc1
    wl.update_best_params(1.0)
    with torch.no_grad():
        wl.min_scale.mul_(0.5)
    wl.update_best_params(2.0)          # worse: not recorded
    wl.apply_best_params()
    assert float(wl.min_scale.detach().min()) == 1.0
    unified_unwrapper(model["blk"], apply_quantization=True)
    assert isinstance(model["blk"].fc1, QuantizedLinear)
    restored = unified_unwrapper(info["head"]["wrapped_module"], apply_quantization=False)
    assert restored is info["head"]["original_module"]
