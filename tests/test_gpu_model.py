"""Mixed-precision model forward: a random-init 12-layer OPT-style decoder (d=768, 12 heads, FFN
3072, vocab 50272, learned positions, LayerNorm, ReLU) whose 72 decoder linears get bits in
{8,4,2} and group sizes in {32,64,128} by seed, as the reference's gradual quantizer would assign
them (gradual/base_wrapper.py:289-315), batch 8 x 512 random token ids.

The logits of the model running this library's fused kernels are compared with the same model
where every QuantizedLinear computes what the reference forward computes, step by step
(bitween/modules.py:85-101): dequantize to fp16 [N,K] (bit-exact kernel), matmul, bias add.
A sample of layers is also checked against the CPU oracle on the real activations.
Synthetic weights and token ids stand in for the OPT-125m checkpoint and its datasets."""
import numpy as np
import pytest
import torch

from bitween_b200 import Bitween, QuantizedLinear, dequantize_rtn
from bitween_b200.kernels import _lib
from helpers import as_f32, assert_close_rms, oracle_forward, rms

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _build_model():
    transformers = pytest.importorskip("transformers")
    cfg = transformers.OPTConfig(vocab_size=50272, hidden_size=768, num_hidden_layers=12, num_attention_heads=12,
                                 ffn_dim=3072, max_position_embeddings=2048, activation_function="relu",
                                 word_embed_proj_dim=768, do_layer_norm_before=True)
    torch.manual_seed(1234)
    return transformers.OPTForCausalLM(cfg).eval()


def _reference_style_forward(self, x):
    # what bitween/modules.py:85-101 does: fp16 weights in HBM, library matmul, separate bias add
    w = dequantize_rtn(self.qweight, self.scale, self.zero_point, self.group_size, bits=self.bits,
                       out_dtype=torch.float16)
    c = torch.matmul(x.to(torch.float16), w.T)
    return c + self.bias if self.bias is not None else c


def test_mixed_precision_opt_style_model_logits():
    model = _build_model().half().to(DEV)
    names = [n for n, m in model.named_modules() if isinstance(m, torch.nn.Linear) and n != "lm_head"]
    assert len(names) == 72
    rng = np.random.RandomState(7)
    qmodel = model
    captured = {}
    # The gradual flow assigns a configuration to the attention and to the MLP linears of every
    # block (precision_optimizer.py separates them) and quantizes them through the per-block RTN
    # loop: here `quantize_block` / `quantized_linears`, one batched launch per group of layers.
    from bitween_b200.gradual import RTNCache, quantize_block
    from bitween_b200.gradual.base_wrapper import quantized_linears
    cache = RTNCache()
    for block in qmodel.model.decoder.layers:
        bits, g = int(rng.choice([8, 4, 2])), int(rng.choice([32, 64, 128]))
        float_q = block.self_attn.q_proj
        block.self_attn = quantize_block(block.self_attn, bits, g, cache)
        # the batched call gives the bits of the one-layer-at-a-time call
        single = QuantizedLinear.from_float(float_q, bits=bits, group_size=g)
        assert torch.equal(single.qweight, block.self_attn.q_proj.qweight)
        assert torch.equal(single.scale, block.self_attn.q_proj.scale)
        assert torch.equal(single.zero_point, block.self_attn.q_proj.zero_point)
        assert torch.equal(single.bias, block.self_attn.q_proj.bias)
        bits, g = int(rng.choice([8, 4, 2])), int(rng.choice([32, 64, 128]))
        block.fc1, block.fc2 = quantized_linears([block.fc1, block.fc2], bits, g, cache)
    assert len(cache) == 72 and cache.hits == 0
    qlayers = {n: m for n, m in qmodel.named_modules() if isinstance(m, QuantizedLinear)}
    assert len(qlayers) == 72 and {m.bits for m in qlayers.values()} == {2, 4, 8}

    gen = torch.Generator().manual_seed(99)
    ids = torch.randint(0, 50272, (8, 512), generator=gen).to(DEV)
    sample = names[::12]
    hooks = [qlayers[n].register_forward_hook(
        lambda mod, inp, out, n=n: captured.__setitem__(n, (inp[0].detach()[0, :24].clone(), out.detach()[0, :24].clone())))
        for n in sample]
    with torch.no_grad():
        logits = qmodel(ids).logits
    for h in hooks:
        h.remove()
    assert _lib.lib().bw_device_status() == 0
    assert torch.isfinite(logits).all()

    orig = QuantizedLinear.forward
    try:
        QuantizedLinear.forward = _reference_style_forward
        with torch.no_grad():
            ref_logits = qmodel(ids).logits
    finally:
        QuantizedLinear.forward = orig
    got, ref = as_f32(logits), as_f32(ref_logits)
    # 24 quantized matmuls deep, fp16 everywhere else: 1e-2 * RMS on the logits
    assert_close_rms(got, ref, 1e-2, "logits")
    assert float(np.mean(got.argmax(-1) == ref.argmax(-1))) > 0.99

    # real activations of a few layers against the CPU oracle (first 24 tokens of sequence 0)
    for n in sample:
        m = qlayers[n]
        x, y = captured[n]
        want = oracle_forward(x.cpu(), m.qweight.cpu(), m.scale.cpu(), m.zero_point.cpu(),
                              None if m.bias is None else m.bias.cpu(), m.bits, m.group_size)
        assert_close_rms(as_f32(y), as_f32(want), 1e-2, n)


def test_bitween_quantize_whole_model_on_gpu():
    model = _build_model().to(DEV)      # fp32 layers, as the reference's test loads them
    import contextlib
    import io
    with contextlib.redirect_stdout(io.StringIO()) as buf:
        q = Bitween(model, bits=4, group_size=64).quantize(rtn=True, ignore_layers=["lm_head"])
    assert buf.getvalue().count("Quantizing layer") == 72 and "Skipping ignored layer: lm_head" in buf.getvalue()
    n_q = sum(isinstance(m, QuantizedLinear) for m in q.modules())
    assert n_q == 72 and isinstance(q.lm_head, torch.nn.Linear)
    ids = torch.randint(0, 50272, (2, 64), generator=torch.Generator().manual_seed(3)).to(DEV)
    with torch.no_grad():
        a = q(ids).logits.float()
        b = model(ids).logits.float()
    # 4-bit RTN of a random-init model: logits stay close to the float model's
    assert torch.isfinite(a).all()
    assert rms(as_f32(a - b)) < 0.5 * rms(as_f32(b))
