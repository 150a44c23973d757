"""GPU parity at the full sizes of the benchmark configurations that the small-shape tests do
not reach: the prefill grid (Llama-3-8B shapes x {512, 2048, 8192} tokens x {W4 g128, W2 g64})
and the Llama-3-70B-shaped linears with their tensor-parallel shards (decode batch 64 and
prefill 4096 tokens), all through the C ABI.

Every case is checked three ways: all fp16 outputs against "dequantize (the bit-pinned kernel)
then matmul in fp32" on the same device (max|err| <= 1e-2 * RMS(output)); sampled weight rows
against the CPU oracle (same bar); and the fp32-accumulate outputs of sampled weight rows
against a float64 product of the same fp16 operands (max|err| <= 1e-5 * max|output| up to
K = 4096, growing in proportion to K beyond that: the tensor cores add each K = 16 block into
the fp32 accumulator with truncation, so a single accumulation chain over K inputs drifts by up
to ~K/16 half-ulps of the running sum -- measured 1.9e-5 at K = 14336 and 3.3e-5 at K = 28672,
the same for any fp16 GEMM with fp32 accumulation on this hardware, the reference's included).
"""
import pytest
import torch

from bitween_b200 import QuantizedLinear, dequantize_rtn, tp
from bitween_b200.functional import quantize_rtn_to_module_buffers
from bitween_b200.kernels import _lib
from bitween_b200.kernels.cuda_loader import quantized_matmul_cuda
from helpers import as_f32, assert_close_rms, oracle_forward

pytestmark = pytest.mark.gpu
DEV = "cuda"

LLAMA8B = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)]
LLAMA70B = [("q_o_proj", 8192, 8192), ("kv_proj", 1024, 8192), ("gate_up_proj", 28672, 8192),
            ("down_proj", 8192, 28672)]


def _layer(seed, N, K, bits, g):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    w = (torch.randn(N, K, device=DEV, generator=gen) * 0.02).to(torch.bfloat16)
    q, s_h, z_h = quantize_rtn_to_module_buffers(w, bits, g)
    del w
    return q, s_h, z_h, gen


def _sample_rows(N):
    return torch.tensor(sorted({0, 1, 127, 128, N // 2 + 3, N - 129, N - 1}))


def _check_acc_against_f64(x, acc, w_h, what):
    """fp32-accumulate output vs a float64 product of the same fp16-rounded operands, on sampled rows."""
    rows = torch.cat([_sample_rows(w_h.shape[0]), torch.arange(0, w_h.shape[0], max(1, w_h.shape[0] // 57))]).unique().to(acc.device)
    ref64 = x.half().double() @ w_h[rows].double().T
    bound = 1e-5 * max(1.0, x.shape[1] / 4096.0)
    err = float((acc[:, rows].double() - ref64).abs().max()) / float(ref64.abs().max())
    assert err <= bound, f"{what}: {err:.3g} > {bound:.3g}"


def _check_against_oracle_rows(x, y, q, s_h, z_h, bits, g, what, tokens=24):
    rows = _sample_rows(q.shape[0])
    tok = torch.linspace(0, x.shape[0] - 1, min(tokens, x.shape[0])).long()
    ref = oracle_forward(x[tok].cpu(), q[rows].cpu(), s_h[rows].cpu(), z_h[rows].cpu(), None, bits, g)
    assert_close_rms(as_f32(y[tok][:, rows.to(y.device)]), as_f32(ref), 1e-2, what)


@pytest.mark.parametrize("bits,g", [(4, 128), (2, 64)])
@pytest.mark.parametrize("shape", LLAMA8B, ids=lambda s: "%dx%d" % s)
def test_prefill_grid_full_size(shape, bits, g):
    N, K = shape
    q, s_h, z_h, gen = _layer(N + K + bits, N, K, bits, g)
    w_h = dequantize_rtn(q, s_h, z_h, g, bits=bits, out_dtype=torch.float16)
    for M in (512, 2048, 8192):
        x = torch.randn(M, K, device=DEV, generator=gen).to(torch.bfloat16)
        y = quantized_matmul_cuda(x, q, s_h, z_h, None, bits, g)
        assert _lib.lib().bw_device_status() == 0
        ref = x.half().float() @ w_h.float().T
        assert_close_rms(as_f32(y), as_f32(ref), 1e-2, f"{shape} M={M} W{bits}")
        _check_against_oracle_rows(x, y, q, s_h, z_h, bits, g, f"oracle rows {shape} M={M} W{bits}")
        acc = quantized_matmul_cuda(x.half(), q, s_h, z_h, None, bits, g, out_dtype=torch.float32)
        _check_acc_against_f64(x, acc, w_h, f"fp32 accumulate {shape} M={M} W{bits}")
        del x, y, ref, acc


def _sum_like_allreduce(parts):
    """Sum of the ranks' partial outputs in their own dtype, rank by rank: what a ring/tree
    all-reduce does up to the order (every hop rounds to the tensor's dtype)."""
    total = parts[0].clone()
    for p in parts[1:]:
        total += p
    return total


@pytest.mark.parametrize("M", [64, 4096])
@pytest.mark.parametrize("name,N,K", LLAMA70B, ids=[s[0] for s in LLAMA70B])
def test_llama70b_linears_and_their_tensor_parallel_shards(name, N, K, M):
    bits, g = 4, 128
    q, s_h, z_h, gen = _layer(N + K + M, N, K, bits, g)
    full = QuantizedLinear(K, N, bits, g, bias=False)
    full.qweight, full.scale, full.zero_point = q, s_h, z_h
    x = torch.randn(M, K, device=DEV, generator=gen).to(torch.bfloat16)
    w_h = dequantize_rtn(q, s_h, z_h, g, bits=bits, out_dtype=torch.float16)
    ref = x.half().float() @ w_h.float().T
    ref_rms_bound = 1e-2
    mode = "row" if name in ("down_proj",) else "column"
    modes = ["column", "row"] if name == "q_o_proj" else [mode]       # q is column-, o row-parallel
    for mode in modes:
        for world in (1, 2, 4, 8):
            outs16, outs32 = [], []
            for rank in range(world):
                sh = tp.shard_quantized_linear(full, mode, rank, world)
                xr = x if mode == "column" else x[:, rank * sh.in_features:(rank + 1) * sh.in_features].contiguous()
                outs16.append(quantized_matmul_cuda(xr, sh.qweight, sh.scale, sh.zero_point, None, bits, g))
                outs32.append(quantized_matmul_cuda(xr, sh.qweight, sh.scale, sh.zero_point, None, bits, g,
                                                    out_dtype=torch.float32))
                assert _lib.lib().bw_device_status() == 0
                del sh
            if mode == "column":
                y16, y32 = torch.cat(outs16, dim=1), torch.cat(outs32, dim=1)
            else:
                # fp16 partials summed in fp16 (what the NCCL all-reduce of the row-parallel layer
                # does); fp32 partials summed in fp32 for the accumulate check
                y16, y32 = _sum_like_allreduce(outs16), _sum_like_allreduce(outs32)
            what = f"{name} {mode} tp{world} M={M}"
            assert_close_rms(as_f32(y16), as_f32(ref), ref_rms_bound, what)
            _check_acc_against_f64(x, y32, w_h, "fp32 accumulate " + what)
            if world in (1, 8):
                _check_against_oracle_rows(x, y16, q, s_h, z_h, bits, g, "oracle rows " + what, tokens=8)
            del outs16, outs32, y16, y32
