"""bw_qmatmul_noalloc: the entry point for callers that cannot allocate device memory (code
inside a CUDA-graph capture, allocation-free serving loops, plugins that are only handed
buffers).  Its scratch is a fixed array inside the library instead of a caller workspace, so
the results must agree with those of the regular entry point -- also on a second call that
finds the first call's data still in the scratch -- and oversized requests must be refused.
(For up to 32 tokens the regular entry point may run the persistent decode kernel, which sums
in another order; there the bar is the suite's 16-bit tolerance plus bit-equality of the
no-allocation entry point with itself whatever the scratch held before.)

Collected last on purpose (file name), so a run that stops at the first failure has already
exercised every other test."""
import ctypes

import pytest
import torch

from bitween_b200 import synth
from bitween_b200.functional import quantize_rtn_to_module_buffers
from bitween_b200.kernels import _lib
from bitween_b200.kernels.cuda_loader import quantized_matmul_cuda, quantized_matmul_noalloc
from helpers import as_f32, assert_close_rms

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _layer(seed, N, K, bits, g):
    w = torch.from_numpy(synth.normal(seed, (N, K), 0.02)).to(DEV)
    return quantize_rtn_to_module_buffers(w, bits, g)


def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row():
    L = _lib.lib()
    assert L.bw_qmatmul_noalloc_max_scratch_bytes() == 2 << 20
    q, s, z = _layer(1, 320, 1024, 4, 128)
    bias = torch.from_numpy(synth.normal(2, (320,), 0.02)).half().to(DEV)
    # first call: 16 tokens; second call: 3 tokens of other data -> the scratch still holds the
    # first call's 16-token layout and must be fully rewritten, padding included
    first = {}
    for call, (M, seed, xdt) in enumerate(((16, 3, torch.float16), (3, 4, torch.bfloat16), (16, 3, torch.float16))):
        x = torch.from_numpy(synth.normal(seed, (M, 1024), 1.0)).to(xdt).to(DEV)
        ref = quantized_matmul_cuda(x, q, s, z, bias, 4, 128)
        out = torch.empty(M, 320, dtype=torch.float16, device=DEV)
        got = quantized_matmul_noalloc(x, q, s, z, bias, 4, 128, out)
        torch.cuda.synchronize()
        assert got.data_ptr() == out.data_ptr()
        # same inputs, same numerics contract: the 16-bit tolerance of the suite (1e-2 * RMS)
        assert_close_rms(as_f32(got), as_f32(ref), 1e-2, f"call {call}")
        # the third call repeats the first after the scratch held other data: identical bits
        if (M, seed) in first:
            assert torch.equal(got, first[(M, seed)]), f"call {call}"
        first[(M, seed)] = got.clone()
    # a different bit width and several 64-token blocks reuse the same scratch
    q8, s8, z8 = _layer(5, 96, 512, 8, 32)
    x = torch.from_numpy(synth.normal(6, (130, 512), 1.0)).half().to(DEV)
    ref = quantized_matmul_cuda(x, q8, s8, z8, None, 8, 32)
    out = torch.empty(130, 96, dtype=torch.float16, device=DEV)
    assert torch.equal(quantized_matmul_noalloc(x, q8, s8, z8, None, 8, 32, out), ref)


def test_noalloc_refuses_requests_beyond_its_scratch():
    L = _lib.lib()
    # 64 bf16 tokens x 32768: neither the GEMM's fp16 cast (4 MiB) nor the streaming kernel's
    # prepared activations (32768 * 64 * 2 B = 4 MiB) fit the 2 MiB array
    N, K, M = 8, 32768, 64
    q, s, z = _layer(7, N, K, 4, 128)
    x = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
    out = torch.full((M, N), 7.0, dtype=torch.float16, device=DEV)
    with pytest.raises(_lib.BitweenKernelError) as e:
        quantized_matmul_noalloc(x, q, s, z, None, 4, 128, out)
    assert e.value.status == 11 and "2 MiB" in str(e.value)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all()), "nothing may be launched for a refused request"
    # the same shape with few tokens fits
    x1 = torch.zeros(8, K, dtype=torch.float16, device=DEV)
    quantized_matmul_noalloc(x1, q, s, z, None, 4, 128, torch.empty(8, N, dtype=torch.float16, device=DEV))
    # fp16 activations on a 16-byte boundary need no scratch at all for more than 32 tokens
    quantized_matmul_noalloc(x.half(), q, s, z, None, 4, 128, torch.empty(M, N, dtype=torch.float16, device=DEV))
    # argument errors are reported like the regular entry point's
    assert L.bw_qmatmul_noalloc(None, 1, 4, 8, 64, None, None, None, None, None, 1, 3, 32, None) == 1
    with pytest.raises(ValueError):
        quantized_matmul_noalloc(x1[:, ::2], q, s, z, None, 4, 128, out)


@pytest.mark.parametrize("xdt", [torch.float16, torch.bfloat16])
def test_noalloc_many_tokens_long_rows(xdt):
    # 256 tokens x 8192: fp16 activations are read in place by the tensor-core GEMM (no scratch);
    # bf16 activations would need a 4 MiB cast, so blocks of 64 tokens stream through the 1 MiB
    # of prepared activations instead -- both must agree with the regular entry point
    q, s, z = _layer(11, 192, 8192, 4, 128)
    x = torch.from_numpy(synth.normal(12, (256, 8192), 1.0)).to(xdt).to(DEV)
    ref = quantized_matmul_cuda(x, q, s, z, None, 4, 128)
    out = torch.empty(256, 192, dtype=torch.float16, device=DEV)
    for _ in range(2):
        got = quantized_matmul_noalloc(x, q, s, z, None, 4, 128, out)
        torch.cuda.synchronize()
        assert_close_rms(as_f32(got), as_f32(ref), 1e-2, str(xdt))
    assert _lib.last_qmatmul_kernel() == ("qmm_tc_kernel" if xdt == torch.float16 else "qmm_smallm_kernel")
