"""The C-ABI library loads and exports every symbol include/bitween_b200.h declares.
No compute call is made here, so this runs without a GPU."""
import ctypes
import os
import re

from bitween_b200.kernels import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "bitween_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"BW_API[^;(]*?\b(bw_[a-z_0-9]+)\s*\(", text)


def test_every_declared_symbol_is_exported():
    names = declared_symbols()
    assert len(names) >= 10 and "bw_qmatmul" in names and "bw_rtn_quantize_pack" in names
    L = _lib.lib()
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in the header but not exported"
    assert L.bw_version() >= 100


def test_status_strings_and_argument_validation_need_no_gpu():
    L = _lib.lib()
    assert L.bw_status_string(0) == b"ok"
    # validation happens before any CUDA call: bad bits, bad group, bad K, NULL pointers
    z = None
    assert L.bw_rtn_quantize_pack(z, 0, 4, 64, 3, 32, z, z, 0, z, 3, 0, z) == 1     # BW_ERR_BITS
    assert L.bw_rtn_quantize_pack(z, 0, 4, 48, 4, 32, z, z, 0, z, 3, 0, z) == 2     # BW_ERR_GROUP
    assert L.bw_rtn_quantize_pack(z, 0, 4, 12, 4, 4, z, z, 0, z, 3, 0, z) == 3      # K % 8 != 0
    assert L.bw_rtn_quantize_pack(z, 7, 4, 64, 4, 32, z, z, 0, z, 3, 0, z) == 4     # BW_ERR_DTYPE
    assert L.bw_rtn_quantize_pack(z, 0, 4, 64, 4, 32, z, z, 0, z, 3, 0, z) == 6     # BW_ERR_NULL
    assert L.bw_rtn_quantize_pack(z, 0, 0, 64, 4, 32, z, z, 0, z, 3, 0, z) == 0     # empty is fine
    assert L.bw_qmatmul(z, 1, 4, 8, 64, z, z, z, z, z, 1, 5, 32, z, 0, z) == 1
    assert L.bw_qmatmul(z, 1, 4, 8, 64, z, z, z, z, z, 1, 4, 0, z, 0, z) == 2
    assert L.bw_qmatmul(z, 1, 4, 8, 64, z, z, z, z, z, 1, 4, 32, z, 0, z) == 6
    assert L.bw_qmatmul(z, 1, 0, 8, 64, z, z, z, z, z, 1, 4, 32, z, 0, z) == 0
    assert L.bw_dequantize(z, z, 0, z, 3, 4, 64, 4, 32, z, 9, z) == 4
    # up to 32 tokens: the decode kernel's row-block shares (2 x 160 slots of [8*ceil(M/8)][128] fp32)
    assert L.bw_qmatmul_workspace_bytes(16, 4096, 4096, 4, 128) == 2 * 160 * 16 * 128 * 4
    assert L.bw_qmatmul_workspace_bytes(1, 4096, 100, 4, 4) == 2 * 160 * 8 * 128 * 4
    # more tokens: the fp16 cast of the activations for the tensor-core GEMM
    assert L.bw_qmatmul_workspace_bytes(64, 4096, 4096, 4, 128) == 64 * 4096 * 2
    assert L.bw_qmatmul_workspace_bytes(0, 8, 64, 4, 32) == 0
    # the query that knows the activation dtype: aligned fp16 activations go to the tensor cores as they
    # are, so only the 64-token scratch of the streaming kernel (its stand-in for odd layouts) is asked for
    assert L.bw_qmatmul_workspace_bytes_for(4096, 4096, 4096, 4, 128, 1, 16) == 64 * 4096 * 2
    assert L.bw_qmatmul_workspace_bytes_for(4096, 4096, 4096, 4, 128, 2, 16) == 4096 * 4096 * 2
    assert L.bw_qmatmul_workspace_bytes_for(4096, 4096, 4096, 4, 128, 1, 2) == 4096 * 4096 * 2
    # fake quantization of the trainable mode: argument rules before any CUDA call
    assert L.bw_fake_quant(z, 0, 4, 64, 3, 32, z, z, z, 0, z, z, z) == 1
    assert L.bw_fake_quant(z, 0, 4, 48, 4, 32, z, z, z, 0, z, z, z) == 2
    assert L.bw_fake_quant(z, 9, 4, 64, 4, 32, z, z, z, 0, z, z, z) == 4
    assert L.bw_fake_quant(z, 0, 4, 64, 4, 32, z, z, z, 0, z, z, z) == 6
    assert L.bw_fake_quant(z, 0, 0, 64, 4, 32, z, z, z, 0, z, z, z) == 0
    assert L.bw_fake_quant_backward(z, 0, 4, 64, 4, 32, z, z, z, 0, z, z, z, z) == 6
    # the gated epilogue: the activation code is checked, and N must hold whole (gate, up) row pairs in fours
    assert L.bw_qmatmul_fused(z, 1, 4, 6, 64, z, z, z, z, z, 1, 4, 32, _lib.Epilogue(_lib.ACT_SILU_MUL, None), z, 0, z) == 3   # BW_ERR_SHAPE
    assert L.bw_qmatmul_fused(z, 1, 4, 8, 64, z, z, z, z, z, 1, 4, 32, _lib.Epilogue(7, None), z, 0, z) == 9                   # unknown activation
    assert L.bw_fake_quant_native16(z, 0, 4, 64, 4, 32, z, z, z, z, z, z) == 4        # fp32 is not a 16-bit dtype
    assert L.bw_fake_quant_native16(z, 1, 4, 64, 4, 32, z, z, z, z, z, z) == 6
