"""Pins the CPU oracle (oracle/bw_oracle.c) to fixtures produced by the reference itself.

The fixtures under tests/golden/ were written by tests/golden/gen_golden.py, which runs the
reference's bitween/functional.py on CPU.  Integer outputs (packed codes, zero-points) and
the scales must match bit for bit; so must the fp32 dequantized weights.
"""
import hashlib
import json
import os

import numpy as np
import pytest

from bitween_b200 import synth
from oracle import oracle

DT = {"f32": oracle.F32, "f16": oracle.F16, "bf16": oracle.BF16}


@pytest.fixture(scope="module")
def meta(golden_dir):
    with open(os.path.join(golden_dir, "digests.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def rtn_small(golden_dir):
    return np.load(os.path.join(golden_dir, "rtn_small.npz"))


@pytest.fixture(scope="module")
def fwd_small(golden_dir):
    return np.load(os.path.join(golden_dir, "forward_small.npz"))


def test_quantize_matches_reference_bit_exact(meta, rtn_small):
    assert len(meta["rtn_meta"]) > 90
    for c in meta["rtn_meta"]:
        n = c["name"]
        q, s, z = oracle.quantize_rtn(rtn_small[n + "/w"], DT[c["dtype"]], c["bits"], c["g"])
        assert np.array_equal(q, rtn_small[n + "/q"]), n
        assert np.array_equal(z, rtn_small[n + "/zp"]), n
        assert s.tobytes() == rtn_small[n + "/scale"].tobytes(), n


def test_dequantize_matches_reference_bit_exact(meta, rtn_small):
    for c in meta["rtn_meta"]:
        n = c["name"]
        d = oracle.dequantize_rtn(rtn_small[n + "/q"], rtn_small[n + "/scale"], rtn_small[n + "/zp"],
                                  c["g"], c["bits"], scale_dtype=DT[c["dtype"]])
        ref = rtn_small[n + "/deq"]
        assert d.dtype == ref.dtype == np.float32, n
        assert np.array_equal(d.view(np.uint32), ref.view(np.uint32)), n


def test_packed_words_can_be_negative(rtn_small):
    assert (rtn_small["edge_top_code_set_b4_f32/q"] < 0).any()
    assert (rtn_small["edge_top_code_set_b8_f32/q"] < 0).any()
    assert (rtn_small["edge_top_code_set_b2_f32/q"] < 0).any()


def test_constant_group_floor(rtn_small):
    # zero-range groups: scale floors at 1e-8, zero_point 0, positive constants saturate
    assert np.all(rtn_small["edge_constant_pos_b4_f32/scale"] == np.float32(1e-8))
    assert np.all(rtn_small["edge_constant_pos_b4_f32/zp"] == 0)
    assert np.all(rtn_small["edge_constant_pos_b4_f32/q"] == -1)


def _seeded(c):
    w = synth.normal(c["seed"], tuple(c["shape"]), c["std"])
    if c["dtype"] == "bf16->f32":
        return oracle.bits_to_f32(oracle.bf16_bits(w), oracle.BF16), oracle.F32
    if c["dtype"] == "f16":
        return oracle.f16_bits(w), oracle.F16
    if c["dtype"] == "bf16":
        return oracle.bf16_bits(w), oracle.BF16
    return w, oracle.F32


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_seeded_large_cases_match_reference_digests(meta):
    for name, c in meta["digests"].items():
        w, dt = _seeded(c)
        assert _sha(w) == c["w_sha256"], f"{name}: synthetic input is not reproducible here"
        q, s, z = oracle.quantize_rtn(w, dt, c["bits"], c["g"])
        assert _sha(q) == c["q_sha256"], name
        assert _sha(s) == c["scale_sha256"], name
        assert _sha(z) == c["zp_sha256"], name
        if dt == oracle.F32:
            # the module-buffer casts of QuantizedLinear.from_float (modules.py:207-209)
            assert _sha(oracle.f16_bits(s)) == c["scale_h_sha256"], name
            assert _sha(oracle.f16_bits(z.astype(np.float32))) == c["zp_h_sha256"], name


def test_forward_weights_bit_exact_and_output_within_tolerance(meta, fwd_small):
    for c in meta["fwd_meta"]:
        n = c["name"]
        x_h = oracle.f16_bits(fwd_small[n + "/x"])
        bias_h = oracle.f16_bits(fwd_small[n + "/bias"]) if c["bias"] else None
        w_h = oracle.dequantize_module(fwd_small[n + "/q"], fwd_small[n + "/scale_h"],
                                       fwd_small[n + "/zp_h"], c["g"], c["bits"])
        assert np.array_equal(w_h, fwd_small[n + "/w_h"]), n
        y, acc = oracle.qlinear_forward(x_h, fwd_small[n + "/q"], fwd_small[n + "/scale_h"],
                                        fwd_small[n + "/zp_h"], bias_h, c["bits"], c["g"],
                                        want_acc=True)
        ref = oracle.bits_to_f32(fwd_small[n + "/y_h"], oracle.F16)
        got = oracle.bits_to_f32(y, oracle.F16)
        rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
        # stated tolerance for 16-bit outputs: max |err| <= 1e-2 * RMS(output)
        assert np.abs(got - ref).max() <= 1e-2 * rms, n
        # fp32-accumulate check: <= 1e-5 relative to the output scale
        ref64 = fwd_small[n + "/y_acc64"]
        assert np.abs(acc - ref64).max() <= 1e-5 * np.abs(ref64).max(), n


def test_error_conventions():
    w = np.zeros((2, 48), dtype=np.float32)
    with pytest.raises(ValueError):
        oracle.quantize_rtn(w, oracle.F32, 4, 32)      # functional.py:12-17
    with pytest.raises(AssertionError):
        oracle.quantize_rtn(w, oracle.F32, 3, 16)      # functional.py:6
