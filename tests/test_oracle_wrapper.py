"""The oracle's restatement of WrapperLinear's fake quantization (bitween/wrapper.py:116-172)
against outputs of the reference class itself (tests/golden/wrapper_small.npz, made by
tests/golden/gen_golden_wrapper.py): bit-exact."""
import json
import os

import numpy as np
import pytest

from oracle import oracle

DT = {"f32": oracle.F32, "f16": oracle.F16, "bf16": oracle.BF16, "float32": oracle.F32, "float16": oracle.F16,
      "bfloat16": oracle.BF16}


@pytest.fixture(scope="module")
def cases(golden_dir):
    with open(os.path.join(golden_dir, "wrapper_meta.json")) as f:
        return json.load(f)["cases"]


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "wrapper_small.npz"))


def same_numbers(a, b):
    """Bitwise equal, except that a zero may carry either sign: round() gives -0.0 for small negative
    t and whether torch.clamp(-0.0, 0, qmax) keeps the sign differs between its CPU and CUDA kernels."""
    a, b = np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)
    return bool(np.all((a.view(np.uint32) == b.view(np.uint32)) | ((a == 0) & (b == 0))))


def as32(gold, key, dt):
    a = gold[key]
    return a if a.dtype == np.float32 else oracle.bits_to_f32(a, DT[dt])


def case_inputs(gold, c):
    n = c["name"]
    w = as32(gold, n + "/w", c["dtype"])
    mn = gold[n + "/min_scale"] if c["minmax"] else None
    mx = gold[n + "/max_scale"] if c["minmax"] else None
    v = as32(gold, n + "/value", c["value_dtype"]) if c["round"] else None
    return w, mn, mx, v


def test_fake_quant_matches_reference_bit_exact(cases, gold):
    assert len(cases) >= 40
    native = 0
    for c in cases:
        n = c["name"]
        if c["out_dtype"] != "float32":
            # every tensor 16-bit: the per-operation rounding of the reference
            assert not c["minmax"] and c["out_dtype"] == {"f16": "float16", "bf16": "bfloat16"}[c["dtype"]]
            dt = DT[c["dtype"]]
            dq, q, scale, zp = oracle.wrapper_fake_quant_native(gold[n + "/w"], gold[n + "/value"] if c["round"] else None,
                                                                dt, c["bits"], c["g"])
            for got, key in ((scale, "/scale"), (zp, "/zp"), (q, "/w_q"), (dq, "/w_dq")):
                assert same_numbers(got, oracle.bits_to_f32(gold[n + key], dt).reshape(got.shape)), (n, key)
            native += 1
            continue
        w, mn, mx, v = case_inputs(gold, c)
        scale, zp = oracle.wrapper_group_params(w, c["bits"], c["g"], mn, mx)
        assert np.array_equal(scale.view(np.uint32), gold[n + "/scale"].view(np.uint32)), n
        assert np.array_equal(zp.view(np.uint32), gold[n + "/zp"].view(np.uint32)), n
        dq, q = oracle.wrapper_fake_quant(w, scale, zp, v, c["bits"], c["g"])
        assert same_numbers(q, gold[n + "/w_q"]), n
        assert same_numbers(dq, gold[n + "/w_dq"]), n
    assert native >= 5


def test_param_grads_match_reference_autograd(cases, gold):
    checked = 0
    for c in cases:
        n = c["name"]
        if n + "/grad_min_scale" not in gold.files:
            continue
        w, mn, mx, v = case_inputs(gold, c)
        scale, zp = oracle.wrapper_group_params(w, c["bits"], c["g"], mn, mx)
        gs, gz = oracle.wrapper_param_grads(w, scale, zp, v, gold[n + "/r"], c["bits"], c["g"])
        # chain rule through bitween/wrapper.py:131-140 in float64 (scale above its 1e-8 floor)
        N, K = w.shape
        grouped = w.reshape(N, K // c["g"], c["g"]).astype(np.float64)
        w_min, w_max = grouped.min(-1), grouped.max(-1)
        qmax = (1 << c["bits"]) - 1
        s = scale.astype(np.float64)
        live = (((w_max * mx - w_min * mn) / qmax) >= 1e-8).astype(np.float64)
        a = w_min * mn
        # zp = -a / s ;  s = (b - a) / qmax
        d_a = gz * (-1.0 / s) + (gs + gz * (a / s ** 2)) * live * (-1.0 / qmax)
        d_b = (gs + gz * (a / s ** 2)) * live * (1.0 / qmax)
        want_min, want_max = gold[n + "/grad_min_scale"].astype(np.float64), gold[n + "/grad_max_scale"].astype(np.float64)
        got_min, got_max = d_a * w_min, d_b * w_max
        tol = 2e-4 * max(1.0, np.abs(want_min).max(), np.abs(want_max).max())
        assert np.abs(got_min - want_min).max() <= tol, n
        assert np.abs(got_max - want_max).max() <= tol, n
        checked += 1
    assert checked >= 30
