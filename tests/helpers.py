"""Shared helpers of the test-suite: torch <-> oracle conversions and tolerance checks."""
import numpy as np
import torch

from oracle import oracle

ORACLE_DT = {torch.float32: oracle.F32, torch.float16: oracle.F16, torch.bfloat16: oracle.BF16}


def to_np(t):
    """torch tensor -> numpy; 16-bit floats become uint16 bit patterns."""
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def from_bits(a, dtype):
    """numpy uint16 bit patterns -> torch fp16/bf16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(dtype)


def as_f32(t):
    return t.detach().float().cpu().numpy()


def rms(a):
    a = np.asarray(a, dtype=np.float64)
    return float(np.sqrt(np.mean(a * a))) if a.size else 0.0


def assert_close_rms(got, ref, factor=1e-2, what=""):
    """The stated 16-bit tolerance: max |err| <= 1e-2 * RMS(reference output)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    if ref.size == 0:
        return
    err = np.abs(got - ref).max()
    bound = factor * max(rms(ref), 1e-30)
    assert err <= bound, f"{what}: max|err|={err:.4g} > {factor:g}*RMS={bound:.4g}"


def oracle_forward(x, q, scale_h, zp_h, bias_h, bits, g, act=torch.float16, want_acc=False):
    """Reference forward semantics on CPU: x is cast to `act` first (modules.py:74)."""
    xb = to_np(x.to(act))
    out = oracle.qlinear_forward(xb, to_np(q), to_np(scale_h), to_np(zp_h),
                                 None if bias_h is None else to_np(bias_h.to(act)), bits, g,
                                 act_dtype=ORACLE_DT[act], want_acc=want_acc)
    if want_acc:
        return from_bits(out[0], act), torch.from_numpy(out[1])
    return from_bits(out, act)
