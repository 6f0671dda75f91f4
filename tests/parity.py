"""Parity metric shared by the GPU tests.

Attention outputs average many N(0,1) values and have entries near zero, so a plain element-wise
relative error is ill-defined.  Both of these must hold, with tol = 1e-4 for float32 paths and
2e-2 for bf16 paths:
  * normalised max error  max|x - ref| / max|ref|  <= tol
  * np.allclose(x, ref, rtol=tol, atol=tol * rms(ref))
"""
import numpy as np

TOL_F32 = 1e-4
TOL_BF16 = 2e-2


def to_np(t):
    import torch
    if isinstance(t, torch.Tensor):
        t = t.detach()
        if t.dtype == torch.bfloat16:
            t = t.float()
        return t.cpu().numpy()
    return np.asarray(t)


def parity_errors(x, ref):
    x = to_np(x).astype(np.float64)
    ref = to_np(ref).astype(np.float64)
    scale = max(np.abs(ref).max(), 1e-30)
    return float(np.abs(x - ref).max() / scale), float(np.sqrt(np.mean(ref * ref)))


def assert_parity(x, ref, tol, what=""):
    xn, rn = to_np(x).astype(np.float64), to_np(ref).astype(np.float64)
    assert xn.shape == rn.shape, f"{what}: shape {xn.shape} vs {rn.shape}"
    assert np.isfinite(xn).all(), f"{what}: non-finite output"
    err, rms = parity_errors(xn, rn)
    assert err <= tol, f"{what}: normalised max error {err:.3e} > {tol}"
    assert np.allclose(xn, rn, rtol=tol, atol=tol * rms), f"{what}: allclose(rtol={tol}, atol={tol}*rms) failed"
    return err


def bf16_round(a):
    """Round a float32 array to bfloat16 and back (ml_dtypes)."""
    import ml_dtypes
    return np.asarray(a, dtype=np.float32).astype(ml_dtypes.bfloat16).astype(np.float32)


def assert_parity_logits(x, ref, tol, what="", max_outlier_fraction=0.01):
    """Model-level variant for logits produced through bf16 GEMM glue (cuBLAS rounds every layer output
    to bf16, so single elements move by one or two bf16 steps of an O(1) logit, i.e. up to a few per cent
    of the rms): the normalised max error must hold, and all but `max_outlier_fraction` of the elements
    must satisfy the allclose criterion."""
    xn, rn = to_np(x).astype(np.float64), to_np(ref).astype(np.float64)
    assert xn.shape == rn.shape and np.isfinite(xn).all(), what
    err, rms = parity_errors(xn, rn)
    assert err <= tol, f"{what}: normalised max error {err:.3e} > {tol}"
    bad = np.abs(xn - rn) > tol * rms + tol * np.abs(rn)
    assert bad.mean() <= max_outlier_fraction, f"{what}: {bad.mean():.4f} of the elements outside allclose"
    return err
