"""Comparison helpers of the test-suite.

Two error measures are used and every test says which one it claims:

* ``rel_err`` / ``assert_close``: MAX-NORMALISED error, ``max|got - want| / max|want|`` -- one number per
  tensor.  This is the measure behind the "1e-5 in fp32" statements of the GPU tests.
* ``assert_close_elementwise``: every element on its own, ``|got - want| <= rtol * |want| + floor``, with the
  absolute floor given as a fraction of ``max|want|`` (gradient entries are sums with cancellation, so an
  element near zero has no meaningful relative error of its own; the floor is kept 10x below the
  max-normalised tolerance).
"""

import numpy as np
import torch


def rel_err(got, want):
    got = torch.as_tensor(got).double().cpu()
    want = torch.as_tensor(want).double().cpu()
    return float((got.detach() - want.detach()).abs().max() / want.abs().max().clamp_min(1e-30))


def assert_close(got, want, tol, what=""):
    e = rel_err(got, want)
    assert e <= tol, f"{what}: max-normalised error {e:.3e} > {tol:.1e}"


def assert_close_elementwise(got, want, rtol, floor_of_max, what=""):
    got = torch.as_tensor(got).detach().double().cpu()
    want = torch.as_tensor(want).detach().double().cpu()
    bound = rtol * want.abs() + floor_of_max * want.abs().max()
    excess = (got - want).abs() - bound
    worst = int(excess.argmax())
    assert float(excess.max()) <= 0, (
        f"{what}: element {worst}: got {float(got.reshape(-1)[worst]):.9g}, want {float(want.reshape(-1)[worst]):.9g}, "
        f"allowed {float(bound.reshape(-1)[worst]):.3g} (rtol {rtol:.1e}, floor {floor_of_max:.1e} of max)")


def assert_same_argmax_up_to_ties(idx, idx_ref, max_fraction, what="arg-max"):
    """Pooled positions may differ from the checker's only where two candidates of a window tie to rounding;
    bound the fraction of such windows (the values themselves are compared separately)."""
    frac = float((torch.as_tensor(idx).cpu() != torch.as_tensor(idx_ref).cpu()).float().mean())
    assert frac <= max_fraction, f"{what}: {frac:.2e} of the windows differ (allowed {max_fraction:.1e})"
    return frac


def random_selection(rng, c, ci, kh, kw):
    ch = rng.integers(0, ci, (c, 8))
    r = rng.integers(0, kh, (c, 8))
    s = rng.integers(0, kw, (c, 8))
    return torch.from_numpy(((ch << 16) | (r << 8) | s).astype(np.int32))
