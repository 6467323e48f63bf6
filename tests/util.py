import numpy as np
import torch


def rel_err(got, want):
    got = torch.as_tensor(got).double().cpu()
    want = torch.as_tensor(want).double().cpu()
    return float((got.detach() - want.detach()).abs().max() / want.abs().max().clamp_min(1e-30))


def assert_close(got, want, tol, what=""):
    e = rel_err(got, want)
    assert e <= tol, f"{what}: relative error {e:.3e} > {tol:.1e}"


def random_selection(rng, c, ci, kh, kw):
    ch = rng.integers(0, ci, (c, 8))
    r = rng.integers(0, kh, (c, 8))
    s = rng.integers(0, kw, (c, 8))
    return torch.from_numpy(((ch << 16) | (r << 8) | s).astype(np.int32))
