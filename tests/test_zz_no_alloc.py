"""The allocation-free gate-gradient entry point (collected last on purpose).

Callers that cannot allocate device memory where they call us get a variant of the fused block's
gate-gradient call whose scratch is a fixed array inside the library.  It must give what the
regular entry point gives, on repeated calls (the array keeps the previous call's contents), and
refuse shapes that do not fit."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(n, ci, c, size, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.rand(n, ci, size, size, generator=g).cuda()
    w = torch.randn(c, 7, 16, generator=g).cuda()
    sel = ((torch.randint(0, ci, (c, 8), generator=g) << 16) | (torch.randint(0, 3, (c, 8), generator=g) << 8)
           | torch.randint(0, 3, (c, 8), generator=g)).to(torch.int32).cuda()
    gy = torch.randn(n, c, size // 2, size // 2, generator=g).cuda()
    return x, w, sel, gy


def test_noalloc_gate_gradient_matches_regular_entry_point_twice():
    from convlogic_b200 import ops
    from convlogic_b200._lib import W_SOFTMAX

    geom = (1, 1, 1, 1, 3, 3)
    # two different problems back to back: the second call sees the first one's leftovers in the array
    for n, ci, c, size, seed in ((64, 9, 96, 32, 1), (24, 5, 40, 16, 2)):
        x, w, sel, gy = _inputs(n, ci, c, size, seed)
        _, amax, _, _, _ = ops.convtree_fwd(x, w, sel, geom, W_SOFTMAX)
        want = ops.convtree_bwd_w(gy, x, w, sel, amax, geom, W_SOFTMAX)
        out = torch.full_like(w, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        ops.convtree_bwd_w_noalloc(gy, x, w, sel, amax, geom, W_SOFTMAX, out)
        again = torch.empty_like(w)
        after_alloc = torch.cuda.memory_allocated()
        ops.convtree_bwd_w_noalloc(gy, x, w, sel, amax, geom, W_SOFTMAX, again)
        torch.cuda.synchronize()
        assert after_alloc - before <= again.numel() * 4 + 512  # nothing but the test's own `again`
        rel = float((out - want).abs().max() / want.abs().max())
        assert rel <= 1e-5, rel
        assert torch.equal(out, again)


def test_noalloc_rejects_what_does_not_fit():
    from convlogic_b200 import _lib, ops
    from convlogic_b200._lib import W_SOFTMAX

    limit = _lib.lib().clb_convtree_bwd_w_noalloc_max_bytes()
    assert limit == 4 << 20
    n, ci, c, size = 2, 2, 40000, 4  # 40000 channels x 28 sums x 4 B > 4 MiB
    need = _lib.lib().clb_convtree_bwd_w_scratch_bytes(n, c, size, size, _lib.F32)
    assert need > limit
    x, w, sel, gy = _inputs(n, ci, c, size, 3)
    amax = torch.zeros(n, c, size // 2, size // 2, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError, match="fixed maximum"):
        ops.convtree_bwd_w_noalloc(gy, x, w, sel, amax, (1, 1, 1, 1, 3, 3), W_SOFTMAX, torch.empty_like(w))
