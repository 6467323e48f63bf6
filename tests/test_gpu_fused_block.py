"""Fused ConvLogic block on the GPU against the golden tensors of the reference's CPU path and
against the CPU oracle.  Tolerances: soft mode fp32 1e-5 relative (to the tensor's max), fp64 1e-10;
hard mode on {0,1} inputs exact."""

import numpy as np
import pytest
import torch

import oracle
from tests.golden.make_golden import FUSED_CASES
from tests.util import assert_close, assert_close_elementwise, assert_same_argmax_up_to_ties, random_selection, rel_err

pytestmark = pytest.mark.gpu

F32_TOL, F64_TOL = 1e-5, 1e-10


def _layer(cb, g, name, dtype):
    sh, sw, ph, pw, kh, kw = (int(v) for v in g[f"{name}/geom"])
    sel = torch.from_numpy(g[f"{name}/selection"])
    c, ci = sel.shape[0], g[f"{name}/x"].shape[1]
    layer = cb.ConvLogicLayer(ci, c, stride=(sh, sw), padding=(ph, pw), kernel=(kh, kw), selection=sel, complete=True)
    layer.weights.data = torch.from_numpy(g[f"{name}/logits"])
    return layer.to("cuda", dtype)


@pytest.mark.parametrize("name", [c[0] for c in FUSED_CASES])
@pytest.mark.parametrize("tag,dtype,tol", [("f32", torch.float32, F32_TOL), ("f64", torch.float64, F64_TOL)])
def test_matches_reference_golden(golden, name, tag, dtype, tol):
    import convlogic_b200 as cb

    g = golden("fused_block")
    layer = _layer(cb, g, name, dtype).train()
    x = torch.from_numpy(g[f"{name}/x"]).to("cuda", dtype).requires_grad_(True)
    gy = torch.from_numpy(g[f"{name}/gy"]).to("cuda", dtype)
    y = layer(x)
    (y * gy).sum().backward()
    assert_close(y, g[f"{name}/{tag}/y_soft"], tol, "soft forward")
    assert_close(x.grad, g[f"{name}/{tag}/gx"], tol, "input gradient")
    assert_close(layer.weights.grad, g[f"{name}/{tag}/gw_logits"], tol, "logit gradient")
    layer.eval()
    with torch.no_grad():
        yh = layer(x.detach())
    if "bits" in name:
        assert np.array_equal(yh.cpu().numpy(), g[f"{name}/{tag}/y_hard"])
    else:
        assert_close(yh, g[f"{name}/{tag}/y_hard"], max(tol, 1e-6), "hard forward")


SHAPES = [
    # N, Ci, C, H, W, stride, pad, kernel, input
    (8, 9, 32, 32, 32, 1, 1, 3, "bits"),     # the microbenchmark's block at reduced batch / width
    (5, 16, 24, 12, 12, 1, 1, 3, "rand"),    # mnist_s block 2 shape
    (3, 1, 16, 28, 28, 1, 0, 5, "bits"),     # mnist_s block 1: 5x5 window, no padding
    (7, 48, 40, 6, 6, 1, 1, 3, "rand"),      # small images, several images per block in backward
    (2, 300, 20, 4, 4, 1, 1, 3, "rand"),     # more input channels than one shared-memory group holds
    (2, 3, 5, 70, 66, 1, 1, 3, "rand"),      # > 1024 pooled positions (the reference's limit)
    (4, 3, 6, 14, 10, 2, 2, 4, "randn"),     # stride 2
    (1, 1, 1, 3, 3, 1, 0, 2, "randn"),       # single output
]


def _case(shape, seed=0):
    n, ci, c, h, w, st, pd, k, kind = shape
    rng = np.random.default_rng(seed)
    g = torch.Generator().manual_seed(seed)
    sel = random_selection(rng, c, ci, k, k)
    logits = torch.randn(c, 7, 16, generator=g)
    if kind == "bits":
        x = (torch.rand(n, ci, h, w, generator=g) < 0.5).float()
    elif kind == "rand":
        x = torch.rand(n, ci, h, w, generator=g)
    else:
        x = torch.randn(n, ci, h, w, generator=g)
    ho, wo = oracle.conv_oracle.out_size(h, w, st, pd, k)
    gy = torch.randn(n, c, ho // 2, wo // 2, generator=g)
    return x, logits, sel, gy, (st, st, pd, pd, k, k)


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(str(v) for v in s))
@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.float64, F64_TOL)])
def test_matches_oracle_function_api(shape, dtype, tol):
    """The reference-style call: probabilities in, gradient w.r.t. probabilities out."""
    from convlogic_b200 import FullConvLogicFunction

    x, logits, sel, gy, geom = _case(shape)
    x, logits, gy = x.to(dtype), logits.to(dtype), gy.to(dtype)
    xo = x.clone().requires_grad_(True)
    po = torch.softmax(logits, -1).requires_grad_(True)
    yo, x2o, x3o, idxo = oracle.full_convlogic(xo, po, sel, geom[0:2], geom[2:4], geom[4:6])

    xd = x.cuda().requires_grad_(True)
    pd = torch.softmax(logits, -1).cuda().requires_grad_(True)
    y, x2, x3, idx = FullConvLogicFunction.apply(xd, pd, sel.cuda(), *geom, True, True)
    gx, gp = torch.autograd.grad((y * gy.cuda()).sum(), (xd, pd))
    assert_close(y, yo.detach(), tol, "y")
    assert_close(x2, x2o.detach(), tol, "x2")
    assert_close(x3, x3o.detach(), tol, "x3")
    # A different arg-max is acceptable only between candidates that tie to fp32 rounding (y is compared above); the
    # gradients are ALWAYS compared: the oracle's backward is taken at the positions the kernels pooled.
    assert_same_argmax_up_to_ties(idx, idxo, 1e-3 if dtype == torch.float32 else 0.0)
    yf = oracle.full_convlogic(xo, po, sel, geom[0:2], geom[2:4], geom[4:6], forced_idx=idx.cpu())[0]
    gxo, gpo = torch.autograd.grad((yf * gy).sum(), (xo, po))
    assert_close(gx, gxo, tol, "gx")
    assert_close(gp, gpo, tol, "gw (mixture)")
    # plain path (no intermediates) gives the same y and gradients
    y2 = FullConvLogicFunction.apply(xd, pd, sel.cuda(), *geom)
    gx2, gp2 = torch.autograd.grad((y2 * gy.cuda()).sum(), (xd, pd))
    assert torch.equal(y2, y) or rel_err(y2, y) < tol
    assert_close(gx2, gx, tol)
    assert_close(gp2, gp, tol)


def test_backward_is_bitwise_deterministic():
    import convlogic_b200 as cb

    x, logits, sel, gy, geom = _case((16, 9, 64, 32, 32, 1, 1, 3, "bits"), seed=3)
    layer = cb.ConvLogicLayer(9, 64, selection=sel, complete=True).cuda().train()
    layer.weights.data = logits.cuda()
    outs = []
    for _ in range(3):
        xd = x.cuda().requires_grad_(True)
        layer.weights.grad = None
        (layer(xd) * gy.cuda()).sum().backward()
        outs.append((xd.grad.clone(), layer.weights.grad.clone()))
    for gx, gw in outs[1:]:
        assert torch.equal(gx, outs[0][0]) and torch.equal(gw, outs[0][1])


@pytest.mark.parametrize("batch", [1, 16])
@pytest.mark.parametrize("c_in,c_out", [(1, 1), (3, 1), (1, 3)])
@pytest.mark.parametrize("stride,pad,kernel", [(1, 1, 3), (2, 2, 4)])
def test_gradcheck_like_reference(batch, c_in, c_out, stride, pad, kernel):
    """The reference's own gradient test (tests/convlogic/test_full_convlogic_autograd.py:36-104)."""
    import convlogic_b200 as cb
    from torch.autograd import gradcheck

    torch.manual_seed(0)
    layer = cb.ConvLogicLayer(c_in, c_out, stride=stride, padding=pad, kernel=kernel, complete=True).double().cuda()
    x = torch.sigmoid(torch.rand(batch, c_in, 6, 6, dtype=torch.double, device="cuda")).requires_grad_(True)
    w = layer.weights.detach().clone().requires_grad_(True)
    sel = layer.selection

    def fn(inp, logits):
        return cb.FullConvLogicFunction.apply(inp, torch.softmax(logits, -1), sel, stride, stride, pad, pad, kernel, kernel, False)

    assert gradcheck(fn, (x, w), eps=1e-6, atol=1e-4)


def test_hard_mode_binary_in_binary_out_and_residual_init():
    import convlogic_b200 as cb

    torch.manual_seed(0)
    layer = cb.ConvLogicLayer(2, 2, padding=1, residual_init=True, complete=True).cuda().eval()
    assert torch.all(layer.weights.argmax(-1) == 3)
    x = (torch.rand(4, 2, 6, 6, device="cuda") < 0.5).float()
    y = layer(x)
    assert y.shape == (4, 2, 3, 3)
    assert set(y.unique().tolist()) <= {0.0, 1.0}
    layer2 = cb.ConvLogicLayer(1, 5, complete=True).cuda().eval()
    assert layer2(torch.randn(1, 1, 6, 6, device="cuda")).shape == (1, 5, 3, 3)
    yr = layer2(torch.rand(3, 1, 6, 6, device="cuda"))
    assert (yr >= 0).all() and (yr <= 1).all() and torch.isfinite(yr).all()


def test_shape_errors_surface_as_exceptions():
    import convlogic_b200 as cb

    layer = cb.ConvLogicLayer(1, 1, kernel=3, padding=0, complete=True).cuda()
    with pytest.raises(RuntimeError, match="divisible by 2"):
        layer(torch.rand(1, 1, 5, 5, device="cuda"))  # 3x3 conv output
    with pytest.raises(RuntimeError):
        layer(torch.rand(1, 1, 6, 6))  # CPU tensor: there is no CPU path
    y = layer(torch.rand(2, 1, 6, 6, device="cuda"))  # the context is still usable
    assert y.shape == (2, 1, 2, 2)


def test_grad_factor_and_eval_mode_input_gradient():
    import convlogic_b200 as cb

    x, logits, sel, gy, geom = _case((3, 4, 6, 8, 8, 1, 1, 3, "rand"), seed=5)
    layer = cb.ConvLogicLayer(4, 6, selection=sel, complete=True, grad_factor=2.0).cuda().eval()
    layer.weights.data = logits.cuda()
    xd = x.cuda().requires_grad_(True)
    (layer(xd) * gy.cuda()).sum().backward()
    xo = x.clone().requires_grad_(True)
    yo = oracle.full_convlogic(xo, oracle.gate_probabilities(logits, False), sel)[0]
    (gxo,) = torch.autograd.grad((yo * gy).sum(), (xo,))
    assert_close(xd.grad, 2.0 * gxo, F32_TOL)
    assert layer.weights.grad is None


def test_group_tables_follow_the_selection_not_its_address():
    """Two layers of equal shape but different taps (and different widths) in a row: the cached
    channel-group tables must never be shared between selection tensors."""
    import convlogic_b200 as cb

    for c in (1, 3, 5, 3):
        x, logits, sel, gy, geom = _case((2, 300, c, 4, 4, 1, 1, 3, "rand"), seed=c)
        layer = cb.ConvLogicLayer(300, c, selection=sel, complete=True).cuda().train()
        layer.weights.data = logits.cuda()
        xd = x.cuda().requires_grad_(True)
        (layer(xd) * gy.cuda()).sum().backward()
        xo = x.clone().requires_grad_(True)
        yo = oracle.full_convlogic(xo, oracle.gate_probabilities(logits, True), sel)[0]
        (gxo,) = torch.autograd.grad((yo * gy).sum(), (xo,))
        assert_close(xd.grad, gxo, F32_TOL)
        del layer, xd


def test_taps_outside_the_kernel_window_are_served():
    """A user selection may name rows/cols beyond the window; the reference kernels read them as
    long as they land inside the image.  The shape-specialised kernel must not be used then."""
    import convlogic_b200 as cb

    g = torch.Generator().manual_seed(9)
    n, ci, c = 4, 3, 8
    ch = torch.randint(0, ci, (c, 8), generator=g)
    r = torch.randint(0, 6, (c, 8), generator=g)   # window is 3x3
    s = torch.randint(0, 6, (c, 8), generator=g)
    sel = ((ch << 16) | (r << 8) | s).to(torch.int32)
    logits = torch.randn(c, 7, 16, generator=g)
    x = torch.rand(n, ci, 16, 16, generator=g)
    layer = cb.ConvLogicLayer(ci, c, selection=sel, complete=True).cuda().train()
    layer.weights.data = logits.cuda()
    xd = x.cuda().requires_grad_(True)
    y = layer(xd)
    gy = torch.randn(*y.shape, generator=g)
    (y * gy.cuda()).sum().backward()
    xo = x.clone().requires_grad_(True)
    wo = logits.clone().requires_grad_(True)
    yo = oracle.full_convlogic(xo, oracle.gate_probabilities(wo, True), sel)[0]
    gxo, gwo = torch.autograd.grad((yo * gy).sum(), (xo, wo))
    assert_close(y, yo.detach(), F32_TOL)
    assert_close(xd.grad, gxo, F32_TOL)
    assert_close(layer.weights.grad, gwo, F32_TOL)


@pytest.mark.parametrize("shape", [
    (256, 9, 256, 32, 32, 1, 1, 3, "bits"),   # the benchmark block at full size
    (37, 9, 19, 32, 32, 1, 1, 3, "rand"),     # ragged batch / channel counts
    (64, 16, 48, 12, 12, 1, 1, 3, "rand"),
    (9, 1, 16, 28, 28, 1, 0, 5, "bits"),
    (33, 32, 20, 16, 16, 1, 1, 3, "rand"),
    (70, 48, 24, 8, 8, 1, 1, 3, "rand"),
    (130, 12, 10, 4, 4, 1, 1, 3, "rand"),
], ids=lambda s: "x".join(str(v) for v in s))
def test_tiled_forward_equals_general_forward(shape):
    """The shape-specialised forward (used when no intermediates are requested) against the
    general kernel (forced by asking for the indices) and, for values, against the oracle."""
    from convlogic_b200 import ops
    from convlogic_b200._lib import W_SOFTMAX

    x, logits, sel, gy, geom = _case(shape, seed=11)
    xd, wd, sd = x.cuda(), logits.cuda(), sel.cuda()
    y_fast, amax_fast, _, _, _ = ops.convtree_fwd(xd, wd, sd, geom, W_SOFTMAX)
    y_gen, amax_gen, _, _, idx = ops.convtree_fwd(xd, wd, sd, geom, W_SOFTMAX, want_indices=True)
    assert torch.equal(y_fast, y_gen)
    assert torch.equal(amax_fast, amax_gen)
    if x.shape[0] <= 40:
        yo = oracle.full_convlogic(x, oracle.gate_probabilities(logits, True), sel, geom[0:2], geom[2:4], geom[4:6])[0]
        assert_close(y_fast, yo, F32_TOL)


@pytest.mark.parametrize("shape", [
    (256, 9, 256, 32, 32, 1, 1, 3, "bits"),
    (37, 9, 19, 32, 32, 1, 1, 3, "rand"),
    (3, 9, 700, 32, 32, 1, 1, 3, "rand"),     # fewer images than blocks: an image's channels are split over many blocks
    (64, 16, 48, 12, 12, 1, 1, 3, "rand"),
    (9, 1, 16, 28, 28, 1, 0, 5, "bits"),
    (33, 32, 20, 16, 16, 1, 1, 3, "rand"),
    (70, 48, 24, 8, 8, 1, 1, 3, "rand"),
    (130, 12, 10, 4, 4, 1, 1, 3, "rand"),
], ids=lambda s: "x".join(str(v) for v in s))
def test_tiled_input_gradient_equals_general(shape):
    """The tiled input-gradient kernel (scratch given) against the general one (no scratch): same
    mathematics, different summation order, so equality is to rounding; and bitwise repeatable."""
    from convlogic_b200 import ops
    from convlogic_b200._lib import W_SOFTMAX

    x, logits, sel, gy, geom = _case(shape, seed=12)
    xd, wd, sd, gd = x.cuda(), logits.cuda(), sel.cuda(), gy.cuda()
    _, amax, _, _, _ = ops.convtree_fwd(xd, wd, sd, geom, W_SOFTMAX)
    g_fast = ops.convtree_bwd_x(gd, xd, wd, sd, amax, geom, W_SOFTMAX)
    g_gen = ops.convtree_bwd_x(gd, xd, wd, sd, amax, geom, W_SOFTMAX, use_scratch=False)
    assert_close(g_fast, g_gen, 2e-6)
    assert torch.equal(g_fast, ops.convtree_bwd_x(gd, xd, wd, sd, amax, geom, W_SOFTMAX))
    # the combined kernel (one arg-max recompute for both gradients) against the separate ones
    gx_c, gw_c = ops.convtree_bwd(gd, xd, wd, sd, amax, geom, W_SOFTMAX)
    assert torch.equal(gx_c, g_fast)
    assert_close(gw_c, ops.convtree_bwd_w(gd, xd, wd, sd, amax, geom, W_SOFTMAX), 2e-5)
    _, gw_only = ops.convtree_bwd(gd, xd, wd, sd, amax, geom, W_SOFTMAX, need_gx=False)
    assert torch.equal(gw_only, gw_c)
    gx_only, none = ops.convtree_bwd(gd, xd, wd, sd, amax, geom, W_SOFTMAX, need_gw=False)
    assert none is None and torch.equal(gx_only, g_fast)
    if x.shape[0] <= 40 and shape[2] <= 64:
        xo = x.clone().requires_grad_(True)
        yo, _, _, idxo = oracle.full_convlogic(xo, oracle.gate_probabilities(logits, True), sel, geom[0:2], geom[2:4], geom[4:6])
        idx = ops.convtree_fwd(xd, wd, sd, geom, W_SOFTMAX, want_indices=True)[4].cpu()
        assert_same_argmax_up_to_ties(idx, idxo, 1e-3)
        wo = logits.clone().requires_grad_(True)
        yf = oracle.full_convlogic(xo, oracle.gate_probabilities(wo, True), sel, geom[0:2], geom[2:4], geom[4:6], forced_idx=idx)[0]
        gxf, gwf = torch.autograd.grad((yf * gy).sum(), (xo, wo))
        assert_close(g_fast, gxf, F32_TOL, "gx at the kernels' own arg-max")
        assert_close(gw_c, gwf, F32_TOL, "gw at the kernels' own arg-max")


@pytest.mark.parametrize("shape", [
    (40, 64, 24, 16, 16, 1, 1, 3, "rand"),     # channels do not fit shared memory: two-plane staging
    (33, 128, 20, 8, 8, 1, 1, 3, "rand"),
    (130, 600, 10, 4, 4, 1, 1, 3, "rand"),
    (5, 40, 6, 32, 32, 1, 1, 3, "rand"),
], ids=lambda s: "x".join(str(v) for v in s))
def test_many_channel_forward_paths_agree(shape):
    """Staged two-plane forward vs the general kernel; also with a selection that names more than two
    channels per output channel (third and later channels are gathered from global memory)."""
    from convlogic_b200 import ops
    from convlogic_b200._lib import W_SOFTMAX

    x, logits, sel, gy, geom = _case(shape, seed=13)   # random_selection: up to 8 distinct channels per output
    n, ci, c = shape[0], shape[1], shape[2]
    rng = np.random.default_rng(5)
    two = rng.integers(0, ci, (c, 2))
    pick = rng.integers(0, 2, (c, 8))
    ch2 = np.take_along_axis(two, pick, 1)
    sel2 = torch.from_numpy(((ch2 << 16) | (rng.integers(0, 3, (c, 8)) << 8) | rng.integers(0, 3, (c, 8))).astype(np.int32))
    for sel_t in (sel2, sel):
        xd, wd, sd = x.cuda(), logits.cuda(), sel_t.cuda()
        y_fast, amax_fast, _, _, _ = ops.convtree_fwd(xd, wd, sd, geom, W_SOFTMAX)
        y_gen, amax_gen, _, _, _ = ops.convtree_fwd(xd, wd, sd, geom, W_SOFTMAX, want_indices=True)
        assert torch.equal(y_fast, y_gen)
        assert torch.equal(amax_fast, amax_gen)


@pytest.mark.parametrize("shape", [
    (40, 64, 24, 16, 16, 1, 1, 3, "rand"),     # 64 windows per image: named barriers per image
    (33, 128, 20, 8, 8, 1, 1, 3, "rand"),      # 16 windows per image: warp-level ordering
    (130, 600, 10, 4, 4, 1, 1, 3, "rand"),     # 4 windows per image
    (5, 40, 6, 32, 32, 1, 1, 3, "rand"),       # 256 windows per image: block barrier
    (20, 70, 12, 12, 12, 1, 1, 3, "rand"),     # 36 windows per image: neither divides a warp nor fills warps
    (64, 256, 96, 16, 16, 1, 1, 3, "bits"),
], ids=lambda s: "x".join(str(v) for v in s))
def test_two_pass_backward_of_many_channel_layers(shape):
    """Layers whose input does not fit the tiled kernel take the two-pass backward (gate sums + tap gradients in one
    kernel, then a scatter into gx): equal to the separate kernels to rounding, repeatable bit for bit, and equal
    to the CPU oracle on small cases.  (The first shape still fits the tiled kernel and is here as a control.)"""
    from convlogic_b200 import ops
    from convlogic_b200._lib import W_SOFTMAX

    x, logits, sel, gy, geom = _case(shape, seed=21)
    xd, wd, sd, gd = x.cuda(), logits.cuda(), sel.cuda(), gy.cuda()
    _, amax, _, _, _ = ops.convtree_fwd(xd, wd, sd, geom, W_SOFTMAX)
    gx_c, gw_c = ops.convtree_bwd(gd, xd, wd, sd, amax, geom, W_SOFTMAX)
    gx_s = ops.convtree_bwd_x(gd, xd, wd, sd, amax, geom, W_SOFTMAX)
    assert_close(gx_c, gx_s, 2e-6)
    assert_close(gw_c, ops.convtree_bwd_w(gd, xd, wd, sd, amax, geom, W_SOFTMAX), 2e-5)
    gx_2, gw_2 = ops.convtree_bwd(gd, xd, wd, sd, amax, geom, W_SOFTMAX)
    assert torch.equal(gx_2, gx_c) and torch.equal(gw_2, gw_c)
    gx_only, none = ops.convtree_bwd(gd, xd, wd, sd, amax, geom, W_SOFTMAX, need_gw=False)
    assert none is None and torch.equal(gx_only, gx_c)
    if x.shape[0] <= 40 and shape[2] <= 64:
        xo = x.clone().requires_grad_(True)
        yo, _, _, idxo = oracle.full_convlogic(xo, oracle.gate_probabilities(logits, True), sel, geom[0:2], geom[2:4], geom[4:6])
        idx = ops.convtree_fwd(xd, wd, sd, geom, W_SOFTMAX, want_indices=True)[4].cpu()
        assert_same_argmax_up_to_ties(idx, idxo, 1e-3)
        wo = logits.clone().requires_grad_(True)
        yf = oracle.full_convlogic(xo, oracle.gate_probabilities(wo, True), sel, geom[0:2], geom[2:4], geom[4:6], forced_idx=idx)[0]
        gxf, gwf = torch.autograd.grad((yf * gy).sum(), (xo, wo))
        assert_close(gx_c, gxf, F32_TOL, "gx at the kernels' own arg-max")
        assert_close(gw_c, gwf, F32_TOL, "gw at the kernels' own arg-max")
