"""The many-channel fused block on the plane kernels (two channel planes per output channel streamed through shared
memory by TMA loads): forward against the general kernel bit for bit, backward against the CPU oracle at the kernels' own
pooled positions (fp32, 1e-5 max-normalised) and against the older two-pass path, repeatable bit for bit, and the
bounded waits never ran out."""

import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from tests.util import assert_close, assert_same_argmax_up_to_ties

pytestmark = pytest.mark.gpu
GEOM = (1, 1, 1, 1, 3, 3)

# batch, C_in, C_out, side: 16x16 (128 threads per image), 8x8 (a warp per image), 4x4 (four / eight images per warp),
# ragged batches, fewer images than a block's warps, batches that split into several parts
SHAPES = [(37, 64, 24, 16), (33, 128, 20, 8), (130, 600, 10, 4), (1, 70, 9, 16), (3, 200, 9, 8), (5, 500, 9, 4),
          (64, 256, 96, 16), (256, 160, 8, 8)]


def _case(shape, seed):
    import convlogic_b200 as cb

    n, ci, c, side = shape
    torch.manual_seed(seed)
    layer = cb.ConvLogicLayer(ci, c, padding=1, complete=True)   # the reference's generator: two input channels per output channel
    g = torch.Generator().manual_seed(seed + 1)
    logits = torch.randn(c, 7, 16, generator=g)
    x = torch.rand(n, ci, side, side, generator=g)
    gy = torch.randn(n, c, side // 2, side // 2, generator=g)
    return x, logits, layer.selection.clone(), gy


def _plane_error():
    from convlogic_b200 import _lib

    flag = C.c_int(-1)
    _lib.check(_lib.lib().clb_plane_error(C.byref(flag)))
    return flag.value


def _tune(on):
    from convlogic_b200 import _lib

    _lib.check(_lib.lib().clb_tune(_lib.TUNE_PLANE_KERNELS, int(on)))


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(str(v) for v in s))
def test_plane_forward_equals_general_forward(shape):
    from convlogic_b200 import _lib, ops
    from convlogic_b200._lib import W_SOFTMAX

    x, logits, sel, gy = _case(shape, 3)
    xd, wd, sd = x.cuda(), logits.cuda(), sel.cuda()
    _lib.trace(True)
    y, amax, _, _, _ = ops.convtree_fwd(xd, wd, sd, GEOM, W_SOFTMAX)
    torch.cuda.synchronize()
    assert "convtree_fwd_plane_kernel" in _lib.trace_report(), "the plane kernel was expected to take this shape"
    _lib.trace(False)
    y_gen, amax_gen, _, _, idx = ops.convtree_fwd(xd, wd, sd, GEOM, W_SOFTMAX, want_indices=True)
    assert torch.equal(y, y_gen)
    assert torch.equal(amax, amax_gen)
    assert _plane_error() == 0
    if shape[0] <= 40:
        yo = oracle.full_convlogic(x, oracle.gate_probabilities(logits, True), sel)[0]
        assert_close(y, yo, 1e-5)
    try:   # switched off, the older staged kernel serves the same call
        _tune(False)
        y_old, amax_old, _, _, _ = ops.convtree_fwd(xd, wd, sd, GEOM, W_SOFTMAX)
    finally:
        _tune(True)
    assert torch.equal(y_old, y) and torch.equal(amax_old, amax)


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(str(v) for v in s))
def test_plane_backward_against_oracle_and_two_pass_path(shape):
    from convlogic_b200 import _lib, ops
    from convlogic_b200._lib import W_SOFTMAX

    x, logits, sel, gy = _case(shape, 5)
    xd, wd, sd, gd = x.cuda(), logits.cuda(), sel.cuda(), gy.cuda()
    _, amax, _, _, idx = ops.convtree_fwd(xd, wd, sd, GEOM, W_SOFTMAX, want_indices=True)
    _lib.trace(True)
    gx, gw = ops.convtree_bwd(gd, xd, wd, sd, amax, GEOM, W_SOFTMAX)
    torch.cuda.synchronize()
    rep = _lib.trace_report()
    _lib.trace(False)
    assert "convtree_bwd_plane_kernel" in rep and "plane_sum_kernel" in rep, rep
    assert _plane_error() == 0
    gx2, gw2 = ops.convtree_bwd(gd, xd, wd, sd, amax, GEOM, W_SOFTMAX)
    assert torch.equal(gx, gx2) and torch.equal(gw, gw2)   # fixed summation order
    try:
        _tune(False)
        gx_old, gw_old = ops.convtree_bwd(gd, xd, wd, sd, amax, GEOM, W_SOFTMAX)
    finally:
        _tune(True)
    assert_close(gx, gx_old, 2e-6, "gx vs two-pass path")
    assert_close(gw, gw_old, 2e-5, "gw vs two-pass path")
    if shape[0] <= 40:
        xo, wo = x.clone().requires_grad_(True), logits.clone().requires_grad_(True)
        yo, _, _, idxo = oracle.full_convlogic(xo, oracle.gate_probabilities(wo, True), sel)
        assert_same_argmax_up_to_ties(idx, idxo, 1e-3)
        yf = oracle.full_convlogic(xo, oracle.gate_probabilities(wo, True), sel, forced_idx=idx.cpu())[0]
        gxo, gwo = torch.autograd.grad((yf * gy).sum(), (xo, wo))
        assert_close(gx, gxo, 1e-5, "gx vs oracle")
        assert_close(gw, gwo, 1e-5, "gw vs oracle")


def test_selection_with_one_channel_and_with_many_channels():
    """All eight taps in ONE channel (slot 1 unused) runs on the plane kernels; more than two channels per output
    channel does not fit two planes: the forward kernel gathers from global memory, the backward falls back."""
    import convlogic_b200 as cb
    from convlogic_b200 import ops
    from convlogic_b200._lib import W_SOFTMAX
    from tests.util import random_selection

    g = torch.Generator().manual_seed(0)
    n, ci, c, side = 9, 40, 6, 8
    x = torch.rand(n, ci, side, side, generator=g)
    logits = torch.randn(c, 7, 16, generator=g)
    gy = torch.randn(n, c, side // 2, side // 2, generator=g)
    rng = np.random.default_rng(1)
    one = torch.from_numpy(((rng.integers(0, ci, (c, 1)) << 16) | (rng.integers(0, 3, (c, 8)) << 8) | rng.integers(0, 3, (c, 8))).astype(np.int32))
    many = random_selection(rng, c, ci, 3, 3)
    for sel in (one, many):
        xd, wd, sd, gd = x.cuda(), logits.cuda(), sel.cuda(), gy.cuda()
        y, amax, _, _, _ = ops.convtree_fwd(xd, wd, sd, GEOM, W_SOFTMAX)
        idx = ops.convtree_fwd(xd, wd, sd, GEOM, W_SOFTMAX, want_indices=True)[4].cpu()
        gx, gw = ops.convtree_bwd(gd, xd, wd, sd, amax, GEOM, W_SOFTMAX)
        xo, wo = x.clone().requires_grad_(True), logits.clone().requires_grad_(True)
        yf = oracle.full_convlogic(xo, oracle.gate_probabilities(wo, True), sel, forced_idx=idx)[0]
        gxo, gwo = torch.autograd.grad((yf * gy).sum(), (xo, wo))
        assert_close(y, yf.detach(), 1e-5)
        assert_close(gx, gxo, 1e-5)
        assert_close(gw, gwo, 1e-5)
    assert _plane_error() == 0


@pytest.mark.parametrize("n,ci,c", [(20, 9, 24), (3, 3, 5), (67, 9, 8)])
def test_gate_gradient_alone_of_a_32x32_block(n, ci, c):
    """A first block (32x32 images) whose input needs no gradient: the gate gradient on the plane kernel against the CPU
    oracle at the kernels' own pooled positions, against the combined tiled kernel, and bit-identical when repeated."""
    from convlogic_b200 import _lib, ops
    from convlogic_b200._lib import W_SOFTMAX

    x, logits, sel, gy = _case((n, ci, c, 32), 7)
    x = (x < 0.5).float()
    xd, wd, sd, gd = x.cuda(), logits.cuda(), sel.cuda(), gy.cuda()
    _, amax, _, _, idx = ops.convtree_fwd(xd, wd, sd, GEOM, W_SOFTMAX, want_indices=True)
    _lib.trace(True)
    none, gw = ops.convtree_bwd(gd, xd, wd, sd, amax, GEOM, W_SOFTMAX, need_gx=False)
    torch.cuda.synchronize()
    rep = _lib.trace_report()
    _lib.trace(False)
    assert none is None and "convtree_bwd_w_plane32_kernel" in rep, rep
    assert _plane_error() == 0
    assert torch.equal(gw, ops.convtree_bwd(gd, xd, wd, sd, amax, GEOM, W_SOFTMAX, need_gx=False)[1])
    _, gw_both = ops.convtree_bwd(gd, xd, wd, sd, amax, GEOM, W_SOFTMAX)   # the tiled kernel that also gives gx
    assert_close(gw, gw_both, 2e-5, "gw vs combined kernel")
    wo = logits.clone().requires_grad_(True)
    yf = oracle.full_convlogic(x, oracle.gate_probabilities(wo, True), sel, forced_idx=idx.cpu())[0]
    (gwo,) = torch.autograd.grad((yf * gy).sum(), (wo,))
    assert_close(gw, gwo, 1e-5, "gw vs oracle")


@pytest.mark.parametrize("shape", [(37, 64, 24, 16), (33, 128, 20, 8), (130, 600, 10, 4), (5, 500, 9, 4)],
                         ids=lambda s: "x".join(str(v) for v in s))
def test_feature_major_output_and_gradient_layout(shape):
    """The plane kernels writing y / reading gy in the flat layers' layout (storage [C, h, w, N]): same values, bit for
    bit, as with the ordinary [N, C, h, w] tensors."""
    from convlogic_b200 import ops
    from convlogic_b200._lib import W_SOFTMAX

    x, logits, sel, gy = _case(shape, 9)
    xd, wd, sd, gd = x.cuda(), logits.cuda(), sel.cuda(), gy.cuda()
    y, amax, _, _, _ = ops.convtree_fwd(xd, wd, sd, GEOM, W_SOFTMAX)
    y_fm, amax_fm, _, _, _ = ops.convtree_fwd(xd, wd, sd, GEOM, W_SOFTMAX, y_feature_major=True)
    assert ops._is_feature_major(y_fm) or shape[0] == 1
    assert torch.equal(y_fm, y) and torch.equal(amax_fm, amax)
    flat = y_fm.flatten(1)
    assert flat.data_ptr() == y_fm.data_ptr() and flat.t().is_contiguous()      # views all the way to [features, batch]
    gx, gw = ops.convtree_bwd(gd, xd, wd, sd, amax, GEOM, W_SOFTMAX)
    gd_fm = gd.permute(1, 2, 3, 0).contiguous().permute(3, 0, 1, 2)            # the same values in feature-major storage
    assert ops._is_feature_major(gd_fm)
    gx2, gw2 = ops.convtree_bwd(gd_fm, xd, wd, sd, amax, GEOM, W_SOFTMAX)
    assert torch.equal(gx, gx2) and torch.equal(gw, gw2)
    assert _plane_error() == 0


def test_block_in_front_of_flat_layers_hands_over_feature_major():
    """fuse_logic_layers marks the block in front of Flatten + flat layers: loss and every gradient equal those of the
    same stack with the ordinary layout, bit for bit, and no transposed copy is launched."""
    import convlogic_b200 as cb
    from convlogic_b200 import _lib

    def build():
        torch.manual_seed(21)
        return torch.nn.Sequential(cb.ConvLogicLayer(64, 40, padding=1, complete=True), torch.nn.Flatten(), cb.LogicLayer(160, 1600),
                                   cb.LogicLayer(1600, 800), cb.LogicLayer(800, 400), cb.GroupSum(10, 2.0)).cuda().train()

    a = cb.fuse_logic_layers(build(), feature_major_blocks=False)
    b = cb.fuse_logic_layers(build())
    assert getattr(b[0], "output_feature_major", False) and not getattr(a[0], "output_feature_major", False)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.rand(48, 64, 4, 4, device="cuda", generator=g)
    lab = torch.randint(0, 10, (48,), device="cuda", generator=g)
    outs = []
    for net in (a, b):
        xi = x.clone().requires_grad_(True)
        _lib.trace(True)
        loss = torch.nn.functional.cross_entropy(net(xi), lab)
        loss.backward()
        torch.cuda.synchronize()
        rep = _lib.trace_report()
        _lib.trace(False)
        outs.append(([loss.detach(), xi.grad] + [p.grad.clone() for p in net.parameters()], rep))
    assert "transpose_f32_kernel" in outs[0][1] and "transpose_f32_kernel" not in outs[1][1], (outs[0][1], outs[1][1])
    for u, v in zip(outs[0][0], outs[1][0]):
        assert torch.equal(u, v)
