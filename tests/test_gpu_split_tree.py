"""Stand-alone first gate level, TreeLogicLayer and the split-vs-fused identity on the GPU."""

import numpy as np
import pytest
import torch

import oracle
from tests.util import assert_close, random_selection

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.mark.parametrize("j", [0, 1])
def test_split_layers_match_reference_golden(golden, j):
    import convlogic_b200 as cb

    g = golden("split_layers")
    sh, sw, ph, pw, kh, kw = (int(v) for v in g[f"split{j}/geom"])
    sel = torch.from_numpy(g[f"split{j}/selection"])
    conv = cb.ConvLogicLayer(3, 2, stride=sh, padding=ph, kernel=kh, selection=sel, complete=False).cuda()
    t1 = cb.TreeLogicLayer(2, 4).cuda()
    t2 = cb.TreeLogicLayer(2, 2).cuda()
    conv.weights.data = torch.from_numpy(g[f"split{j}/conv_logits"]).cuda()
    t1.weights.data = torch.from_numpy(g[f"split{j}/tree1_logits"]).cuda()
    t2.weights.data = torch.from_numpy(g[f"split{j}/tree2_logits"]).cuda()
    pool = cb.PoolLogicLayer(return_indices=True)
    x = torch.from_numpy(g[f"split{j}/x"]).cuda().requires_grad_(True)
    for mode in ("soft", "hard"):
        for m in (conv, t1, t2):
            m.train(mode == "soft")
        x1 = conv(x)
        x2 = t1(x1)
        x3 = t2(x2)
        y, idx = pool(x3)
        pre = f"split{j}/{mode}"
        assert_close(x1, g[f"{pre}/x1"], TOL, "conv")
        assert_close(x2, g[f"{pre}/x2"], TOL, "tree1")
        assert_close(x3, g[f"{pre}/x3"], TOL, "tree2")
        assert_close(y, g[f"{pre}/y"], TOL, "pool")
        assert np.array_equal(idx.flatten(2).cpu().numpy(), g[f"{pre}/idx"])
        if mode == "soft":
            gx, gw = torch.autograd.grad((x1 * torch.from_numpy(g[f"split{j}/g_x1"]).cuda()).sum(), (x, conv.weights),
                                         retain_graph=True)
            assert_close(gx, g[f"split{j}/conv_gx"], TOL, "conv gx")
            assert_close(gw, g[f"split{j}/conv_gw_logits"], TOL, "conv gw")
            x1d = x1.detach().requires_grad_(True)
            gx1, gwt = torch.autograd.grad((t1(x1d) * torch.from_numpy(g[f"split{j}/g_x2"]).cuda()).sum(), (x1d, t1.weights))
            assert_close(gx1, g[f"split{j}/tree_gx"], TOL, "tree gx")
            assert_close(gwt, g[f"split{j}/tree_gw_logits"], TOL, "tree gw")


@pytest.mark.parametrize("stride,pad", [(1, 1), (2, 2)])
def test_split_layers_vs_complete_block(stride, pad):
    """The reference's fused-vs-split test (tests/convlogic/test_full_convlogic_forward.py:165-233)."""
    import convlogic_b200 as cb

    torch.manual_seed(0)
    full = cb.ConvLogicLayer(3, 2, stride=stride, padding=pad, kernel=3, complete=True, return_indices=True,
                             return_intermediate=True).cuda()
    conv = cb.ConvLogicLayer(3, 2, stride=stride, padding=pad, kernel=3, complete=False).cuda()
    t1, t2 = cb.TreeLogicLayer(2, 4).cuda(), cb.TreeLogicLayer(2, 2).cuda()
    pool = cb.PoolLogicLayer(return_indices=True)
    conv.selection = full.selection
    conv.weights.data.copy_(full.weights[:, 0:4])
    t1.weights.data.copy_(full.weights[:, 4:6])
    t2.weights.data.copy_(full.weights[:, 6:7])
    x = torch.randn(4, 3, 10, 10, device="cuda")
    with torch.no_grad():
        y_full, x1_full, x2_full, idx_full = full(x)
        x1 = conv(x)
        x2 = t1(x1)
        y, idx = pool(t2(x2))
    assert torch.equal(idx.flatten(2).to(torch.int32), idx_full)
    assert torch.allclose(x1, x1_full, atol=1e-6)
    assert torch.allclose(x2, x2_full, atol=1e-6)
    assert torch.allclose(y, y_full, atol=1e-6)


def test_all_logic_gates_tree():
    """Known-answer test of the 16 gates (tests/convlogic/test_treelogic_forward.py:66-86)."""
    import convlogic_b200 as cb

    for gate in range(16):
        layer = cb.TreeLogicLayer(1, 2).cuda().eval()
        w = torch.full((1, 1, 16), -float("inf"))
        w[..., gate] = 0.0
        layer.weights.data = w.cuda()
        for a in (0.0, 1.0):
            for b in (0.0, 1.0):
                y = layer(torch.tensor([a, b], device="cuda").view(1, 1, 1, 1, 2))
                want = oracle.bin_op(torch.tensor(a), torch.tensor(b), gate)
                assert torch.equal(y.cpu().view(()), want), (gate, a, b)


@pytest.mark.parametrize("n,c,h,w,xo", [(2, 3, 5, 4, 2), (1, 2, 3, 3, 1), (3, 2, 2, 2, 8), (2, 1, 40, 33, 4)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float64, 1e-10)])
def test_tree_layer_matches_oracle(n, c, h, w, xo, dtype, tol):
    from convlogic_b200 import TreeLogicFunction

    g = torch.Generator().manual_seed(1)
    x = torch.rand(n, c, h, w, 2 * xo, generator=g, dtype=dtype)
    p = torch.softmax(torch.randn(c, xo, 16, generator=g, dtype=dtype), -1)
    gy = torch.randn(n, c, h, w, xo, generator=g, dtype=dtype)
    xo_, po = x.clone().requires_grad_(True), p.clone().requires_grad_(True)
    yo = oracle.tree_stage(xo_, po)
    gxo, gpo = torch.autograd.grad((yo * gy).sum(), (xo_, po))
    xd, pd = x.cuda().requires_grad_(True), p.cuda().requires_grad_(True)
    y = TreeLogicFunction.apply(xd, pd)
    gx, gp = torch.autograd.grad((y * gy.cuda()).sum(), (xd, pd))
    assert_close(y, yo.detach(), tol)
    assert_close(gx, gxo, tol)
    assert_close(gp, gpo, tol)


@pytest.mark.parametrize("shape", [(4, 3, 6, 9, 9, (1, 1), (1, 1), (3, 3)), (2, 5, 4, 8, 11, (2, 1), (0, 2), (2, 4))])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float64, 1e-10)])
def test_split_conv_matches_oracle(shape, dtype, tol):
    from convlogic_b200 import ConvLogicFunction

    n, ci, c, h, w, st, pd_, k = shape
    rng = np.random.default_rng(2)
    g = torch.Generator().manual_seed(2)
    sel = random_selection(rng, c, ci, *k)
    x = torch.randn(n, ci, h, w, generator=g, dtype=dtype)
    p = torch.softmax(torch.randn(c, 4, 16, generator=g, dtype=dtype), -1)
    xo_, po = x.clone().requires_grad_(True), p.clone().requires_grad_(True)
    yo = oracle.conv_stage(xo_, po, sel, st, pd_, k)
    gy = torch.randn(*yo.shape, generator=g, dtype=dtype)
    gxo, gpo = torch.autograd.grad((yo * gy).sum(), (xo_, po))
    xd, pdv = x.cuda().requires_grad_(True), p.cuda().requires_grad_(True)
    y = ConvLogicFunction.apply(xd, pdv, sel.cuda(), *st, *pd_, *k)
    gx, gp = torch.autograd.grad((y * gy.cuda()).sum(), (xd, pdv))
    assert_close(y, yo.detach(), tol)
    assert_close(gx, gxo, tol)
    assert_close(gp, gpo, tol)


def test_pool_layer_matches_max_pool2d():
    import convlogic_b200 as cb

    x = torch.randn(2, 3, 8, 8, device="cuda")
    assert torch.equal(cb.PoolLogicLayer()(x), torch.nn.functional.max_pool2d(x, 2, 2))
    assert torch.equal(cb.PoolLogicLayer()(x.unsqueeze(-1)), torch.nn.functional.max_pool2d(x, 2, 2))
    with pytest.raises(ValueError):
        cb.PoolLogicLayer()(torch.randn(2, 3, 8, 8, 2, device="cuda"))
    with pytest.raises(ValueError):
        cb.PoolLogicLayer()(torch.randn(8, 8, device="cuda"))
