"""Pin the CPU oracle to tensors produced by the reference's own CPU path.

The golden files were written by tests/golden/make_golden.py, which runs the reference's
``implementation="python"`` layers; here the oracle must reproduce them.
"""

import numpy as np
import pytest
import torch

import oracle
from tests.golden.make_golden import FUSED_CASES

F64_TOL = dict(rtol=1e-10, atol=1e-12)
F32_TOL = dict(rtol=1e-5, atol=1e-6)


def _t(a, dtype=None):
    t = torch.from_numpy(np.asarray(a))
    return t.to(dtype) if dtype is not None else t


@pytest.mark.parametrize("name", [c[0] for c in FUSED_CASES])
@pytest.mark.parametrize("tag,dtype", [("f64", torch.float64), ("f32", torch.float32)])
def test_fused_block_matches_reference(golden, name, tag, dtype):
    g = golden("fused_block")
    tol = F64_TOL if tag == "f64" else F32_TOL
    sh, sw, ph, pw, kh, kw = (int(v) for v in g[f"{name}/geom"])
    x = _t(g[f"{name}/x"], dtype).requires_grad_(True)
    logits = _t(g[f"{name}/logits"], dtype).requires_grad_(True)
    sel = _t(g[f"{name}/selection"])
    gy = _t(g[f"{name}/gy"], dtype)
    y, _, _, _ = oracle.full_convlogic(x, oracle.gate_probabilities(logits, True), sel, (sh, sw), (ph, pw), (kh, kw))
    gx, gw = torch.autograd.grad((y * gy).sum(), (x, logits))
    np.testing.assert_allclose(y.detach().numpy(), g[f"{name}/{tag}/y_soft"], **tol)
    np.testing.assert_allclose(gx.numpy(), g[f"{name}/{tag}/gx"], **tol)
    np.testing.assert_allclose(gw.numpy(), g[f"{name}/{tag}/gw_logits"], **tol)
    with torch.no_grad():
        yh = oracle.full_convlogic(x, oracle.gate_probabilities(logits, False), sel, (sh, sw), (ph, pw), (kh, kw))[0]
    if "bits" in name:  # one-hot gates on {0,1} inputs are exact in every formulation
        assert np.array_equal(yh.numpy(), g[f"{name}/{tag}/y_hard"])
        assert set(np.unique(yh.numpy())) <= {0.0, 1.0}
    else:
        np.testing.assert_allclose(yh.numpy(), g[f"{name}/{tag}/y_hard"], **tol)


@pytest.mark.parametrize("j", [0, 1])
def test_split_layers_match_reference(golden, j):
    g = golden("split_layers")
    sh, sw, ph, pw, kh, kw = (int(v) for v in g[f"split{j}/geom"])
    x = _t(g[f"split{j}/x"]).requires_grad_(True)
    sel = _t(g[f"split{j}/selection"])
    lc = _t(g[f"split{j}/conv_logits"]).requires_grad_(True)
    l1 = _t(g[f"split{j}/tree1_logits"]).requires_grad_(True)
    l2 = _t(g[f"split{j}/tree2_logits"])
    for mode in ("soft", "hard"):
        tr = mode == "soft"
        x1 = oracle.conv_stage(x, oracle.gate_probabilities(lc, tr), sel, (sh, sw), (ph, pw), (kh, kw))
        x2 = oracle.tree_stage(x1, oracle.gate_probabilities(l1, tr))
        x3 = oracle.tree_stage(x2, oracle.gate_probabilities(l2, tr))
        y, idx = oracle.pool_first_max(x3[..., 0])
        pre = f"split{j}/{mode}"
        np.testing.assert_allclose(x1.detach().numpy(), g[f"{pre}/x1"], **F32_TOL)
        np.testing.assert_allclose(x2.detach().numpy(), g[f"{pre}/x2"], **F32_TOL)
        np.testing.assert_allclose(x3.detach().numpy(), g[f"{pre}/x3"], **F32_TOL)
        np.testing.assert_allclose(y.detach().numpy(), g[f"{pre}/y"], **F32_TOL)
        assert np.array_equal(idx.numpy(), g[f"{pre}/idx"])
        if tr:
            gx, gw = torch.autograd.grad((x1 * _t(g[f"split{j}/g_x1"])).sum(), (x, lc), retain_graph=True)
            np.testing.assert_allclose(gx.numpy(), g[f"split{j}/conv_gx"], **F32_TOL)
            np.testing.assert_allclose(gw.numpy(), g[f"split{j}/conv_gw_logits"], **F32_TOL)
            x1d = x1.detach().requires_grad_(True)
            x2b = oracle.tree_stage(x1d, oracle.gate_probabilities(l1, True))
            gx1, gwt = torch.autograd.grad((x2b * _t(g[f"split{j}/g_x2"])).sum(), (x1d, l1))
            np.testing.assert_allclose(gx1.numpy(), g[f"split{j}/tree_gx"], **F32_TOL)
            np.testing.assert_allclose(gwt.numpy(), g[f"split{j}/tree_gw_logits"], **F32_TOL)


@pytest.mark.parametrize("j", [0, 1, 2])
def test_flat_layer_matches_reference(golden, j):
    g = golden("flat_layers")
    pre = f"flat{j}"
    x = _t(g[f"{pre}/x"]).requires_grad_(True)
    logits = _t(g[f"{pre}/logits"]).requires_grad_(True)
    a, b = _t(g[f"{pre}/a"]), _t(g[f"{pre}/b"])
    k, tau = g[f"{pre}/k_tau"]
    y = oracle.logic_layer(x, a, b, oracle.gate_probabilities(logits, True))
    gx, gw = torch.autograd.grad((y * _t(g[f"{pre}/gy"])).sum(), (x, logits), retain_graph=True)
    np.testing.assert_allclose(y.detach().numpy(), g[f"{pre}/y_soft"], **F32_TOL)
    np.testing.assert_allclose(gx.numpy(), g[f"{pre}/gx"], **F32_TOL)
    np.testing.assert_allclose(gw.numpy(), g[f"{pre}/gw_logits"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(oracle.group_sum(y, int(k), float(tau)).detach().numpy(), g[f"{pre}/group_sum"], **F32_TOL)
    yh = oracle.logic_layer(x.detach(), a, b, oracle.gate_probabilities(logits.detach(), False))
    np.testing.assert_allclose(yh.numpy(), g[f"{pre}/y_hard"], **F32_TOL)
    if j == 0:
        assert np.array_equal(yh.numpy(), g[f"{pre}/y_hard"])


def test_truth_table_known_answers(golden):
    """The reference tests' known-answer vector: each gate on inputs 00, 01, 10, 11."""
    table = golden("flat_layers")["truth_table"]
    a = torch.tensor([0.0, 0.0, 1.0, 1.0])
    b = torch.tensor([0.0, 1.0, 0.0, 1.0])
    ai = np.array([0, 0, 1, 1], dtype=np.int64)
    bi = np.array([0, 1, 0, 1], dtype=np.int64)
    for i in range(16):
        assert np.array_equal(oracle.bin_op(a, b, i).numpy(), table[i])
        assert np.array_equal(oracle.bin_op_bits(ai, bi, i) & 1, table[i].astype(np.int64))
        assert list(table[i]) == [float(v) for v in oracle.logic_ops.TRUTH[i]]
    # the 4-term basis reproduces every gate
    basis = torch.stack([a * b, a, b, torch.ones(4)]).numpy()
    assert np.array_equal((oracle.COEFS_T.T @ basis), table)


def test_coefs_equal_reference_table():
    ref = np.array([[0, 1, -1, 0, -1, 0, -2, -1, 1, 2, 0, 1, 0, 1, -1, 0],
                    [0, 0, 1, 1, 0, 0, 1, 1, -1, -1, 0, 0, -1, -1, 0, 0],
                    [0, 0, 0, 0, 1, 1, 1, 1, -1, -1, -1, -1, 0, 0, 0, 0],
                    [0, 0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 1, 1, 1, 1, 1]])
    assert np.array_equal(oracle.COEFS_T, ref)


def test_packed_path_equals_hard_float_path():
    """Packed inference has no reference-side test; it is defined by the eval-mode float path."""
    rng = np.random.default_rng(0)
    g = torch.Generator().manual_seed(0)
    n, ci, c, h, w = 70, 3, 5, 8, 8
    xb = rng.random((n, ci, h, w)) < 0.5
    logits = torch.randn(c, 7, 16, generator=g)
    sel = torch.from_numpy(((rng.integers(0, ci, (c, 8)) << 16) | (rng.integers(0, 3, (c, 8)) << 8)
                            | rng.integers(0, 3, (c, 8))).astype(np.int32))
    yf = oracle.full_convlogic(torch.from_numpy(xb).float(), oracle.gate_probabilities(logits, False), sel)[0]
    for bits in (8, 32, 64):
        xp, pad = oracle.pack_bits(xb.reshape(n, -1).T, bits)
        assert pad == (bits - n % bits) % bits
        assert np.array_equal(oracle.unpack_bits(xp, n), xb.reshape(n, -1).T)
        yp = oracle.packed_convtree(xp.reshape(ci, h, w, -1), logits.argmax(-1).numpy().astype(np.uint8), sel.numpy())
        got = oracle.unpack_bits(yp, n)  # [C, Hp, Wp, n]
        assert np.array_equal(np.moveaxis(got, -1, 0).astype(np.float32), yf.numpy())
    # flat layer + group sum
    in_dim, out_dim, k = 24, 60, 10
    a = rng.integers(0, in_dim, out_dim)
    b = rng.integers(0, in_dim, out_dim)
    fl = torch.randn(out_dim, 16, generator=g)
    xf = rng.random((n, in_dim)) < 0.5
    y = oracle.logic_layer(torch.from_numpy(xf).float(), torch.from_numpy(a), torch.from_numpy(b),
                           oracle.gate_probabilities(fl, False))
    xp, pad = oracle.pack_bits(xf.T, 64)
    yp = oracle.packed_logic(xp, a, b, fl.argmax(-1).numpy().astype(np.uint8))
    assert np.array_equal(oracle.unpack_bits(yp, n).T.astype(np.float32), y.numpy())
    counts = oracle.packed_group_sum(yp, pad, k)
    assert counts.dtype == np.int32 and counts.shape == (n, k)
    assert np.array_equal(counts, oracle.group_sum(y, k, 1.0).numpy().astype(np.int32))
    with pytest.raises(ValueError):
        oracle.packed_group_sum(yp, pad, 7)


def test_inverse_connections_lists_consumers_in_neuron_order():
    a = np.array([2, 0, 2, 1]); b = np.array([1, 2, 2, 0])
    start, cons = oracle.inverse_connections(a, b, 3)
    assert start.tolist() == [0, 2, 4, 8]
    assert cons.tolist() == [1, 3, 0, 3, 0, 1, 2, 2]


def test_thermometer_thresholds():
    px = np.array([[[[0.0, 1 / 32, 0.5, 31.5 / 32]]]], dtype=np.float32).repeat(3, 1)
    t = oracle.thermometer(px, 31)
    assert t.shape == (1, 93, 1, 4)
    assert t[0, :, 0, 0].sum() == 0 and t[0, 0:3, 0, 1].sum() == 0  # strict '>'
    assert t[0, :, 0, 2].sum() == 3 * 15 and t[0, :, 0, 3].sum() == 93


def test_mnist_s_stack_matches_reference_scores(golden):
    """The oracle, assembled into the mnist_s-shaped stack, reproduces the class scores the
    reference's CPU path gave for the same seeded network (first 24 of the 256 images)."""
    from tests.golden.make_golden import mnist_inputs

    g = golden("mnist_s")
    gen = torch.Generator().manual_seed(1)
    k, n = 16, 24
    conv_shapes = [(k, 7, 16), (3 * k, 7, 16), (9 * k, 7, 16)]
    flat_shapes = [(1280 * k, 16), (640 * k, 16), (320 * k, 16)]
    logits = [torch.randn(*s, generator=gen) for s in conv_shapes + flat_shapes]
    np.testing.assert_allclose([float(w.double().sum()) for w in logits], g["logit_checksum"], rtol=1e-12)
    x0 = mnist_inputs()[:n]
    for training, key in ((True, "scores_soft"), (False, "scores_hard")):
        x = x0
        for i, (kern, pad) in enumerate([(5, 0), (3, 1), (3, 1)]):
            x = oracle.full_convlogic(x, oracle.gate_probabilities(logits[i], training),
                                      torch.from_numpy(g[f"conv{i}/selection"]), 1, pad, kern)[0]
        x = x.flatten(1)
        for i in range(3):
            x = oracle.logic_layer(x, torch.from_numpy(g[f"flat{i}/a"]), torch.from_numpy(g[f"flat{i}/b"]),
                                   oracle.gate_probabilities(logits[3 + i], training))
        s = oracle.group_sum(x, 10, 6.5).numpy()
        if training:
            np.testing.assert_allclose(s, g[key][:n], rtol=1e-5, atol=1e-5)
        else:
            assert np.array_equal(s, g[key][:n])


def test_thermometer_restatement_equals_the_transform_expression():
    """The oracle's thermometer == the reference's input transform written out with torch
    (`cat([(x > t).float() for t in thresholds], dim=0)` per image, uniform thresholds i / (L + 1))."""
    import torch

    torch.manual_seed(0)
    for levels, cp in ((31, 3), (3, 1), (1, 2)):
        x = torch.rand(6, cp, 5, 4)
        th = torch.linspace(1, levels, levels, dtype=torch.float32) / (levels + 1)
        x.view(-1)[:levels] = th  # ties: strict '>'
        ref = torch.stack([torch.cat([(xi > t).float() for t in th], dim=0) for xi in x])
        got = oracle.thermometer(x.numpy(), levels)
        assert got.shape == (6, levels * cp, 5, 4)
        assert np.array_equal(ref.numpy().astype(bool), got)
