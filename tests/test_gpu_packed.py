"""Packed (bit-level) inference on the GPU: bit-exact against the numpy oracle and against the
eval-mode float path of the same layers."""

import numpy as np
import pytest
import torch

import oracle
from tests.util import random_selection

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [8, 16, 32, 64])
@pytest.mark.parametrize("batch,feat", [(1, 3), (70, 33), (256, 40), (1000, 7)])
def test_pack_bits_and_group_sum(bits, batch, feat):
    import convlogic_b200 as cb
    from convlogic_b200 import ops

    rng = np.random.default_rng(batch + bits)
    xb = rng.random((batch, feat * 4)) < 0.4
    want, pad = oracle.pack_bits(xb.T, bits)
    p = cb.PackBitsTensor(torch.from_numpy(xb).cuda(), bits)
    assert p.pad_len == pad and p.t.dtype == torch.from_numpy(want).dtype
    assert np.array_equal(p.t.cpu().numpy(), want)
    got2, pad2 = ops.pack_bits(torch.from_numpy(np.ascontiguousarray(xb.T)).cuda(), bits)  # the reference's [F, B] layout
    assert pad2 == pad and np.array_equal(got2.cpu().numpy(), want)
    counts = p.group_sum(4)
    assert counts.dtype == torch.int32 and counts.shape == (batch, 4)
    assert np.array_equal(counts.cpu().numpy(), oracle.packed_group_sum(want, pad, 4))
    with pytest.raises(ValueError):
        p.group_sum(feat * 4 + 1)


def test_group_sum_many_rows_uses_row_splits():
    import convlogic_b200 as cb

    rng = np.random.default_rng(0)
    xb = rng.random((96, 10 * 700)) < 0.5
    p = cb.PackBitsTensor(torch.from_numpy(xb).cuda(), 64)
    want = xb.reshape(96, 10, 700).sum(-1).astype(np.int32)
    for _ in range(2):
        assert np.array_equal(cb.GroupSum(10)(p).cpu().numpy(), want)


@pytest.mark.parametrize("bits", [8, 32, 64])
@pytest.mark.parametrize("batch", [5, 64, 130, 1024])
def test_packed_logic_layer(bits, batch):
    import convlogic_b200 as cb

    torch.manual_seed(batch)
    rng = np.random.default_rng(batch)
    layer = cb.LogicLayer(24, 60).cuda().eval()
    xb = rng.random((batch, 24)) < 0.5
    p = cb.PackBitsTensor(torch.from_numpy(xb).cuda(), bits)
    y = layer(p)
    want = oracle.packed_logic(oracle.pack_bits(xb.T, bits)[0], layer.indices_0.cpu().numpy(), layer.indices_1.cpu().numpy(),
                               layer.weights.argmax(-1).cpu().numpy().astype(np.uint8))
    # pad bits of the oracle's output may be set by negating gates; compare real samples only
    assert np.array_equal(oracle.unpack_bits(y.t.cpu().numpy(), batch), oracle.unpack_bits(want, batch))
    with torch.no_grad():
        yf = layer(torch.from_numpy(xb).float().cuda())
    assert np.array_equal(oracle.unpack_bits(y.t.cpu().numpy(), batch).T.astype(np.float32), yf.cpu().numpy())


@pytest.mark.parametrize("bits,batch", [(64, 70), (64, 256), (32, 33), (8, 9)])
@pytest.mark.parametrize("geom", [(3, 6, 8, 8, 1, 1, 3), (1, 4, 12, 12, 1, 0, 5), (5, 3, 6, 10, 2, 2, 4)])
def test_packed_conv_block(bits, batch, geom):
    import convlogic_b200 as cb

    ci, c, h, w, st, pd, k = geom
    rng = np.random.default_rng(bits + batch)
    torch.manual_seed(bits + batch)
    sel = random_selection(rng, c, ci, k, k)
    layer = cb.ConvLogicLayer(ci, c, stride=st, padding=pd, kernel=k, selection=sel, complete=True).cuda().eval()
    xb = rng.random((batch, ci, h, w)) < 0.5
    p = cb.PackBitsTensor(torch.from_numpy(xb).cuda(), bits)
    assert p.t.shape[:3] == (ci, h, w)
    y = layer(p)
    want = oracle.packed_convtree(oracle.pack_bits(xb.reshape(batch, -1).T, bits)[0].reshape(ci, h, w, -1),
                                  layer.weights.argmax(-1).cpu().numpy().astype(np.uint8), sel.numpy(), st, pd, k)
    assert y.slab == (st == 1 and (batch + bits - 1) // bits * bits % 128 == 0)
    got = oracle.unpack_bits(y.rows().cpu().numpy(), batch)
    assert np.array_equal(got, oracle.unpack_bits(want, batch))
    with torch.no_grad():
        yf = layer(torch.from_numpy(xb).float().cuda())
    assert np.array_equal(np.moveaxis(got, -1, 0).astype(np.float32), yf.cpu().numpy())


@pytest.mark.parametrize("geom", [(3, 40, 32, 32, 1, 3), (16, 24, 16, 16, 1, 3), (24, 16, 8, 8, 1, 3), (7, 5, 14, 10, 0, 5),
                                  (2, 9, 6, 6, 2, 3), (5, 7, 4, 4, 1, 3), (3, 3, 2, 2, 1, 3)])
@pytest.mark.parametrize("batch", [128, 1000])
def test_packed_conv_block_slab_layout_equals_rows_layout(geom, batch):
    """The slab-layout kernel (staged channel planes, and its global-gather path when a window's taps span
    more channels than are staged) gives the very words of the rows-layout kernel; layout round trip is exact."""
    from convlogic_b200 import ops

    ci, c, h, w, pd, k = geom
    rng = np.random.default_rng(ci * 1000 + batch)
    sel = random_selection(rng, c, ci, k, k).cuda()
    gate_ids = torch.from_numpy(rng.integers(0, 16, (c, 7)).astype(np.uint8)).cuda()
    words = (batch + 63) // 64
    words += words % 2
    x = torch.from_numpy(rng.integers(-2**63, 2**63 - 1, (ci, h, w, words), dtype=np.int64)).cuda()
    slab = ops.packed_to_slab(x)
    assert slab.shape == (ci, words // 2, h, w, 2)
    assert torch.equal(ops.packed_to_rows(slab), x)
    g = (1, 1, pd, pd, k, k)
    want = ops.packed_convtree(x, gate_ids, sel, g)
    got = ops.packed_convtree_slab(slab, gate_ids, sel, g)
    assert torch.equal(ops.packed_to_rows(got), want)
    ref = oracle.packed_convtree(x.cpu().numpy(), gate_ids.cpu().numpy(), sel.cpu().numpy(), 1, pd, k)
    assert np.array_equal(want.cpu().numpy(), ref)


def test_packed_slab_rejects_what_it_does_not_cover():
    from convlogic_b200 import ops

    rng = np.random.default_rng(0)
    sel = random_selection(rng, 4, 3, 3, 3).cuda()
    gate_ids = torch.zeros(4, 7, dtype=torch.uint8).cuda()
    slab = torch.zeros(3, 1, 8, 8, 2, dtype=torch.int64).cuda()
    with pytest.raises(Exception):
        ops.packed_convtree_slab(slab, gate_ids, sel, (2, 2, 1, 1, 3, 3))   # stride 2
    big = torch.zeros(3, 1, 36, 36, 2, dtype=torch.int64).cuda()
    with pytest.raises(Exception):
        ops.packed_convtree_slab(big, gate_ids, sel, (1, 1, 1, 1, 3, 3))    # 18*18 pooled outputs > 256
    assert ops.packed_to_slab(torch.zeros(3, 4, 4, 3, dtype=torch.int64).cuda()) is None


def test_packed_model_equals_float_eval_model():
    """A whole (small) CIFAR-shaped stack: packed class counts == tau * float eval-mode scores
    (tau a power of two, so the division is exact)."""
    import convlogic_b200 as cb

    torch.manual_seed(0)
    net = cb.ConvLogicCifarModel(k_param=4, input_channels=6, input_size=32, tau=8.0).cuda().eval()
    for prm in net.parameters():
        prm.data = torch.randn_like(prm)
    x = torch.rand(100, 6, 32, 32, device="cuda") < 0.5
    with torch.no_grad():
        scores = net(x.float())
        counts = net(cb.PackBitsTensor(x, 64))
    assert counts.dtype == torch.int32 and counts.shape == (100, 10)
    assert torch.equal(counts.float(), scores * 8.0)


@pytest.mark.parametrize("n,cp,h,w,levels", [(70, 3, 8, 8, 31), (256, 3, 32, 32, 31), (300, 1, 5, 7, 3), (128, 2, 4, 4, 40), (1, 3, 2, 2, 1)])
@pytest.mark.parametrize("u8", [False, True])
def test_thermometer_pack_equals_transform_then_pack(n, cp, h, w, levels, u8):
    """Fused thermometer + pack == the reference's input transform (cat of x > t, threshold-major) followed by
    PackBitsTensor, bit for bit, in the rows layout and (when the batch fills 128-sample units) the slab layout."""
    import convlogic_b200 as cb
    from convlogic_b200 import ops

    rng = np.random.default_rng(n * 7 + levels)
    th = (np.arange(1, levels + 1, dtype=np.float32) / np.float32(levels + 1))
    if u8:
        raw = rng.integers(0, 256, (n, cp, h, w), dtype=np.uint8)
        # make sure values sitting exactly on a threshold occur (k/255 vs i/(L+1))
        pix = torch.from_numpy(raw)
        val = (pix.float() / 255).numpy()  # ToTensor's arithmetic
    else:
        val = rng.random((n, cp, h, w), dtype=np.float32)
        val.reshape(-1)[: levels] = th  # equality with a threshold: strict '>' must give 0
        pix = torch.from_numpy(val)
    bits = oracle.thermometer(val, levels)                      # [n, levels*cp, h, w] bool
    want, pad = oracle.pack_bits(bits.reshape(n, -1).T, 64)     # [F, words]
    want = want.reshape(levels * cp, h, w, -1)
    got, pad_g = ops.thermometer_pack(pix.cuda(), torch.from_numpy(th).cuda())
    assert pad_g == pad and np.array_equal(got.cpu().numpy(), want)
    p = cb.PackBitsTensor.from_pixels(pix.cuda(), torch.from_numpy(th).cuda())
    assert p.pad_len == pad and np.array_equal(p.rows().cpu().numpy(), want)
    assert p.slab == (want.shape[-1] % 2 == 0)
    if want.shape[-1] % 2:
        with pytest.raises(RuntimeError):
            ops.thermometer_pack(pix.cuda(), torch.from_numpy(th).cuda(), slab=True)


def test_cached_gate_ids_follow_the_logits():
    """Packed inference caches the arg-max gate ids; an in-place update, a re-assignment of .data and a
    train()/eval() round trip must each be seen."""
    import convlogic_b200 as cb

    torch.manual_seed(1)
    layer = cb.LogicLayer(64, 80).cuda().eval()
    x = torch.rand(130, 64, device="cuda") < 0.5

    def run():
        y = layer(cb.PackBitsTensor(x, 64))
        with torch.no_grad():
            want = layer(x.float())
        got = oracle.unpack_bits(y.t.cpu().numpy(), 130).T.astype(np.float32)
        assert np.array_equal(got, want.cpu().numpy())
        return got

    a = run()
    with torch.no_grad():
        layer.weights.copy_(torch.randn_like(layer.weights))     # in place: version changes
    b = run()
    layer.weights.data = torch.randn_like(layer.weights)          # new storage
    c = run()
    layer.train()
    layer.weights.data.copy_(torch.randn_like(layer.weights))     # invisible to the version counter ...
    layer.eval()                                                  # ... but train()/eval() drops the cache
    d = run()
    assert not np.array_equal(a, b) and not np.array_equal(b, c) and not np.array_equal(c, d)
