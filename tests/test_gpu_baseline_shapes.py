"""Parity at the benchmark configurations' OWN shapes (everything else in the suite uses small shapes).

The checker is the reference's own CUDA extension, compiled unmodified for sm_100a by oracle/build_ref.py
(skipped when it has not been built), in fp32 -- "the reference on identical seeded inputs" -- and in fp64,
where its summation error is negligible, plus the CPU oracle where it finishes in seconds.  Tolerances are
max-normalised (tests/util.py): 1e-5 for fp32 values and gradients.

Size-dependent dispatch of the library (several weight-gradient parts, the two-pass backward and its scratch,
channel-group plans, more than 65535 output rows, slab groups, row offsets beyond 2^31 bytes) only happens at
these sizes.

Arg-max ties: the reference's backward kernels take the pooled positions as an argument, so they are handed
the positions THIS library pooled (after bounding how many differ from the reference's own): every gradient
element is then compared, ties or not.
"""

import numpy as np
import pytest
import torch

import oracle
from oracle.build_ref import load_ref
from tests.util import assert_close, assert_same_argmax_up_to_ties

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def ref_conv():
    m = load_ref("convlogic_cuda")
    if m is None:
        pytest.skip("reference CUDA extension not built (python oracle/build_ref.py --reference ...)")
    return m


@pytest.fixture(scope="module")
def ref_flat():
    m = load_ref("difflogic_cuda")
    if m is None:
        pytest.skip("reference CUDA extension not built (python oracle/build_ref.py --reference ...)")
    return m


def _softmax_jacobian(p, g):
    """Gradient w.r.t. logits from the gradient w.r.t. their soft-max ``p`` (what autograd does in the reference)."""
    p, g = p.double(), g.double()
    return p * (g - (g * p).sum(-1, keepdim=True))


def _reference_block(ref, x, p, sel, idx, gy, dtype):
    """The reference's fused block at ``dtype``: forward, then backward through the given pooled positions."""
    xr, pr, gr = x.to(dtype), p.to(dtype), gy.to(dtype)
    y, x2, x3, idx_r = ref.full_convlogic_forward(xr, pr, sel, 1, 1, 1, 1, 3, 3)
    gx, gx2, gx3 = ref.full_convlogic_backward_x(gr, xr, x2, x3, pr, idx, sel, 1, 1, 1, 1)
    gp = ref.full_convlogic_backward_weight(gx2, gx3, gr, xr, x2, x3, idx, sel, 1, 1, 1, 1)
    return y, idx_r, gx, gp


# name, batch, C_in, C_out, side, input kind
BLOCKS = [
    ("c2_block_9_256_32", 256, 9, 256, 32, "bits"),         # config 2 at full size
    ("c3_block2_256_1024_16", 64, 256, 1024, 16, "rand"),   # the many-channel layers of the cifar10_m stack
    ("c3_block3_1024_4096_8", 64, 1024, 4096, 8, "rand"),
    ("c3_block4_4096_8192_4", 64, 4096, 8192, 4, "rand"),
    ("c3_block2_full_batch", 256, 256, 1024, 16, "rand"),   # batch 256: the scratch sizes of the training step
]


@pytest.mark.parametrize("name,n,ci,c,side,kind", BLOCKS, ids=[b[0] for b in BLOCKS])
def test_fused_block_at_benchmark_shape_against_reference_kernels(ref_conv, name, n, ci, c, side, kind):
    import convlogic_b200 as cb
    from convlogic_b200 import ops
    from convlogic_b200._lib import W_SOFTMAX

    torch.manual_seed(len(name))
    layer = cb.ConvLogicLayer(ci, c, padding=1, complete=True).cuda().train()
    g = torch.Generator(device="cuda").manual_seed(c)
    layer.weights.data = torch.randn(c, 7, 16, device="cuda", generator=g)
    x = torch.rand(n, ci, side, side, device="cuda", generator=g)
    if kind == "bits":
        x = (x < 0.5).float()
    gy = torch.randn(n, c, side // 2, side // 2, device="cuda", generator=g)
    sel = layer.selection

    # the module path: logits in, soft-max and its Jacobian inside the kernels
    xd = x.clone().requires_grad_(True)
    y = layer(xd)
    y.backward(gy)
    gx, gl = xd.grad, layer.weights.grad
    idx = ops.convtree_fwd(x, layer.weights.detach(), sel, (1, 1, 1, 1, 3, 3), W_SOFTMAX, want_indices=True)[4]

    p = torch.softmax(layer.weights.detach().double(), -1)
    # fp32 reference
    y_r, idx_r, gx_r, gp_r = _reference_block(ref_conv, x, p, sel, idx, gy, torch.float32)
    assert_close(y, y_r, TOL, "y vs reference fp32")
    assert_same_argmax_up_to_ties(idx, idx_r, 1e-3)
    assert_close(gx, gx_r, TOL, "gx vs reference fp32")
    # the reference sums the gate gradient serially in fp32 (one partial per image and channel, then torch.sum):
    # its own rounding error at these sizes is a few 1e-5, so the tight statement is made against its fp64 run
    assert_close(gl, _softmax_jacobian(p, gp_r), 1e-4, "gw vs reference fp32")
    del y_r, gx_r, gp_r
    # fp64 reference (same kernels, negligible summation error)
    y_d, idx_d, gx_d, gp_d = _reference_block(ref_conv, x, p, sel, idx, gy, torch.float64)
    assert_close(y, y_d, TOL, "y vs reference fp64")
    assert_same_argmax_up_to_ties(idx, idx_d, 1e-3)
    assert_close(gx, gx_d, TOL, "gx vs reference fp64")
    assert_close(gl, _softmax_jacobian(p, gp_d), TOL, "gw vs reference fp64")
    del gx_d, gp_d
    # the reference-style Function call (mixture in, gradient w.r.t. the mixture out).  Its mixture is the fp64
    # soft-max rounded to fp32, not the kernels' own fp32 soft-max, so near-tied windows may pool elsewhere than
    # above: the reference's backward is run again at the positions THIS call pooled.
    from convlogic_b200._lib import W_PROB

    pf = p.float()
    pd = pf.clone().requires_grad_(True)
    xd2 = x.clone().requires_grad_(True)
    y2 = cb.FullConvLogicFunction.apply(xd2, pd, sel, 1, 1, 1, 1, 3, 3)
    gx2, gp2 = torch.autograd.grad((y2 * gy).sum(), (xd2, pd))
    idx2 = ops.convtree_fwd(x, pf, sel, (1, 1, 1, 1, 3, 3), W_PROB, want_indices=True)[4]
    assert_close(y2, y_d, TOL, "Function y")
    assert_same_argmax_up_to_ties(idx2, idx_d, 1e-3)
    _, _, gx_f, gp_f = _reference_block(ref_conv, x, pf, sel, idx2, gy, torch.float64)
    assert_close(gx2, gx_f, TOL, "Function gx")
    assert_close(gp2, gp_f, TOL, "Function gw (mixture)")


@pytest.mark.parametrize("ci,c,side", [(1024, 4096, 8), (256, 1024, 16)])
def test_many_channel_block_against_cpu_oracle(ci, c, side):
    """A many-channel layer of the cifar10_m stack at batch 2 against the CPU oracle (autograd through it at the
    kernels' pooled positions)."""
    import convlogic_b200 as cb
    from convlogic_b200 import ops
    from convlogic_b200._lib import W_SOFTMAX

    torch.manual_seed(ci)
    layer = cb.ConvLogicLayer(ci, c, padding=1, complete=True)
    g = torch.Generator().manual_seed(c)
    logits = torch.randn(c, 7, 16, generator=g)
    x = torch.rand(2, ci, side, side, generator=g)
    gy = torch.randn(2, c, side // 2, side // 2, generator=g)
    layer.weights.data = logits.clone()
    layer = layer.cuda().train()
    xd = x.cuda().requires_grad_(True)
    y = layer(xd)
    y.backward(gy.cuda())
    idx = ops.convtree_fwd(x.cuda(), layer.weights.detach(), layer.selection, (1, 1, 1, 1, 3, 3), W_SOFTMAX, want_indices=True)[4].cpu()
    xo, wo = x.clone().requires_grad_(True), logits.clone().requires_grad_(True)
    sel = layer.selection.cpu()
    yo, _, _, idxo = oracle.full_convlogic(xo, oracle.gate_probabilities(wo, True), sel)
    assert_close(y, yo.detach(), TOL, "y")
    assert_same_argmax_up_to_ties(idx, idxo, 1e-3)
    yf = oracle.full_convlogic(xo, oracle.gate_probabilities(wo, True), sel, forced_idx=idx)[0]
    gxo, gwo = torch.autograd.grad((yf * gy).sum(), (xo, wo))
    assert_close(xd.grad, gxo, TOL, "gx")
    assert_close(layer.weights.grad, gwo, TOL, "gw")


def _no_self_pairs(layer):
    """The reference's input-gradient kernel applies d/da twice to a neuron whose two inputs are one feature
    (difflogic_kernel.cu:196-226); keep such neurons out of the comparison by moving their second input."""
    import convlogic_b200 as cb

    a, b = layer.indices_0, layer.indices_1
    clash = a == b
    b[clash] = (b[clash] + 1) % layer.in_dim
    start, cons = cb.LogicLayer.build_consumer_lists(a, b, layer.in_dim)
    layer.given_x_indices_of_y_start.copy_(start)
    layer.given_x_indices_of_y.copy_(cons)


def _reference_flat_chain(ref, layers, x_fm, gy_fm):
    """The reference's flat kernels layer by layer (feature-major), forward then backward; returns the output,
    the input gradient and the gradients w.r.t. the gate mixtures."""
    probs = [torch.softmax(l.weights.detach(), -1) for l in layers]
    acts = [x_fm]
    for l, p in zip(layers, probs):
        acts.append(ref.forward(acts[-1], l.indices_0, l.indices_1, p))
    g = gy_fm
    gps = []
    for l, p, xin in zip(reversed(layers), reversed(probs), reversed(acts[:-1])):
        gps.append(ref.backward_w(xin, l.indices_0, l.indices_1, g))
        g = ref.backward_x(xin, l.indices_0, l.indices_1, p, g, l.given_x_indices_of_y_start, l.given_x_indices_of_y)
    return acts[-1], g, list(reversed(gps)), probs


def test_c3_flat_trio_fused_and_layerwise_against_reference_kernels(ref_flat):
    """The cifar10_m flat stack 32768 -> 327680 -> 163840 -> 81920 at batch 64: the fused gate-tree path and the
    layer-by-layer path against ``difflogic_cuda.forward / backward_w / backward_x``."""
    import convlogic_b200 as cb

    torch.manual_seed(5)
    dims = [32768, 327680, 163840, 81920]
    layers = [cb.LogicLayer(i, o) for i, o in zip(dims[:-1], dims[1:])]
    for l in layers:
        _no_self_pairs(l)
    seq = torch.nn.Sequential(*layers).cuda().train()
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.rand(64, dims[0], device="cuda", generator=g)
    gy = torch.randn(64, dims[-1], device="cuda", generator=g)
    y_r, gx_r, gp_r, probs = _reference_flat_chain(ref_flat, layers, x.t().contiguous(), gy.t().contiguous())
    want_gw = [_softmax_jacobian(p, gp) for p, gp in zip(probs, gp_r)]
    for net, what in ((cb.fuse_logic_layers(seq), "fused"), (seq, "layer by layer")):
        if what == "fused":
            assert isinstance(net[0], cb.FusedLogicLayers), "the stack must qualify for the fused path"
        for l in layers:
            l.weights.grad = None
        xd = x.clone().requires_grad_(True)
        y = net(xd)
        y.backward(gy)
        assert_close(y.t(), y_r, TOL, f"{what}: y")
        assert_close(xd.grad.t(), gx_r, TOL, f"{what}: gx")
        for i, l in enumerate(layers):
            assert_close(l.weights.grad, want_gw[i], TOL, f"{what}: gw of layer {i}")


@pytest.mark.parametrize("in_dim,out_dim", [(3072, 256000), (256000, 256000)])
def test_c5_layer_at_batch_1024_against_reference_kernels(ref_flat, in_dim, out_dim):
    import convlogic_b200 as cb

    torch.manual_seed(in_dim % 1000)
    layer = cb.LogicLayer(in_dim, out_dim)
    _no_self_pairs(layer)
    layer = layer.cuda().train()
    g = torch.Generator(device="cuda").manual_seed(11)
    layer.weights.data = torch.randn(out_dim, 16, device="cuda", generator=g)
    x = torch.rand(1024, in_dim, device="cuda", generator=g)
    if in_dim == 3072:
        x = (x < 0.5).float()
    gy = torch.randn(1024, out_dim, device="cuda", generator=g)
    y_r, gx_r, gp_r, probs = _reference_flat_chain(ref_flat, [layer], x.t().contiguous(), gy.t().contiguous())
    xd = x.clone().requires_grad_(True)
    y = layer(xd)
    y.backward(gy)
    assert_close(y.t(), y_r, TOL, "y")
    assert_close(xd.grad.t(), gx_r, TOL, "gx")
    assert_close(layer.weights.grad, _softmax_jacobian(probs[0], gp_r[0]), TOL, "gw")


def test_c5_group_sum_at_full_width():
    import convlogic_b200 as cb

    g = torch.Generator(device="cuda").manual_seed(3)
    y_fm = torch.rand(256000, 1024, device="cuda", generator=g).requires_grad_(True)
    out = cb.GroupSum(10, 100.0)(y_fm.t())
    want = y_fm.detach().double().t().reshape(1024, 10, 25600).sum(-1) / 100.0
    assert_close(out, want, TOL)
    go = torch.randn(1024, 10, device="cuda", generator=g)
    out.backward(go)
    assert_close(y_fm.grad, (go / 100.0).t().repeat_interleave(25600, 0), 1e-7)


@pytest.fixture(scope="module")
def cifar10_l():
    """The cifar10_l-shaped stack (k = 1024, two extra flat widths), N(0,1) logits, eval mode, compiled."""
    import convlogic_b200 as cb

    torch.manual_seed(0)
    net = cb.ConvLogicCifarModel(k_param=1024, input_channels=93, input_size=32, tau=340).network
    g = torch.Generator().manual_seed(1)
    for prm in net.parameters():
        prm.data = torch.randn(*prm.shape, generator=g)
    net = net.cuda().eval()
    return net, cb.CompiledLogicNet(net, input_shape=(93, 32, 32)).compile()


def test_c4_stack_compiled_equals_modules_equals_float_eval(cifar10_l):
    """Config 4 on 256 seeded images: thermometer input -> the compiled network == the nn.Modules on packed
    activations == tau x the float eval-mode scores, exactly; and two half-shards give the unsharded counts."""
    import convlogic_b200 as cb

    net, cnet = cifar10_l
    g = torch.Generator().manual_seed(42)
    pixels = torch.rand(256, 3, 32, 32, generator=g).cuda()
    th = (torch.arange(1, 32, dtype=torch.float32) / 32).cuda()
    counts = cnet.forward_pixels(pixels, th)
    assert counts.dtype == torch.int32 and counts.shape == (256, 10)
    with torch.no_grad():
        by_modules = net(cb.PackBitsTensor.from_pixels(pixels, th))
        bits = torch.cat([(pixels > t) for t in th.tolist()], dim=1)      # the reference's input transform
        by_bool = net(cb.PackBitsTensor(bits, 64))
        scores = net(bits.float())
    assert torch.equal(counts, by_modules)
    assert torch.equal(counts, by_bool)
    assert torch.equal(counts, (scores.double() * 340).round().to(torch.int32))
    assert int(counts.sum()) > 0 and len(counts.unique()) > 10   # not a degenerate answer
    halves = torch.cat([cnet.forward_pixels(pixels[:128].contiguous(), th), cnet.forward_pixels(pixels[128:].contiguous(), th)])
    assert torch.equal(halves, counts)
    ragged = torch.cat([cnet.forward_pixels(pixels[:100].contiguous(), th), cnet.forward_pixels(pixels[100:].contiguous(), th)])
    assert torch.equal(ragged, counts)


def test_c4_first_block_and_flat_layers_against_cpu_oracle(cifar10_l):
    """The two ends of the cifar10_l stack at their own widths against the CPU oracle's packed kernels: block 1
    (93 -> 1024 channels at 32x32) and the 131072 -> 2621440 flat layer, bit for bit, on 128 images."""
    import convlogic_b200 as cb

    net, _ = cifar10_l
    g = torch.Generator().manual_seed(43)
    pixels = torch.rand(128, 3, 32, 32, generator=g)
    th = np.arange(1, 32, dtype=np.float32) / np.float32(32)
    bits = oracle.thermometer(pixels.numpy(), 31)                       # [128, 93, 32, 32]
    packed, pad = oracle.pack_bits(bits.reshape(128, -1).T, 64)
    p = cb.PackBitsTensor.from_pixels(pixels.cuda(), torch.from_numpy(th).cuda())
    assert np.array_equal(p.rows().cpu().numpy().reshape(packed.shape), packed)
    block = net[0]
    with torch.no_grad():
        got = block(p).rows().cpu().numpy()
    want = oracle.packed_convtree(packed.reshape(93, 32, 32, -1), block.weights.argmax(-1).cpu().numpy().astype(np.uint8),
                                  block.selection.cpu().numpy())
    assert np.array_equal(got, want)
    flat = [m for m in net if isinstance(m, cb.LogicLayer)][0]
    rng = np.random.default_rng(0)
    rows = rng.integers(-2 ** 63, 2 ** 63 - 1, (flat.in_dim, 2), dtype=np.int64)
    with torch.no_grad():
        got = flat(cb.PackBitsTensor.from_packed(torch.from_numpy(rows).cuda(), 0)).t.cpu().numpy()
    want = oracle.packed_logic(rows, flat.indices_0.cpu().numpy(), flat.indices_1.cpu().numpy(),
                               flat.weights.argmax(-1).cpu().numpy().astype(np.uint8))
    assert np.array_equal(got, want)
