"""Cross-check against the reference's OWN CUDA kernels, built for sm_100a by oracle/build_ref.py.

Skipped when ``oracle/_ref`` has not been built.  This pins, on the GPU, what the reference's tests do
not cover on the CPU: packed inference (``eval``, ``tensor_packbits_cuda``, ``groupbitsum``) bit for
bit, and the float kernels of both extensions within fp32 tolerance."""

import numpy as np
import pytest
import torch

from oracle.build_ref import load_ref
from tests.util import assert_close, assert_same_argmax_up_to_ties

pytestmark = pytest.mark.gpu


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


@pytest.mark.parametrize("n,ci,c,size,pad,k", [(16, 9, 64, 32, 1, 3), (8, 16, 24, 12, 1, 3), (4, 1, 16, 28, 0, 5), (6, 64, 32, 16, 1, 3)])
def test_fused_block_against_reference_kernels(ref_conv, n, ci, c, size, pad, k):
    import convlogic_b200 as cb
    from convlogic_b200 import FullConvLogicFunction

    torch.manual_seed(n + c)
    layer = cb.ConvLogicLayer(ci, c, padding=pad, kernel=k, complete=True).cuda()
    sel = layer.selection
    x = torch.rand(n, ci, size, size, device="cuda")
    w_prob = torch.softmax(torch.randn(c, 7, 16, device="cuda"), -1)
    y_r, x2_r, x3_r, idx_r = ref_conv.full_convlogic_forward(x, w_prob, sel, 1, 1, pad, pad, k, k)
    xd = x.clone().requires_grad_(True)
    wd = w_prob.clone().requires_grad_(True)
    y, x2, x3, idx = FullConvLogicFunction.apply(xd, wd, sel, 1, 1, pad, pad, k, k, True, True)
    assert_close(y, y_r, 1e-5, "y")
    assert_close(x2, x2_r, 1e-5, "x2")
    assert_close(x3, x3_r, 1e-5, "x3")
    assert_same_argmax_up_to_ties(idx, idx_r, 1e-3)  # only fp32 near-ties may differ (y is compared above)
    # The reference's backward kernels take the pooled positions as an argument: hand them the positions this
    # library pooled, so that both sides route the gradient through the same elements and EVERY gradient value
    # is compared, ties or not.
    gy = torch.randn_like(y_r)
    gx_r, gx2_r, gx3_r = ref_conv.full_convlogic_backward_x(gy, x, x2_r, x3_r, w_prob, idx, sel, 1, 1, pad, pad)
    gw_r = ref_conv.full_convlogic_backward_weight(gx2_r, gx3_r, gy, x, x2_r, x3_r, idx, sel, 1, 1, pad, pad)
    y2 = FullConvLogicFunction.apply(xd, wd, sel, 1, 1, pad, pad, k, k)
    gx, gw = torch.autograd.grad((y2 * gy).sum(), (xd, wd))
    assert_close(gx, gx_r, 1e-5, "gx")
    assert_close(gw, gw_r, 1e-5, "gw")


def test_flat_layer_against_reference_kernels(ref_flat):
    import convlogic_b200 as cb

    torch.manual_seed(0)
    layer = cb.LogicLayer(96, 400).cuda()
    a, b = layer.indices_0, layer.indices_1
    # the reference's input-gradient kernel mishandles a neuron whose two inputs coincide; avoid such neurons here
    b[a == b] = (b[a == b] + 1) % 96
    start, cons = cb.LogicLayer.build_consumer_lists(a, b, 96)
    start, cons = start.cuda(), cons.cuda()
    x = torch.rand(96, 512, device="cuda")
    w = torch.softmax(torch.randn(400, 16, device="cuda"), -1)
    gy = torch.randn(400, 512, device="cuda")
    y_r = ref_flat.forward(x, a, b, w)
    gw_r = ref_flat.backward_w(x, a, b, gy)
    gx_r = ref_flat.backward_x(x, a, b, w, gy, start, cons)
    xd, wd = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y = cb.LogicLayerCudaFunction.apply(xd, a, b, wd, start, cons)
    gx, gw = torch.autograd.grad((y * gy).sum(), (xd, wd))
    assert_close(y, y_r, 1e-5)
    assert_close(gw, gw_r, 1e-5)
    assert_close(gx, gx_r, 1e-5)


@pytest.mark.parametrize("bits", [8, 16, 32, 64])
@pytest.mark.parametrize("batch", [64, 100, 1024])
def test_packed_path_bit_exact_against_reference_kernels(ref_flat, bits, batch):
    import convlogic_b200 as cb
    from convlogic_b200 import ops

    torch.manual_seed(bits + batch)
    layer = cb.LogicLayer(40, 120).cuda().eval()
    xb = torch.rand(batch, 40, device="cuda") < 0.5
    packed_r, pad_r = ref_flat.tensor_packbits_cuda(xb.T.contiguous(), bits)
    p = cb.PackBitsTensor(xb, bits)
    assert p.pad_len == pad_r and torch.equal(p.t, packed_r)
    got2, pad2 = ops.pack_bits(xb.T.contiguous(), bits)
    assert pad2 == pad_r and torch.equal(got2, packed_r)
    gate_ids = layer.weights.argmax(-1).to(torch.uint8)
    y_r = ref_flat.eval(packed_r, layer.indices_0, layer.indices_1, gate_ids)
    y = layer(p)
    assert torch.equal(y.t, y_r)  # pad bits included: same bitwise gates
    counts_r = ref_flat.groupbitsum(y_r, pad_r, 10)
    assert torch.equal(cb.GroupSum(10)(y), counts_r)
