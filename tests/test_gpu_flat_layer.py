"""Flat LogicLayer and GroupSum on the GPU against the reference's golden tensors and the oracle."""

import numpy as np
import pytest
import torch

import oracle
from tests.util import assert_close

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _layer(cb, g, pre):
    a, b = torch.from_numpy(g[f"{pre}/a"]), torch.from_numpy(g[f"{pre}/b"])
    in_dim, out_dim = g[f"{pre}/x"].shape[1], a.shape[0]
    layer = cb.LogicLayer(in_dim, out_dim)
    state = layer.state_dict()
    start, cons = cb.LogicLayer.build_consumer_lists(a, b, in_dim)
    state.update(weights=torch.from_numpy(g[f"{pre}/logits"]), indices_0=a, indices_1=b,
                 given_x_indices_of_y_start=start, given_x_indices_of_y=cons)
    layer.load_state_dict(state)
    return layer.cuda()


@pytest.mark.parametrize("j", [0, 1, 2])
def test_matches_reference_golden(golden, j):
    import convlogic_b200 as cb

    g = golden("flat_layers")
    pre = f"flat{j}"
    layer = _layer(cb, g, pre).train()
    k, tau = g[f"{pre}/k_tau"]
    x = torch.from_numpy(g[f"{pre}/x"]).cuda().requires_grad_(True)
    y = layer(x)
    gx, gw = torch.autograd.grad((y * torch.from_numpy(g[f"{pre}/gy"]).cuda()).sum(), (x, layer.weights), retain_graph=True)
    assert_close(y, g[f"{pre}/y_soft"], TOL, "soft forward")
    assert_close(gx, g[f"{pre}/gx"], TOL, "input gradient")
    assert_close(gw, g[f"{pre}/gw_logits"], TOL, "logit gradient")
    assert_close(cb.GroupSum(int(k), float(tau))(y), g[f"{pre}/group_sum"], TOL, "group sum")
    layer.eval()
    yh = layer(x.detach())
    assert_close(yh, g[f"{pre}/y_hard"], TOL, "hard forward")
    if j == 0:
        assert np.array_equal(yh.cpu().numpy(), g[f"{pre}/y_hard"])


@pytest.mark.parametrize("batch,in_dim,out_dim", [(1, 8, 16), (3, 10, 30), (256, 64, 200), (1028, 32, 96), (2050, 6, 12)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float64, 1e-10)])
def test_function_api_matches_oracle(batch, in_dim, out_dim, dtype, tol):
    """Reference-style call: feature-major x, probabilities in, gradient w.r.t. probabilities out;
    batches beyond the reference kernel's 1024 limit included."""
    import convlogic_b200 as cb

    g = torch.Generator().manual_seed(batch)
    a = torch.randint(0, in_dim, (out_dim,), generator=g)
    b = torch.randint(0, in_dim, (out_dim,), generator=g)
    b[0] = a[0]  # a neuron reading the same feature twice
    x = torch.rand(batch, in_dim, generator=g, dtype=dtype)
    p = torch.softmax(torch.randn(out_dim, 16, generator=g, dtype=dtype), -1)
    gy = torch.randn(batch, out_dim, generator=g, dtype=dtype)
    xo, po = x.clone().requires_grad_(True), p.clone().requires_grad_(True)
    yo = oracle.logic_layer(xo, a, b, po)
    gxo, gpo = torch.autograd.grad((yo * gy).sum(), (xo, po))
    start, cons = cb.LogicLayer.build_consumer_lists(a, b, in_dim)
    xd = x.T.contiguous().cuda().requires_grad_(True)
    pd = p.cuda().requires_grad_(True)
    y = cb.LogicLayerCudaFunction.apply(xd, a.cuda(), b.cuda(), pd, start.cuda(), cons.cuda())
    gx, gp = torch.autograd.grad((y * gy.T.contiguous().cuda()).sum(), (xd, pd))
    assert_close(y.T, yo.detach(), tol)
    assert_close(gx.T, gxo, tol)
    assert_close(gp, gpo, tol)


def test_all_logic_gates_flat():
    """Known-answer test of the 16 gates (tests/difflogic/test_difflogic_forward.py:74-100)."""
    import convlogic_b200 as cb

    layer = cb.LogicLayer(2, 16).cuda().eval()
    w = torch.full((16, 16), -float("inf"))
    w[torch.arange(16), torch.arange(16)] = 0.0
    layer.weights.data = w.cuda()
    layer.indices_0.zero_()
    layer.indices_1.fill_(1)
    x = torch.tensor([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]], device="cuda")
    y = layer(x).cpu()
    for gate in range(16):
        want = oracle.bin_op(x[:, 0].cpu(), x[:, 1].cpu(), gate)
        assert torch.equal(y[:, gate], want), gate


def test_gradcheck_like_reference():
    """tests/difflogic/test_difflogic_autograd.py:31-54."""
    import convlogic_b200 as cb
    from torch.autograd import gradcheck

    torch.manual_seed(0)
    layer = cb.LogicLayer(6, 10).double().cuda()
    x = torch.rand(6, 5, dtype=torch.double, device="cuda", requires_grad=True)
    w = layer.weights.detach().clone().requires_grad_(True)

    def fn(inp, logits):
        return cb.LogicLayerCudaFunction.apply(inp, layer.indices_0, layer.indices_1, torch.softmax(logits, -1),
                                               layer.given_x_indices_of_y_start, layer.given_x_indices_of_y)

    assert gradcheck(fn, (x, w), eps=1e-6, atol=1e-4)


def test_layer_stack_stays_feature_major_and_deterministic():
    import convlogic_b200 as cb

    torch.manual_seed(0)
    l1, l2 = cb.LogicLayer(32, 64).cuda(), cb.LogicLayer(64, 40).cuda()
    x = torch.rand(20, 32, device="cuda", requires_grad=True)
    outs = []
    for _ in range(2):
        for m in (l1, l2):
            m.weights.grad = None
        x.grad = None
        h = l1(x)
        assert h.T.is_contiguous()  # the next layer's transpose is a free view
        y = cb.GroupSum(10, 3.0)(l2(h))
        y.square().sum().backward()
        outs.append((y.detach().clone(), x.grad.clone(), l1.weights.grad.clone()))
    assert all(torch.equal(u, v) for u, v in zip(*outs))


def test_empty_batch_runs_through_a_small_stack():
    """Edge case: a batch of zero samples gives empty outputs and zero gate gradients."""
    import convlogic_b200 as cb

    torch.manual_seed(0)
    net = torch.nn.Sequential(cb.ConvLogicLayer(3, 4, complete=True), torch.nn.Flatten(), cb.LogicLayer(64, 40),
                              cb.GroupSum(10, 2.0)).cuda().train()
    x = torch.zeros(0, 3, 8, 8, device="cuda", requires_grad=True)
    y = net(x)
    assert y.shape == (0, 10)
    y.sum().backward()
    assert x.grad.shape == x.shape
    for prm in net.parameters():
        assert prm.grad is not None and float(prm.grad.abs().sum()) == 0.0
    # the context is fine afterwards
    assert net(torch.rand(2, 3, 8, 8, device="cuda")).shape == (2, 10)


@pytest.mark.parametrize("f,b,k", [(640, 256, 10), (81920, 64, 10), (30, 7, 3), (1280, 33, 10), (12, 1, 4)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.float64, 1e-13)])
def test_group_sum_on_feature_major_storage(f, b, k, dtype, tol):
    """GroupSum fed with the transposed view a LogicLayer returns sums the feature-major storage directly:
    same values and gradients as the reference expression `x.reshape(B, k, F/k).sum(-1) / tau` (and as the oracle)."""
    import convlogic_b200 as cb

    torch.manual_seed(f + b)
    y_fm = torch.randn(f, b, dtype=dtype, device="cuda")
    gs = cb.GroupSum(k, tau=3.5)
    x = y_fm.t().requires_grad_(True)            # [B, F] view of feature-major storage, as LogicLayer returns it
    out = gs(x)
    xr = y_fm.t().contiguous().requires_grad_(True)
    ref = xr.reshape(b, k, f // k).sum(-1) / 3.5
    assert out.shape == (b, k)
    assert_close(out.detach(), ref.detach(), tol)
    assert_close(out.detach().cpu(), oracle.group_sum(y_fm.t().cpu(), k, 3.5), tol)
    g = torch.randn(b, k, dtype=dtype, device="cuda")
    (gx,) = torch.autograd.grad(out, x, g)
    (gr,) = torch.autograd.grad(ref, xr, g)
    assert_close(gx, gr, tol)                     # torch multiplies by 1/tau where the kernel divides
    assert torch.equal(gs(x), out)                # fixed summation order: repeatable
    with pytest.raises(AssertionError):
        cb.GroupSum(7)(x)


@pytest.mark.parametrize("in_dim,out_dim,batch", [(50, 40, 64), (500, 60, 20), (33, 700, 256), (2000, 1000, 96), (7, 3, 5)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float64, 1e-12)])
def test_input_gradient_with_arbitrary_connections(in_dim, out_dim, batch, dtype, tol):
    """Hand-made connections, drawn uniformly: inputs without any consumer (their gradient is zero), neurons fed
    twice by the same input, fan-outs from 0 to dozens inside one unit of the segmented kernel -- against autograd
    through the oracle."""
    from convlogic_b200 import ops
    from convlogic_b200._lib import W_SOFTMAX

    rng = np.random.default_rng(in_dim + out_dim)
    a = torch.from_numpy(rng.integers(0, in_dim, out_dim))
    b = torch.from_numpy(rng.integers(0, in_dim, out_dim))
    b[: max(1, out_dim // 10)] = a[: max(1, out_dim // 10)]      # self-paired neurons
    if in_dim > 20:                                               # a run of inputs nobody reads
        a[(a >= 5) & (a < 12)] = 0
        b[(b >= 5) & (b < 12)] = 1
    start, cons = oracle.inverse_connections(a.numpy(), b.numpy(), in_dim)
    torch.manual_seed(0)
    x = torch.rand(batch, in_dim, dtype=dtype)
    logits = torch.randn(out_dim, 16, dtype=dtype)
    gy = torch.randn(batch, out_dim, dtype=dtype)
    xo = x.clone().requires_grad_(True)
    yo = oracle.logic_layer(xo, a, b, oracle.gate_probabilities(logits, True))
    (gxo,) = torch.autograd.grad((yo * gy).sum(), (xo,))
    x_fm, gy_fm = x.t().contiguous().cuda(), gy.t().contiguous().cuda()
    gx = ops.logic_bwd_x(x_fm, a.cuda(), b.cuda(), logits.cuda(), gy_fm, torch.from_numpy(start).cuda(),
                         torch.from_numpy(cons).cuda(), W_SOFTMAX)
    assert_close(gx.t().cpu(), gxo, tol)
    if in_dim > 20:
        assert float(gx[5:12].abs().max()) == 0.0
    again = ops.logic_bwd_x(x_fm, a.cuda(), b.cuda(), logits.cuda(), gy_fm, torch.from_numpy(start).cuda(),
                            torch.from_numpy(cons).cuda(), W_SOFTMAX)
    assert torch.equal(gx, again)


@pytest.mark.parametrize("dims,batch", [((40, 320, 160, 80), 64), ((96, 640, 320, 160), 256), ((30, 200, 100, 50), 37), ((64, 480, 240, 120), 4)])
def test_three_fused_layers_equal_the_layers_one_by_one(dims, batch):
    """FusedLogicLayers (one gate tree per neuron of the last layer) against the same three LogicLayers run in
    sequence: soft and hard forward, input gradient and the logit gradients of all three layers; repeatable."""
    import convlogic_b200 as cb

    torch.manual_seed(sum(dims))
    seq = torch.nn.Sequential(*[cb.LogicLayer(i, o) for i, o in zip(dims[:-1], dims[1:])], cb.GroupSum(10, 2.0)).cuda()
    g = torch.Generator().manual_seed(3)
    for prm in seq.parameters():
        prm.data = torch.randn(*prm.shape, generator=g).cuda()
    fused = cb.fuse_logic_layers(seq)
    assert isinstance(fused[0], cb.FusedLogicLayers) and len(fused) == 2
    assert fused[0].layers[0].weights is seq[0].weights          # shared parameters
    x = torch.rand(batch, dims[0], device="cuda")
    gy = torch.randn(batch, 10, device="cuda")

    def run(model):
        model.train()
        for prm in model.parameters():
            prm.grad = None
        xi = x.clone().requires_grad_(True)
        out = model(xi)
        out.backward(gy)
        grads = [seq[i].weights.grad.clone() for i in range(3)]
        model.eval()
        with torch.no_grad():
            hard = model(x)
        return out.detach(), xi.grad.clone(), grads, hard

    y_s, gx_s, gw_s, h_s = run(seq)
    y_f, gx_f, gw_f, h_f = run(fused)
    assert_close(y_f, y_s, 1e-5)
    assert_close(gx_f, gx_s, 1e-5)
    for a, b in zip(gw_f, gw_s):
        assert_close(a, b, 2e-5)
    assert torch.equal(h_f, h_s)                                   # one-hot gates on the same inputs: exact
    y_2, gx_2, gw_2, _ = run(fused)
    assert torch.equal(y_2, y_f) and torch.equal(gx_2, gx_f) and all(torch.equal(a, b) for a, b in zip(gw_2, gw_f))
    # packed input goes through the three layers themselves
    xb = torch.rand(batch, dims[0], device="cuda") < 0.5
    fused.eval()
    seq.eval()
    with torch.no_grad():
        assert torch.equal(fused(cb.PackBitsTensor(xb, 64)), seq(cb.PackBitsTensor(xb, 64)))


def test_fusing_is_refused_when_outputs_are_read_twice():
    import convlogic_b200 as cb

    torch.manual_seed(0)
    layers = [cb.LogicLayer(40, 100), cb.LogicLayer(100, 90), cb.LogicLayer(90, 60)]   # 2 * 90 > 100: outputs reused
    with pytest.raises(ValueError):
        cb.FusedLogicLayers(layers)
    model = cb.fuse_logic_layers(torch.nn.Sequential(*layers, cb.GroupSum(10)))
    assert all(isinstance(m, cb.LogicLayer) for m in list(model)[:3])
