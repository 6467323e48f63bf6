"""The tail of the training step on this library's kernels: GroupSum + cross-entropy in one pass, gate gradients written
straight into the flat bucket, Adam over the flat buffer -- each against the torch expression it stands in for, and a
three-step training trajectory of a small CIFAR-shaped stack against the all-torch tail (fp32, 1e-5)."""

import pytest
import torch

from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _model(seed):
    import convlogic_b200 as cb

    torch.manual_seed(seed)
    net = cb.ConvLogicCifarModel(k_param=8, input_channels=9, input_size=32, tau=7.0).network
    g = torch.Generator().manual_seed(seed + 1)
    for prm in net.parameters():
        prm.data = torch.randn(*prm.shape, generator=g)
    return net.cuda().train()


@pytest.mark.parametrize("batch,features,k,tau", [(64, 160, 10, 2.0), (300, 2560, 10, 40.0), (5, 32, 4, 1.0), (1030, 330, 11, 3.5)])
def test_group_sum_cross_entropy_equals_torch(batch, features, k, tau):
    import convlogic_b200 as cb

    torch.manual_seed(batch)
    layer = cb.LogicLayer(48, features).cuda().train()
    x = torch.rand(batch, 48, device="cuda")
    labels = torch.randint(0, k, (batch,), device="cuda")
    y = layer(x)                                   # the transposed view of feature-major storage
    y1 = y.detach().clone().requires_grad_(True)   # same values, ordinary layout -> the torch expression
    want = torch.nn.functional.cross_entropy(cb.GroupSum(k, tau)(y1), labels)
    (gwant,) = torch.autograd.grad(want * 3.0, (y1,))
    yt = y.detach().t().contiguous().t().requires_grad_(True)
    got = cb.GroupSumCrossEntropy(k, tau)(yt, labels)
    (ggot,) = torch.autograd.grad(got * 3.0, (yt,))
    assert got.shape == () and abs(float(got) - float(want)) <= 1e-5 * max(1.0, abs(float(want)))
    assert_close(ggot, gwant, 1e-5, "gradient w.r.t. the activations")
    # an input in the ordinary layout takes the torch expression and gives the same loss
    assert abs(float(cb.GroupSumCrossEntropy(k, tau)(y1, labels)) - float(want)) <= 1e-6


@pytest.mark.parametrize("decoupled,wd", [(False, 0.0), (False, 0.01), (True, 0.002)])
def test_flat_adam_equals_torch_adam(decoupled, wd):
    import convlogic_b200 as cb
    from convlogic_b200 import dp

    model = torch.nn.Sequential(cb.LogicLayer(32, 100), cb.LogicLayer(100, 50), cb.GroupSum(10, 2.0)).cuda().train()
    twin = torch.nn.Sequential(cb.LogicLayer(32, 100), cb.LogicLayer(100, 50), cb.GroupSum(10, 2.0)).cuda().train()
    twin.load_state_dict(model.state_dict())
    ref = (torch.optim.AdamW if decoupled else torch.optim.Adam)(twin.parameters(), lr=0.01, weight_decay=wd)
    bucket = dp.GradBucket(model)
    opt = cb.FlatAdam(bucket, lr=0.01, weight_decay=wd, decoupled=decoupled)
    names = [n for n, _ in model.named_parameters()]
    assert names == [n for n, _ in twin.named_parameters()]      # parameters are views now, names and shapes unchanged
    g = torch.Generator(device="cuda").manual_seed(0)
    for step in range(4):
        x = torch.rand(40, 32, device="cuda", generator=g)
        lab = torch.randint(0, 10, (40,), device="cuda", generator=g)
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), lab).backward()
        opt.step()
        ref.zero_grad()
        torch.nn.functional.cross_entropy(twin(x), lab).backward()
        ref.step()
        for (n, p), q in zip(model.named_parameters(), twin.parameters()):
            assert_close(p, q, 2e-6, f"step {step}: {n}")


def test_three_step_trajectory_equals_torch_tail():
    """Fused tail (gate-tree flat layers, GroupSum + cross-entropy kernel, gradients written into the bucket, flat Adam)
    against the module-by-module stack with torch's cross-entropy and Adam: the same loss, gradients and updated parameters
    for each of three consecutive steps."""
    import convlogic_b200 as cb
    from convlogic_b200 import dp

    a, b = _model(3), _model(3)
    opt_a = torch.optim.Adam(a.parameters(), lr=0.01)
    fused = cb.fuse_logic_layers(b)
    assert isinstance(fused[-1], cb.GroupSum)
    body, head = fused[:-1], cb.GroupSumCrossEntropy(fused[-1].k, fused[-1].tau)
    bucket = dp.GradBucket(b).direct()
    opt_b = cb.FlatAdam(bucket, lr=0.01)
    g = torch.Generator(device="cuda").manual_seed(5)
    params_a, params_b = list(a.parameters()), list(b.parameters())
    for step in range(3):
        x = (torch.rand(32, 9, 32, 32, device="cuda", generator=g) < 0.5).float()
        lab = torch.randint(0, 10, (32,), device="cuda", generator=g)
        # every step starts from the module-by-module side's exact state (parameters and Adam moments): what is compared
        # is one whole step from equal states, three times along a real trajectory, not the drift of two trajectories
        with torch.no_grad():
            for i, (pa, pb) in enumerate(zip(params_a, params_b)):
                pb.copy_(pa)
                lo, hi = bucket.ranges[[id(q) for q in bucket.params].index(id(pb))]
                st = opt_a.state.get(pa)
                if st:
                    opt_b.exp_avg[lo:hi].copy_(st["exp_avg"].reshape(-1))
                    opt_b.exp_avg_sq[lo:hi].copy_(st["exp_avg_sq"].reshape(-1))
        opt_a.zero_grad()
        loss_a = torch.nn.functional.cross_entropy(a(x), lab)
        loss_a.backward()
        grads_a = [p.grad.clone() for p in a.parameters()]
        opt_a.step()
        loss_b = head(body(x), lab)
        loss_b.backward()
        bucket.finish()
        for (n, p), ga in zip(b.named_parameters(), grads_a):
            assert p.grad is not None and p.grad.data_ptr() == bucket.flat[bucket.ranges[[id(q) for q in bucket.params].index(id(p))][0]:].data_ptr()
            # both sides are fp32 with different summation orders (one gate tree per output neuron against three layers
            # one after the other): a few 1e-5 of the largest gradient, max-normalised
            assert_close(p.grad, ga, 5e-5, f"step {step}: gradient of {n}")
        opt_b.step()
        assert abs(float(loss_a) - float(loss_b)) <= 1e-5 * max(1.0, abs(float(loss_a))), (step, float(loss_a), float(loss_b))
        # Adam moves an entry by lr * m / (sqrt(v) + eps): where a gradient is itself of the size of the fp32 summation
        # differences above (around eps = 1e-8), the two sides move that entry by different fractions of lr.  So: no entry
        # differs by more than a tenth of one step, and all but 1 in 1000 agree to 1e-5 of the largest parameter.
        for (n, p), q in zip(b.named_parameters(), a.parameters()):
            diff = (p - q).abs()
            assert float(diff.max()) <= 0.1 * 0.01, (step, n, float(diff.max()))
            off = float((diff > 1e-5 * float(q.abs().max())).float().mean())
            assert off <= 1e-3, (step, n, off)


@pytest.mark.parametrize("rows,cols", [(256, 32768), (37, 1001), (1, 5), (1031, 64)])
def test_tiled_transpose_equals_torch(rows, cols):
    from convlogic_b200 import ops
    from convlogic_b200.functional import to_feature_major

    g = torch.Generator(device="cuda").manual_seed(rows)
    x = torch.randn(rows, cols, device="cuda", generator=g)
    assert torch.equal(ops.transpose2d(x), x.t().contiguous())
    xr = x.clone().requires_grad_(True)
    y = to_feature_major(xr)
    gy = torch.randn(cols, rows, device="cuda", generator=g)
    y.backward(gy)
    assert torch.equal(y, x.t()) and torch.equal(xr.grad, gy.t()) and xr.grad.is_contiguous()
    assert to_feature_major(x.t()).data_ptr() == x.data_ptr()   # the transposed view of a flat layer's output: no copy


def test_adam_update_in_two_pieces_equals_one_step():
    """FlatAdam.finish_and_step updates the slice whose exchange is still in flight after the rest: with a stand-in for the
    exchange (one GPU), parameters and moments must equal those of a plain step, bit for bit."""
    import convlogic_b200 as cb
    from convlogic_b200 import dp

    def make():
        torch.manual_seed(11)
        m = torch.nn.Sequential(cb.LogicLayer(32, 96), cb.LogicLayer(96, 48), cb.GroupSum(8, 2.0)).cuda()
        bucket = dp.GradBucket(m)
        return m, bucket, cb.FlatAdam(bucket, lr=0.01)

    (ma, ba, oa), (mb, bb, ob) = make(), make()
    g = torch.Generator(device="cuda").manual_seed(2)
    for step in range(2):
        grad = torch.randn(ba.numel, device="cuda", generator=g)
        ba.flat.copy_(grad), bb.flat.copy_(grad)
        oa.step()
        lo, hi = bb.ranges[0]                      # pretend the first layer's exchange is the one still in flight
        bb.finish_but_last = lambda lo=lo, hi=hi: (lo, hi)
        ob.finish_and_step()
        assert oa.steps == ob.steps == step + 1
        assert torch.equal(oa.params, ob.params) and torch.equal(oa.exp_avg, ob.exp_avg) and torch.equal(oa.exp_avg_sq, ob.exp_avg_sq)


@pytest.mark.parametrize("dims,batch", [((40, 320, 160, 80), 64), ((40, 320, 160, 80), 37), ((96, 2560, 1280, 640), 256),
                                        ((96, 2560, 1280, 640), 132), ((64, 1280, 640, 320), 512)])
def test_fused_layers_with_the_loss_head_equal_the_separate_modules(dims, batch):
    """FusedLogicLayers.cross_entropy (trees + GroupSum + cross-entropy as one autograd node) against FusedLogicLayers ->
    GroupSumCrossEntropy: loss, input gradient and all gate gradients.  With a batch the summing forward does not take (37)
    only the backward differs -- it derives the values the GroupSum backward kernel would have written -- and everything is
    equal bit for bit; with batch 64 the class sums are added in another order (fp32): 1e-6 on the loss, 1e-5 of the largest
    entry on the gradients."""
    import convlogic_b200 as cb

    torch.manual_seed(4)
    k, tau = 10, 3.0
    seq = torch.nn.Sequential(*[cb.LogicLayer(i, o) for i, o in zip(dims[:-1], dims[1:])], cb.GroupSum(k, tau)).cuda()
    fused = cb.fuse_logic_layers(seq)[0].train()
    g = torch.Generator(device="cuda").manual_seed(batch)
    x = torch.rand(batch, dims[0], device="cuda", generator=g)
    lab = torch.randint(0, k, (batch,), device="cuda", generator=g)

    def grads(loss_fn):
        for p in fused.parameters():
            p.grad = None
        xi = x.clone().requires_grad_(True)
        loss = loss_fn(xi) * 1.7          # a scale other than one reaches the head's backward
        loss.backward()
        return [loss.detach(), xi.grad] + [p.grad.clone() for p in fused.parameters()]

    a = grads(lambda xi: cb.GroupSumCrossEntropy(k, tau)(fused(xi), lab))
    b = grads(lambda xi: fused.cross_entropy(xi, lab, k, tau))
    if batch % 4:
        for u, v in zip(a, b):
            assert torch.equal(u, v)
    else:
        assert abs(float(a[0]) - float(b[0])) <= 1e-6 * abs(float(a[0]))
        for i, (u, v) in enumerate(zip(a[1:], b[1:])):
            assert_close(v, u, 1e-5, f"gradient {i}")
