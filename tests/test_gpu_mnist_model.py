"""mnist_s-shaped stack at batch 256 against class scores produced by the reference's CPU path."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_mnist_s_scores_match_reference(golden):
    import convlogic_b200 as cb
    from tests.golden.make_golden import mnist_inputs, mnist_set_logits

    g = golden("mnist_s")
    torch.manual_seed(0)  # the constructors draw connections in the reference's order
    model = cb.ConvLogicMnistModel(k_param=16, tau=6.5)
    net = model.network
    mnist_set_logits(net)
    convs = [m for m in net if isinstance(m, cb.ConvLogicLayer)]
    flats = [m for m in net if isinstance(m, cb.LogicLayer)]
    checks = [float(m.weights.detach().double().sum()) for m in net if hasattr(m, "weights")]
    np.testing.assert_allclose(checks, g["logit_checksum"], rtol=1e-12)
    for i, m in enumerate(convs):  # connections: fixture values are authoritative
        assert np.array_equal(m.selection.numpy(), g[f"conv{i}/selection"]), "selection differs from the reference's"
    for i, m in enumerate(flats):
        assert np.array_equal(m.indices_0.numpy(), g[f"flat{i}/a"]) and np.array_equal(m.indices_1.numpy(), g[f"flat{i}/b"])
    net = net.cuda()
    x = mnist_inputs().cuda()
    with torch.no_grad():
        net.train()
        soft = net(x).cpu().numpy()
        net.eval()
        hard = net(x).cpu().numpy()
        packed = net(cb.PackBitsTensor(x > 0.5, 64)).cpu().numpy()
    rel = np.abs(soft - g["scores_soft"]).max() / np.abs(g["scores_soft"]).max()
    assert rel < 1e-5, rel
    # hard scores are integer gate counts / tau; the counts must agree exactly (the division itself
    # rounds differently on CPU and GPU in the last bit)
    want_counts = np.rint(g["scores_hard"].astype(np.float64) * 6.5).astype(np.int32)
    assert np.abs(g["scores_hard"].astype(np.float64) * 6.5 - want_counts).max() < 1e-3
    assert np.array_equal(np.rint(hard.astype(np.float64) * 6.5).astype(np.int32), want_counts)
    assert np.abs(hard - g["scores_hard"]).max() < 1e-5
    assert packed.dtype == np.int32 and np.array_equal(packed, want_counts)
