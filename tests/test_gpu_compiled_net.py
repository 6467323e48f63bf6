"""CompiledLogicNet: the serialised network run by the library's own runtime (one C call) gives the counts of
the layer-by-layer packed path, of the float eval-mode model, and of the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _randomise(net, seed):
    g = torch.Generator().manual_seed(seed)
    for prm in net.parameters():
        prm.data = torch.randn(*prm.shape, generator=g).to(prm.device)


@pytest.mark.parametrize("batch", [1, 60, 64, 100, 128, 300])
def test_flat_stack_counts_equal_packed_layers_and_oracle(batch):
    import convlogic_b200 as cb

    torch.manual_seed(3)
    model = torch.nn.Sequential(cb.LogicLayer(96, 400), cb.LogicLayer(400, 250), cb.LogicLayer(250, 130), cb.GroupSum(10, 4.0)).cuda().eval()
    _randomise(model, 5)
    x = torch.rand(batch, 96, device="cuda") < 0.5
    net = cb.CompiledLogicNet(model).compile()
    assert (net.num_inputs, net.num_classes, net.num_layers) == (96, 10, 3)
    got = net(x)
    assert got.dtype == torch.int32 and got.shape == (batch, 10)
    with torch.no_grad():
        want = model(cb.PackBitsTensor(x, 64))
    assert torch.equal(got, want)
    # CPU oracle: packed logic per layer, then per-class bit counts
    h, pad = oracle.pack_bits(x.cpu().numpy().T, 64)
    for layer in list(model)[:-1]:
        h = oracle.packed_logic(h, layer.indices_0.cpu().numpy(), layer.indices_1.cpu().numpy(),
                                layer.weights.argmax(-1).cpu().numpy().astype(np.uint8))
    assert np.array_equal(got.cpu().numpy(), oracle.packed_group_sum(h, pad, 10))
    assert np.array_equal(net(x.cpu().numpy()).cpu().numpy(), got.cpu().numpy())  # numpy input, as the reference accepts


@pytest.mark.parametrize("batch", [70, 256])
def test_cifar_shaped_stack_equals_packed_and_float_eval(batch):
    import convlogic_b200 as cb

    torch.manual_seed(0)
    model = cb.ConvLogicCifarModel(k_param=4, input_channels=6, input_size=32, tau=8.0).cuda().eval()
    _randomise(model, 1)
    x = torch.rand(batch, 6, 32, 32, device="cuda") < 0.5
    net = cb.CompiledLogicNet(model.network, input_shape=(6, 32, 32)).compile()
    got = net(x)
    with torch.no_grad():
        assert torch.equal(got, model(cb.PackBitsTensor(x, 64)))
        assert torch.equal(got.float(), model(x.float()) * 8.0)


def test_mnist_shaped_stack_and_strided_block():
    import convlogic_b200 as cb

    torch.manual_seed(0)
    model = cb.ConvLogicMnistModel(k_param=4, tau=4.0).cuda().eval()
    _randomise(model, 2)
    x = torch.rand(130, 1, 28, 28, device="cuda") < 0.3
    net = cb.CompiledLogicNet(model.network, input_shape=(1, 28, 28)).compile()
    with torch.no_grad():
        assert torch.equal(net(x), model(cb.PackBitsTensor(x, 64)))
    # a stride-2 block (rows-layout kernel) between two stride-1 blocks (slab-layout kernel)
    seq = torch.nn.Sequential(
        cb.ConvLogicLayer(3, 8, complete=True), cb.ConvLogicLayer(8, 12, stride=2, padding=1, kernel=3, complete=True),
        cb.ConvLogicLayer(12, 10, complete=True), torch.nn.Flatten(), cb.LogicLayer(10 * 2 * 2, 60), cb.GroupSum(10, 1.0)).cuda().eval()
    _randomise(seq, 4)
    x = torch.rand(200, 3, 32, 32, device="cuda") < 0.5
    net = cb.CompiledLogicNet(seq, input_shape=(3, 32, 32)).compile()
    with torch.no_grad():
        assert torch.equal(net(x), seq(cb.PackBitsTensor(x, 64)))


def test_save_load_and_fused_pixel_input(tmp_path):
    import convlogic_b200 as cb

    torch.manual_seed(0)
    model = cb.ConvLogicCifarModel(k_param=2, input_channels=9, input_size=16, tau=1.0).cuda().eval()
    _randomise(model, 7)
    path = str(tmp_path / "net.clb")
    a = cb.CompiledLogicNet(model.network, input_shape=(9, 16, 16)).compile(save_lib_path=path)
    b = cb.CompiledLogicNet.load(path, num_classes=10)
    with pytest.raises(ValueError):
        cb.CompiledLogicNet.load(path, num_classes=7)
    pixels = torch.rand(90, 3, 16, 16)
    th = torch.tensor([0.25, 0.5, 0.75])
    bits = torch.from_numpy(oracle.thermometer(pixels.numpy(), 3))  # [90, 9, 16, 16]
    want = a(bits)
    assert torch.equal(b(bits), want)
    assert torch.equal(b.forward_pixels(pixels, th), want)
    u8 = torch.randint(0, 256, (90, 3, 16, 16), dtype=torch.uint8)
    bits8 = torch.from_numpy(oracle.thermometer((u8.float() / 255).numpy(), 3))
    assert torch.equal(a.forward_pixels(u8, th), a(bits8))
    with pytest.raises(ValueError):
        a(torch.zeros(4, 7, dtype=torch.bool))


@pytest.mark.parametrize("dims", [(64, 320, 160, 150), (96, 640, 320, 160), (50, 400, 200, 100, 50, 30)])
def test_fused_flat_layers_equal_layer_by_layer(dims):
    """Runs of flat layers that halve their width are emitted as one gate-tree layer (two or three levels): same
    counts as the unfused blob and as the module path, for batches that do and do not fill the last word."""
    import convlogic_b200 as cb
    from convlogic_b200.compiled_model import fuse_flat_layers

    torch.manual_seed(len(dims))
    layers = [cb.LogicLayer(i, o) for i, o in zip(dims[:-1], dims[1:])]
    model = torch.nn.Sequential(*layers, cb.GroupSum(10, 1.0)).cuda().eval()
    _randomise(model, 11)
    fused = cb.CompiledLogicNet(model, fuse=True).compile()
    plain = cb.CompiledLogicNet(model, fuse=False).compile()
    assert plain.num_layers == len(layers) and fused.num_layers < plain.num_layers
    for batch in (1, 64, 200):
        x = torch.rand(batch, dims[0], device="cuda") < 0.5
        with torch.no_grad():
            want = model(cb.PackBitsTensor(x, 64))
        assert torch.equal(fused(x), want) and torch.equal(plain(x), want)
    # the tables themselves, against a direct evaluation of the two layers on the CPU oracle
    leaf, ops = fuse_flat_layers(layers[:2])
    xb = (np.random.default_rng(0).random((dims[0], 70)) < 0.5)
    h, _ = oracle.pack_bits(xb, 64)
    for layer in layers[:2]:
        h = oracle.packed_logic(h, layer.indices_0.cpu().numpy(), layer.indices_1.cpu().numpy(),
                                layer.weights.argmax(-1).cpu().numpy().astype(np.uint8))
    from convlogic_b200 import _lib
    x_dev = torch.from_numpy(oracle.pack_bits(xb, 64)[0]).cuda()
    y_dev = torch.empty((dims[2], x_dev.shape[1]), dtype=torch.int64, device="cuda")
    _lib.check(_lib.lib().clb_packed_tree(_lib.ptr(x_dev), _lib.ptr(torch.from_numpy(leaf).cuda()), _lib.ptr(torch.from_numpy(ops).cuda()),
                                          _lib.ptr(y_dev), dims[0], dims[2], 2, x_dev.shape[1], 64, _lib.stream()))
    torch.cuda.synchronize()
    assert np.array_equal(y_dev.cpu().numpy(), h)


def test_graph_replay_equals_direct_calls():
    """A captured CUDA graph of one forward call replays to the same counts, for bit input and for pixel input."""
    import convlogic_b200 as cb

    torch.manual_seed(0)
    model = cb.ConvLogicMnistModel(k_param=4, tau=4.0).cuda().eval()
    _randomise(model, 9)
    net = cb.CompiledLogicNet(model.network, input_shape=(1, 28, 28)).compile()
    xs = [torch.rand(130, 1, 28, 28, device="cuda") < 0.3 for _ in range(3)]
    replay = net.capture(xs[0])
    for x in xs:
        want = net(x).clone()
        assert torch.equal(replay(x), want)
    pix_model = cb.ConvLogicCifarModel(k_param=2, input_channels=9, input_size=16, tau=1.0).cuda().eval()
    _randomise(pix_model, 10)
    pnet = cb.CompiledLogicNet(pix_model.network, input_shape=(9, 16, 16)).compile()
    th = torch.tensor([0.25, 0.5, 0.75])
    ps = [torch.randint(0, 256, (256, 3, 16, 16), dtype=torch.uint8) for _ in range(2)]
    preplay = pnet.capture(ps[0], th)
    for p_ in ps:
        assert torch.equal(preplay(p_), pnet.forward_pixels(p_, th))


@pytest.mark.parametrize("batch", [70, 128, 300])
def test_packed_rows_input(batch):
    """The runtime also takes already packed rows (padded to whole 128-sample units)."""
    import convlogic_b200 as cb

    torch.manual_seed(0)
    model = cb.ConvLogicCifarModel(k_param=2, input_channels=3, input_size=16, tau=1.0).cuda().eval()
    _randomise(model, 12)
    net = cb.CompiledLogicNet(model.network, input_shape=(3, 16, 16)).compile()
    x = torch.rand(batch, 3, 16, 16) < 0.5
    rows, _ = oracle.pack_bits(x.reshape(batch, -1).T.numpy(), 64)          # [F, ceil(batch/64)]
    words = 2 * (-(-batch // 128))
    padded = np.zeros((rows.shape[0], words), dtype=np.int64)
    padded[:, : rows.shape[1]] = rows
    assert torch.equal(net.forward_packed(torch.from_numpy(padded), batch), net(x))
    with pytest.raises(ValueError):
        net.forward_packed(torch.from_numpy(padded[:, :1].copy()), batch)
