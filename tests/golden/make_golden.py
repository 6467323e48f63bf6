"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE'S OWN CPU PATH.

Run once, on a machine that has a checkout of lkorinek/convlogic:

    python tests/golden/make_golden.py --reference /path/to/convlogic [--mnist] [--jobs 8]

The reference package ``convlogic`` cannot be imported as a package without
pytorch_lightning (its ``__init__`` pulls the Lightning module in), so the two layer files
are loaded by path; ``difflogic`` imports cleanly.  All layers are built with
``implementation="python"`` (convlogic_layer.py:231-316, treelogic_layer.py:110-127,
difflogic.py:112-123) and gradients come from torch autograd through that path.

Outputs (``.npz``, a few hundred KB in total):
  fused_block.npz   ConvLogicLayer(complete=True): soft/hard outputs and autograd gradients
  split_layers.npz  ConvLogicLayer(complete=False), TreeLogicLayer, PoolLogicLayer
  flat_layers.npz   LogicLayer (+ GroupSum): soft/hard outputs and autograd gradients
  mnist_s.npz       (--mnist) the mnist_s-shaped stack at batch 256: connections and logits
                    checksums plus the soft and hard class scores

The tests never read the reference; they read these files.
"""

import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    src = os.path.join(root, "src")
    sys.path.insert(0, src)
    import difflogic  # noqa: F401  (imports cleanly; its CUDA module is absent)

    def by_path(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(src, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    cl = by_path("ref_convlogic_layer", "convlogic/convlogic_layer.py")
    tl = by_path("ref_treelogic_layer", "convlogic/treelogic_layer.py")
    return cl, tl, difflogic


def seeded_logits(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g)


FUSED_CASES = [
    # name, N, Ci, C, H, W, stride, pad, kernel, input kind
    ("s1p1k3_randn", 4, 3, 2, 8, 8, 1, 1, 3, "randn"),
    ("s1p0k3_randn", 4, 3, 2, 8, 8, 1, 0, 3, "randn"),
    ("s2p2k4_rand", 3, 3, 3, 6, 6, 2, 2, 4, "rand"),
    ("s1p0k5_bits", 3, 1, 4, 12, 12, 1, 0, 5, "bits"),
    ("s1p1k3_bits", 2, 5, 6, 8, 12, 1, 1, 3, "bits"),
    ("rect", 2, 2, 3, 9, 9, (1, 2), (1, 2), (2, 3), "rand"),
]


def make_input(kind, shape, seed):
    g = torch.Generator().manual_seed(seed)
    if kind == "randn":
        return torch.randn(*shape, generator=g)
    if kind == "rand":
        return torch.rand(*shape, generator=g)
    return (torch.rand(*shape, generator=g) < 0.5).float()


def gen_fused(cl, out):
    for i, (name, n, ci, c, h, w, st, pd, k, kind) in enumerate(FUSED_CASES):
        torch.manual_seed(100 + i)
        layer = cl.ConvLogicLayer(ci, c, stride=st, padding=pd, kernel=k, complete=True, implementation="python")
        layer.weights.data = seeded_logits((c, 7, 16), 200 + i)
        x = make_input(kind, (n, ci, h, w), 300 + i)
        for dt, tag in ((torch.float32, "f32"), (torch.float64, "f64")):
            lay = layer.double() if dt == torch.float64 else layer.float()
            xx = x.to(dt).clone().requires_grad_(True)
            lay.train()
            lay.weights.grad = None
            y = lay(xx)
            gy = make_input("randn", tuple(y.shape), 400 + i).to(dt)
            (y * gy).sum().backward()
            out[f"{name}/{tag}/y_soft"] = y.detach().numpy()
            out[f"{name}/{tag}/gx"] = xx.grad.numpy()
            out[f"{name}/{tag}/gw_logits"] = lay.weights.grad.numpy().copy()
            lay.eval()
            with torch.no_grad():
                out[f"{name}/{tag}/y_hard"] = lay(xx.detach()).numpy()
        out[f"{name}/x"] = x.numpy()
        out[f"{name}/gy"] = gy.float().numpy()
        out[f"{name}/logits"] = layer.float().weights.detach().numpy()
        out[f"{name}/selection"] = layer.selection.numpy()
        out[f"{name}/geom"] = np.array(
            [*((st, st) if isinstance(st, int) else st), *((pd, pd) if isinstance(pd, int) else pd),
             *((k, k) if isinstance(k, int) else k)], dtype=np.int32)
        print("fused", name, tuple(y.shape))


def gen_split(cl, tl, out):
    torch.manual_seed(7)
    n, ci, c, h, w = 3, 3, 2, 10, 10
    for j, (st, pd) in enumerate([(1, 1), (2, 2)]):
        conv = cl.ConvLogicLayer(ci, c, stride=st, padding=pd, kernel=3, complete=False, implementation="python")
        t1 = tl.TreeLogicLayer(c, 4, implementation="python")
        t2 = tl.TreeLogicLayer(c, 2, implementation="python")
        pool = cl.PoolLogicLayer(return_indices=True)
        x = make_input("randn", (n, ci, h, w), 500 + j).requires_grad_(True)
        for mode in ("soft", "hard"):
            for m in (conv, t1, t2):
                m.train(mode == "soft")
                m.weights.grad = None
            x.grad = None
            x1 = conv(x)
            x2 = t1(x1)
            x3 = t2(x2)
            y, idx = pool(x3)
            pre = f"split{j}/{mode}"
            out[f"{pre}/x1"], out[f"{pre}/x2"], out[f"{pre}/x3"] = (v.detach().numpy() for v in (x1, x2, x3))
            out[f"{pre}/y"], out[f"{pre}/idx"] = y.detach().numpy(), idx.flatten(2).numpy().astype(np.int32)
            if mode == "soft":
                g1 = make_input("randn", tuple(x1.shape), 600 + j)
                gx, gwc = torch.autograd.grad((x1 * g1).sum(), (x, conv.weights), retain_graph=True)
                out[f"split{j}/g_x1"], out[f"split{j}/conv_gx"], out[f"split{j}/conv_gw_logits"] = (
                    g1.numpy(), gx.numpy(), gwc.numpy())
                g2 = make_input("randn", tuple(x2.shape), 700 + j)
                x1d = x1.detach().requires_grad_(True)
                x2b = t1(x1d)
                gx1, gwt = torch.autograd.grad((x2b * g2).sum(), (x1d, t1.weights))
                out[f"split{j}/g_x2"], out[f"split{j}/tree_gx"], out[f"split{j}/tree_gw_logits"] = (
                    g2.numpy(), gx1.numpy(), gwt.numpy())
        out[f"split{j}/x"] = x.detach().numpy()
        out[f"split{j}/conv_logits"] = conv.weights.detach().numpy()
        out[f"split{j}/tree1_logits"] = t1.weights.detach().numpy()
        out[f"split{j}/tree2_logits"] = t2.weights.detach().numpy()
        out[f"split{j}/selection"] = conv.selection.numpy()
        out[f"split{j}/geom"] = np.array([st, st, pd, pd, 3, 3], dtype=np.int32)
        print("split", j)


def gen_flat(dl, out):
    for j, (b, i_dim, o_dim, k, tau, conn) in enumerate(
        [(5, 16, 40, 10, 3.5, "random"), (33, 24, 60, 10, 1.0, "unique"), (1024 + 7, 8, 32, 4, 2.0, "random")]
    ):
        torch.manual_seed(900 + j)
        layer = dl.LogicLayer(i_dim, o_dim, implementation="python", connections=conn)
        gs = dl.GroupSum(k, tau)
        x = make_input("rand" if j else "bits", (b, i_dim), 910 + j).requires_grad_(True)
        layer.train()
        y = layer(x)
        s = gs(y)
        gy = make_input("randn", tuple(y.shape), 920 + j)
        gx, gw = torch.autograd.grad((y * gy).sum(), (x, layer.weights))
        layer.eval()
        with torch.no_grad():
            yh = layer(x.detach())
        pre = f"flat{j}"
        out[f"{pre}/x"], out[f"{pre}/logits"] = x.detach().numpy(), layer.weights.detach().numpy()
        out[f"{pre}/a"], out[f"{pre}/b"] = layer.indices_0.numpy(), layer.indices_1.numpy()
        out[f"{pre}/y_soft"], out[f"{pre}/y_hard"] = y.detach().numpy(), yh.numpy()
        out[f"{pre}/group_sum"] = s.detach().numpy()
        out[f"{pre}/gy"], out[f"{pre}/gx"], out[f"{pre}/gw_logits"] = gy.numpy(), gx.numpy(), gw.numpy()
        out[f"{pre}/k_tau"] = np.array([k, tau], dtype=np.float64)
        print("flat", j)
    # the reference tests' known-answer vector: every gate on the four input pairs
    # (tests/difflogic/test_difflogic_forward.py:74-100, tests/convlogic/test_treelogic_forward.py:66-86)
    a = torch.tensor([0.0, 0.0, 1.0, 1.0])
    b = torch.tensor([0.0, 1.0, 0.0, 1.0])
    out["truth_table"] = np.stack([dl.functional.bin_op(a, b, i).numpy() for i in range(16)])


def build_mnist_s(cl, dl, k=16, tau=6.5):
    """The layer stack of ConvLogicMnistModel (src/convlogic/model.py:64-109)."""
    C = cl.ConvLogicLayer
    kw = dict(residual_init=True, complete=True, implementation="python")
    return torch.nn.Sequential(
        C(1, k, kernel=5, padding=0, **kw),
        C(k, 3 * k, kernel=3, padding=1, **kw),
        C(3 * k, 9 * k, kernel=3, padding=1, **kw),
        torch.nn.Flatten(),
        dl.LogicLayer(81 * k, 1280 * k, residual_init=True, implementation="python"),
        dl.LogicLayer(1280 * k, 640 * k, residual_init=True, implementation="python"),
        dl.LogicLayer(640 * k, 320 * k, residual_init=True, implementation="python"),
        dl.GroupSum(k=10, tau=tau),
    )


def mnist_inputs(batch=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(batch, 1, 28, 28, generator=g) < 0.2).float()


def mnist_set_logits(net, seed=1):
    g = torch.Generator().manual_seed(seed)
    for m in net:
        if hasattr(m, "weights"):
            m.weights.data = torch.randn(*m.weights.shape, generator=g)


def _mnist_worker(args):
    root, lo, hi = args
    torch.set_num_threads(1)
    cl, _, dl = load_reference(root)
    torch.manual_seed(0)
    net = build_mnist_s(cl, dl)
    mnist_set_logits(net)
    x = mnist_inputs()[lo:hi]
    res = []
    with torch.no_grad():
        for training in (True, False):
            net.train(training)
            res.append(net(x).numpy())
    return lo, res[0], res[1]


def gen_mnist(root, jobs):
    import multiprocessing as mp

    cl, _, dl = load_reference(root)
    torch.manual_seed(0)
    net = build_mnist_s(cl, dl)
    mnist_set_logits(net)
    out = {}
    convs = [m for m in net if isinstance(m, cl.ConvLogicLayer)]
    flats = [m for m in net if isinstance(m, dl.LogicLayer)]
    for i, m in enumerate(convs):
        out[f"conv{i}/selection"] = m.selection.numpy()
    for i, m in enumerate(flats):
        out[f"flat{i}/a"] = m.indices_0.numpy().astype(np.int32)
        out[f"flat{i}/b"] = m.indices_1.numpy().astype(np.int32)
    out["logit_checksum"] = np.array(
        [float(m.weights.double().sum()) for m in net if hasattr(m, "weights")], dtype=np.float64)
    step = 256 // jobs
    chunks = [(root, lo, min(256, lo + step)) for lo in range(0, 256, step)]
    with mp.get_context("spawn").Pool(jobs) as pool:
        parts = sorted(pool.map(_mnist_worker, chunks))
    out["scores_soft"] = np.concatenate([p[1] for p in parts])
    out["scores_hard"] = np.concatenate([p[2] for p in parts])
    np.savez_compressed(os.path.join(HERE, "mnist_s.npz"), **out)
    print("mnist_s", out["scores_soft"].shape)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--mnist", action="store_true")
    ap.add_argument("--only-mnist", action="store_true")
    ap.add_argument("--jobs", type=int, default=8)
    a = ap.parse_args()
    if not a.only_mnist:
        cl, tl, dl = load_reference(a.reference)
        for name, fn in (("fused_block", lambda o: gen_fused(cl, o)),
                         ("split_layers", lambda o: gen_split(cl, tl, o)),
                         ("flat_layers", lambda o: gen_flat(dl, o))):
            out = {}
            fn(out)
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    if a.mnist or a.only_mnist:
        gen_mnist(a.reference, a.jobs)


if __name__ == "__main__":
    main()
