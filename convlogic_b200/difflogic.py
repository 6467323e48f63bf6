"""Flat LogicLayer and GroupSum with the reference's constructor and state layout
(src/difflogic/difflogic.py:14-211).

Buffers ``indices_0`` / ``indices_1`` (int64 ``[out]``) and the consumer lists
``given_x_indices_of_y_start`` / ``given_x_indices_of_y`` keep their names, shapes and dtypes.
The consumer lists are built with a stable sort instead of the reference's per-neuron Python
loop (same result, seconds instead of minutes for million-neuron layers).
"""

import torch

from . import ops
from ._lib import W_ARGMAX, W_SOFTMAX
from .functional import (GradFactor, GroupSumCrossEntropyFunction, GroupSumFunction, LogicLayerCudaFunction,
                         LogicTreeCrossEntropyFunction, LogicTreeFunction, to_feature_major)
from .packbitstensor import PackBitsTensor


def get_unique_connections(in_dim, out_dim):
    """Pairs (0,1),(2,3),..., then (1,2),(3,4),..., then growing offsets, shuffled
    (src/difflogic/functional.py:77-125)."""
    assert out_dim * 2 >= in_dim, (
        f"The number of neurons ({out_dim}) must not be smaller than half of the number of inputs "
        f"({in_dim}) because otherwise not all inputs could be used or considered.")
    x = torch.arange(in_dim).long()

    def trimmed(a, b):
        m = min(a.shape[0], b.shape[0])
        return a[:m], b[:m]

    a, b = trimmed(x[::2], x[1::2])
    if a.shape[0] < out_dim:
        a2, b2 = trimmed(x[1::2], x[2::2])
        a, b = trimmed(torch.cat([a, a2]), torch.cat([b, b2]))
    offset = 2
    while out_dim > a.shape[0] > offset:
        a, b = torch.cat([a, x[:-offset]]), torch.cat([b, x[offset:]])
        offset += 1
    if a.shape[0] < out_dim:
        raise AssertionError((a.shape[0], offset, out_dim))
    perm = torch.randperm(out_dim)
    return a[:out_dim][perm].contiguous(), b[:out_dim][perm].contiguous()


class LogicLayer(torch.nn.Module):
    def __init__(self, in_dim, out_dim, grad_factor=1.0, implementation=None, connections="random",
                 residual_init=False):
        super().__init__()
        if implementation not in (None, "cuda"):
            raise ValueError(f"convlogic_b200 only provides the CUDA implementation, got {implementation!r}")
        if residual_init:
            w = torch.zeros(out_dim, 16)
            w[:, 3] = 5.0
        else:
            w = torch.randn(out_dim, 16)
        self.weights = torch.nn.Parameter(w)
        self.in_dim, self.out_dim, self.grad_factor = in_dim, out_dim, grad_factor
        self.implementation = "cuda"
        self.connections = connections
        assert connections in ("random", "unique"), connections
        a, b = self.get_connections(connections)
        self.register_buffer("indices_0", a.to(torch.int64))
        self.register_buffer("indices_1", b.to(torch.int64))
        start, cons = self.build_consumer_lists(self.indices_0, self.indices_1, in_dim)
        self.register_buffer("given_x_indices_of_y_start", start)
        self.register_buffer("given_x_indices_of_y", cons)
        self.num_neurons = self.num_weights = out_dim

    @staticmethod
    def build_consumer_lists(a, b, in_dim):
        """CSR of 'which neurons read input feature i', neurons ascending, a neuron listed twice when
        both inputs are feature i (what the loop at src/difflogic/difflogic.py:71-87 produces)."""
        out = a.shape[0]
        feat = torch.stack([a, b], 1).reshape(-1).cpu()
        neuron = torch.arange(out, dtype=torch.int64).repeat_interleave(2)
        order = torch.sort(feat, stable=True).indices
        counts = torch.bincount(feat, minlength=in_dim)
        start = torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)])
        return start.to(a.device), neuron[order].to(a.device)

    def forward(self, x):
        if isinstance(x, PackBitsTensor):
            assert not self.training, "PackBitsTensor is not supported for the differentiable training mode."
            return self.forward_cuda_eval(x)
        if self.grad_factor != 1.0:
            x = GradFactor.apply(x, self.grad_factor)
        return self.forward_cuda(x)

    def forward_cuda(self, x):
        assert x.is_cuda, f"x must be a CUDA tensor, got device: {x.device}"
        assert x.ndim == 2, x.ndim
        x = to_feature_major(x)  # free when x came from another LogicLayer
        assert x.shape[0] == self.in_dim, (x.shape, self.in_dim)
        w = self.weights if self.weights.dtype == x.dtype else self.weights.to(x.dtype)
        args = (x, self.indices_0, self.indices_1, w, self.given_x_indices_of_y_start, self.given_x_indices_of_y)
        if self.training:
            return LogicLayerCudaFunction.apply(*args, W_SOFTMAX).transpose(0, 1)
        with torch.no_grad():
            return LogicLayerCudaFunction.apply(*args, W_ARGMAX).transpose(0, 1)

    def forward_cuda_eval(self, x: PackBitsTensor):
        """Packed inference; returns a new PackBitsTensor (the reference rebinds ``x.t``)."""
        assert not self.training
        t = x.rows()
        t = t.reshape(-1, t.shape[-1])
        assert t.shape[0] == self.in_dim, (tuple(t.shape), self.in_dim)
        gate_ids = self._gate_ids()
        y = ops.packed_logic(t, self.indices_0, self.indices_1, gate_ids)
        return PackBitsTensor.from_packed(y, x.pad_len)

    def _gate_ids(self):
        """uint8 arg-max gate of every neuron for packed inference, cached until the logits change (in-place
        updates bump the tensor version, re-assignment changes the storage, ``train()`` drops the cache)."""
        w = self.weights
        key = (w._version, w.data_ptr(), w.device)
        cached = getattr(self, "_gate_cache", None)
        if cached is None or cached[0] != key:
            cached = (key, w.detach().argmax(-1).to(torch.uint8))
            self._gate_cache = cached
        return cached[1]

    def train(self, mode=True):
        self._gate_cache = None
        return super().train(mode)

    def extra_repr(self):
        return "{}, {}, {}".format(self.in_dim, self.out_dim, "train" if self.training else "eval")

    def get_connections(self, connections):
        assert self.out_dim * 2 >= self.in_dim, (
            f"The number of neurons ({self.out_dim}) must not be smaller than half of the "
            f"number of inputs ({self.in_dim}) because otherwise not all inputs could be "
            "used or considered.")
        if connections == "random":
            # same draws, in the same order, as src/difflogic/difflogic.py:176-181
            c = torch.randperm(2 * self.out_dim) % self.in_dim
            c = torch.randperm(self.in_dim)[c].reshape(2, self.out_dim)
            return c[0].to(torch.int64), c[1].to(torch.int64)
        if connections == "unique":
            return get_unique_connections(self.in_dim, self.out_dim)
        raise ValueError(connections)


class GroupSum(torch.nn.Module):
    """Sum the outputs in k groups; float input is divided by tau, packed input gives raw int32
    counts ``[B, k]`` (src/difflogic/difflogic.py:188-211)."""

    def __init__(self, k: int, tau: float = 1.0):
        super().__init__()
        self.k, self.tau = k, tau

    def forward(self, x):
        if isinstance(x, PackBitsTensor):
            return x.group_sum(self.k)
        assert x.shape[-1] % self.k == 0, (x.shape, self.k)
        if x.is_cuda and x.dim() == 2 and x.dtype in (torch.float32, torch.float64) and x.numel() and x.t().is_contiguous():
            # the transposed view a LogicLayer returns: sum its feature-major storage directly
            return GroupSumFunction.apply(x.t(), self.k, self.tau)
        return x.reshape(*x.shape[:-1], self.k, x.shape[-1] // self.k).sum(-1) / self.tau

    def extra_repr(self):
        return f"k={self.k}, tau={self.tau}"


class GroupSumCrossEntropy(torch.nn.Module):
    """``cross_entropy(GroupSum(k, tau)(x), labels)`` (mean reduction) as one module -- the tail of the reference's
    training step (src/convlogic/model.py:137-152).  On the transposed view a ``LogicLayer`` returns, the class sums, the
    loss and the gradient w.r.t. the scores come from two kernels and the backward is one broadcast kernel; any other
    input takes the torch expression."""

    def __init__(self, k: int, tau: float = 1.0):
        super().__init__()
        self.k, self.tau = k, tau

    def forward(self, x, labels):
        assert x.shape[-1] % self.k == 0, (x.shape, self.k)
        if (x.is_cuda and x.dim() == 2 and x.dtype == torch.float32 and x.numel() and x.t().is_contiguous() and self.k <= 32
                and labels.dtype == torch.int64):
            return GroupSumCrossEntropyFunction.apply(x.t(), labels, self.k, self.tau)
        scores = x.reshape(*x.shape[:-1], self.k, x.shape[-1] // self.k).sum(-1) / self.tau
        return torch.nn.functional.cross_entropy(scores, labels)

    def extra_repr(self):
        return f"k={self.k}, tau={self.tau}"


class FusedLogicLayers(torch.nn.Module):
    """Three consecutive ``LogicLayer`` s run as one kernel per pass in training (float) mode.

    When every output of a layer is read at most once by the next one -- the stacks of the reference's models halve
    their width, and ``randperm(2 * out) % in`` then uses every output exactly once -- a neuron of the last layer
    is a gate tree over 8 features of the first layer's input, and the two intermediate activations (the largest
    tensors of the flat stack) need not exist.  The three layers stay what they are (same parameters and buffers,
    reachable as ``self.layers``); packed inference and any input the fused path does not cover run through them
    one after the other.  Opt-in: see ``fuse_logic_layers``."""

    def __init__(self, layers):
        super().__init__()
        layers = list(layers)
        if len(layers) != 3 or not all(isinstance(l, LogicLayer) for l in layers):
            raise ValueError("FusedLogicLayers takes exactly three LogicLayers")
        for prev, nxt in zip(layers[:-1], layers[1:]):
            if prev.out_dim != nxt.in_dim:
                raise ValueError("the layers do not follow each other")
            used = torch.cat([nxt.indices_0, nxt.indices_1])
            if used.unique().numel() != used.numel():
                raise ValueError("a layer's output is read more than once by the next layer: fusing would recompute it")
        self.layers = torch.nn.ModuleList(layers)
        self.in_dim, self.out_dim = layers[0].in_dim, layers[-1].out_dim
        idx = [(l.indices_0.long().cpu(), l.indices_1.long().cpu()) for l in layers]
        n2 = torch.arange(self.out_dim)[:, None]                                  # third-layer neuron of every tree
        n1 = torch.stack([idx[2][0][n2], idx[2][1][n2]], -1).reshape(self.out_dim, 2)   # its two second-layer neurons
        n0 = torch.stack([idx[1][0][n1], idx[1][1][n1]], -1).reshape(self.out_dim, 4)   # their four first-layer neurons
        leaf = torch.stack([idx[0][0][n0], idx[0][1][n0]], -1).reshape(self.out_dim, 8)
        node = torch.cat([n0, n1, n2], 1)
        # every neuron of the first two layers sits in some tree (true of the models' halving stacks): the backward kernel
        # then writes every gate gradient, and the buffers it is given need no clearing
        self.covers_all = bool(n0.unique().numel() == layers[0].out_dim and n1.unique().numel() == layers[1].out_dim)
        order = torch.sort(leaf.reshape(-1), stable=True)                          # leaf slots grouped by feature
        start = torch.zeros(self.in_dim + 1, dtype=torch.int64)
        start[1:] = torch.cumsum(torch.bincount(leaf.reshape(-1), minlength=self.in_dim), 0)
        dev = layers[0].indices_0.device
        self.register_buffer("leaf", leaf.to(torch.int32).to(dev), persistent=False)
        self.register_buffer("node", node.to(torch.int32).to(dev), persistent=False)
        self.register_buffer("leaf_start", start.to(dev), persistent=False)
        self.register_buffer("leaf_slots", order.indices.to(torch.int32).to(dev), persistent=False)

    def forward(self, x):
        first = self.layers[0]
        fused = (not isinstance(x, PackBitsTensor) and x.is_cuda and x.dtype == torch.float32 and x.dim() == 2
                 and all(l.grad_factor == 1.0 for l in self.layers) and x.shape[0] > 0)
        if not fused:
            for layer in self.layers:
                x = layer(x)
            return x
        assert x.shape[1] == first.in_dim, (x.shape, first.in_dim)
        x_fm = to_feature_major(x)
        w = [l.weights for l in self.layers]
        if self.training:
            y = LogicTreeFunction.apply(x_fm, w[0], w[1], w[2], self.leaf, self.node, self.leaf_start, self.leaf_slots, W_SOFTMAX, self.covers_all)
        else:
            with torch.no_grad():
                y = LogicTreeFunction.apply(x_fm, w[0], w[1], w[2], self.leaf, self.node, self.leaf_start, self.leaf_slots, W_ARGMAX, self.covers_all)
        return y.transpose(0, 1)

    def cross_entropy(self, x, labels, k, tau=1.0):
        """``cross_entropy(GroupSum(k, tau)(self(x)), labels)`` of a training step as one autograd node: same loss and
        gradients as the three calls (src/convlogic/model.py:137-152), but the gradient tensor between the flat layers
        and the class sums is never materialised.  Falls back to the separate modules for inputs the fused path does not
        take (see ``forward``), for eval mode and for more than 32 classes."""
        fused = (self.training and not isinstance(x, PackBitsTensor) and x.is_cuda and x.dtype == torch.float32 and x.dim() == 2
                 and all(l.grad_factor == 1.0 for l in self.layers) and x.shape[0] > 0 and k <= 32 and self.out_dim % k == 0
                 and labels.dtype == torch.int64)
        if not fused:
            return GroupSumCrossEntropy(k, tau)(self(x), labels)
        assert x.shape[1] == self.layers[0].in_dim, (x.shape, self.layers[0].in_dim)
        w = [l.weights for l in self.layers]
        return LogicTreeCrossEntropyFunction.apply(to_feature_major(x), w[0], w[1], w[2], self.leaf, self.node, self.leaf_start,
                                                   self.leaf_slots, labels, k, float(tau), self.covers_all)

    def extra_repr(self):
        return f"{self.in_dim} -> {' -> '.join(str(l.out_dim) for l in self.layers)}"


def fuse_logic_layers(model, feature_major_blocks=True):
    """A copy of an ``nn.Sequential`` in which every run of three LogicLayers that can be fused is replaced by a
    ``FusedLogicLayers`` over the SAME layer objects (parameters are shared with ``model``).

    ``feature_major_blocks``: a fused ConvLogic block that sits right in front of ``Flatten`` + flat layers is asked to
    write its training output in the flat layers' layout (``output_feature_major`` on that -- shared -- layer object): what
    it returns is then a non-contiguous [N, C, h, w] view whose ``flatten(1)`` the flat layers take without a copy, and the
    gradient comes back the same way."""
    out, run = [], []

    def flush():
        while len(run) >= 3:
            try:
                out.append(FusedLogicLayers(run[:3]))
                del run[:3]
            except ValueError:
                out.append(run.pop(0))
        out.extend(run)
        run.clear()

    for m in model:
        if isinstance(m, LogicLayer):
            run.append(m)
        else:
            flush()
            out.append(m)
    flush()
    if feature_major_blocks:
        for i in range(2, len(out)):
            if (isinstance(out[i], (FusedLogicLayers, LogicLayer)) and isinstance(out[i - 1], torch.nn.Flatten)
                    and type(out[i - 2]).__name__ == "ConvLogicLayer" and getattr(out[i - 2], "complete", False)):
                out[i - 2].output_feature_major = True
    return torch.nn.Sequential(*out)
