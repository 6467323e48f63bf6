"""ConvLogicLayer / PoolLogicLayer with the reference's constructor and state layout
(src/convlogic/convlogic_layer.py:85-160, 455-480), computed by the sm_100a kernels.

Parameter ``weights`` ``[C_out, 7 if complete else 4, 16]`` and buffer ``selection`` int32
``[C_out, 8]`` keep the reference's names, shapes and dtypes, so state dicts interchange.
``implementation`` is accepted for signature compatibility; only ``"cuda"`` exists here.
"""

import torch
from torch import nn

from . import ops
from ._lib import W_ARGMAX, W_SOFTMAX
from .functional import ConvLogicFunction, FullConvLogicFunction, GradFactor
from .packbitstensor import PackBitsTensor


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class ConvLogicLayer(nn.Module):
    """8 taps per output channel -> 4 gates, and with ``complete=True`` -> 2 -> 1 gate -> 2x2 max pool."""

    def __init__(self, in_channels, out_channels, stride=1, padding=1, kernel=3, groups=1, selection=None,
                 residual_init=False, implementation="cuda", grad_factor=1.0, complete=False,
                 return_intermediate=False, return_indices=False):
        super().__init__()
        if implementation != "cuda":
            raise ValueError(f"convlogic_b200 only provides the CUDA implementation, got {implementation!r}")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.stride, self.padding, self.kernel = _pair(stride), _pair(padding), _pair(kernel)
        self.groups, self.grad_factor, self.complete = groups, grad_factor, complete
        self.return_intermediate, self.return_indices = return_intermediate, return_indices
        self.input_bits = 8
        self.implementation = implementation

        gates = 7 if complete else 4
        if residual_init:  # favour gate 3 ("A"): soft-max weight 0.908
            w = torch.zeros(out_channels, gates, 16)
            w[..., 3] = 5.0
        else:
            w = torch.randn(out_channels, gates, 16)
        self.weights = nn.Parameter(w)
        if selection is None:
            selection = self.generate_selection()
        assert selection.shape == (out_channels, 8)
        self.register_buffer("selection", selection.to(torch.int32))

    # -- forward -------------------------------------------------------------------------------
    def forward(self, x):
        if isinstance(x, PackBitsTensor):
            return self.forward_cuda_eval(x)
        x = x.contiguous()
        if self.grad_factor != 1.0:
            x = GradFactor.apply(x, self.grad_factor)
        return self.forward_cuda(x)

    def forward_cuda(self, x):
        if not x.is_cuda:
            raise RuntimeError("CUDA implementation requested, but the input is not a CUDA tensor.")
        wmode = W_SOFTMAX if self.training else W_ARGMAX
        w = self.weights if self.weights.dtype == x.dtype else self.weights.to(x.dtype)
        sel = self.selection.contiguous()
        geom = (*self.stride, *self.padding, *self.kernel)
        if self.complete:
            return FullConvLogicFunction.apply(x, w, sel, *geom, self.return_intermediate, self.return_indices, wmode,
                                               getattr(self, "output_feature_major", False) and self.training)
        return ConvLogicFunction.apply(x, w, sel, *geom, wmode)

    def forward_cuda_eval(self, x: PackBitsTensor):
        """Discretised block on bit-packed activations ``[C_in, H, W, words]`` (returns a new
        PackBitsTensor ``[C_out, H_out/2, W_out/2, words]``)."""
        assert not self.training, "PackBitsTensor is not supported for the differentiable training mode."
        assert self.complete, "packed inference is defined for the complete block"
        gate_ids = self._gate_ids()
        geom = (*self.stride, *self.padding, *self.kernel)
        sel = self.selection.contiguous()
        if not x.slab:
            assert x.t.dim() == 4 and x.t.shape[0] == self.in_channels, (tuple(x.t.shape), self.in_channels)
        # The slab layout (one contiguous image per channel and 128-sample slab) is what the fast kernel wants;
        # activations stay in it from block to block and return to rows at Flatten / GroupSum.
        h, w = (x.t.shape[2], x.t.shape[3]) if x.slab else (x.t.shape[1], x.t.shape[2])
        ho = (h + 2 * self.padding[0] - self.kernel[0]) // self.stride[0] + 1
        wo = (w + 2 * self.padding[1] - self.kernel[1]) // self.stride[1] + 1
        fits = self.stride == (1, 1) and ho > 0 and wo > 0 and ho % 2 == 0 and wo % 2 == 0 and (ho // 2) * (wo // 2) <= 256
        slab = x.t if x.slab else (ops.packed_to_slab(x.t) if fits else None)
        if slab is not None and fits:
            assert slab.shape[0] == self.in_channels, (tuple(slab.shape), self.in_channels)
            try:
                return PackBitsTensor.from_packed(ops.packed_convtree_slab(slab, gate_ids, sel, geom), x.pad_len, slab=True)
            except ValueError:
                pass  # a tile the kernel cannot hold in shared memory: the rows-layout kernel takes any shape
        y = ops.packed_convtree(x.rows(), gate_ids, sel, geom)
        return PackBitsTensor.from_packed(y, x.pad_len)

    def unpack_selection(self, selection):
        return (selection >> 16) & 0xFFFF, (selection >> 8) & 0xFF, selection & 0xFF

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
        return f"in_channels={self.in_channels}, out_channels={self.out_channels}, groups={self.groups}"

    # -- connectivity --------------------------------------------------------------------------
    def generate_selection(self):
        """Random taps: each output channel draws two input channels from its group, each of its 8
        taps one of the two and a (row, col) in the kernel window; the second tap of a pair is
        re-drawn while it coincides with the first (src/convlogic/convlogic_layer.py:377-452).
        The global torch RNG is consumed in the reference's order, so equal seeds give equal taps."""
        dev = self.weights.device
        kh, kw = self.kernel
        cout, cin, groups = self.out_channels, self.in_channels, self.groups
        sizes = torch.full((groups,), cin // groups, device=dev)
        sizes[: cin % groups] += 1
        starts = torch.cat([torch.zeros(1, device=dev), sizes.cumsum(0)])[:-1].to(torch.int32)
        all_idx = torch.arange(cin, device=dev, dtype=torch.int32)
        members = [all_idx[s: s + sizes[i]] for i, s in enumerate(starts)]
        gid = torch.clamp(torch.arange(cout, device=dev) // (cout // groups), 0, groups - 1)
        chosen = torch.empty((cout, 2), dtype=torch.int32, device=dev)
        for g, chans in enumerate(members):
            rows_of_g = (gid == g).nonzero(as_tuple=True)[0]
            if rows_of_g.numel():
                for col in (0, 1):
                    chosen[rows_of_g, col] = chans[torch.randint(0, chans.numel(), (rows_of_g.numel(),), device=dev)]
        pick = torch.randint(0, 2, (cout, 8), device=dev, dtype=torch.int32)
        ch = torch.where(pick == 0, chosen[:, :1].expand(-1, 8), chosen[:, 1:].expand(-1, 8))
        rows = torch.randint(0, kh, (cout, 8), device=dev, dtype=torch.int32)
        cols = torch.randint(0, kw, (cout, 8), device=dev, dtype=torch.int32)
        for k in range(0, 8, 2):
            clash = (ch[:, k] == ch[:, k + 1]) & (rows[:, k] == rows[:, k + 1]) & (cols[:, k] == cols[:, k + 1])
            for i in clash.nonzero(as_tuple=True)[0].tolist():
                while True:
                    r = torch.randint(0, kh, (1,), device=dev, dtype=torch.int32)
                    c = torch.randint(0, kw, (1,), device=dev, dtype=torch.int32)
                    if (r.item(), c.item()) != (rows[i, k].item(), cols[i, k].item()):
                        rows[i, k + 1], cols[i, k + 1] = r, c
                        break
        return (ch << 16) | (rows << 8) | cols


class PoolLogicLayer(nn.Module):
    """2x2 max pool = OR on binary activations (src/convlogic/convlogic_layer.py:455-480)."""

    def __init__(self, kernel=2, stride=2, return_indices=False):
        super().__init__()
        self.kernel, self.stride, self.return_indices = _pair(kernel), _pair(stride), return_indices

    def forward(self, x):
        if x.ndim == 5:
            if x.size(4) != 1:
                raise ValueError(f"Expected last dim=1, got {x.size(4)}")
            x = x.view(*x.shape[:4])
        elif x.ndim != 4:
            raise ValueError("Input must be 4D or 5D")
        return nn.functional.max_pool2d(x, self.kernel, self.stride, return_indices=self.return_indices)
