"""Bit-packed activations for discretised inference.

Mirrors the reference's ``PackBitsTensor`` (src/difflogic/packbitstensor.py:11-43): ``.t`` is
feature-major ``[features, ceil(B / bits)]`` with sample ``bits * word + i`` in bit ``i``,
``.pad_len`` the number of pad samples, ``group_sum(k)`` the per-class bit counts and
``flatten()`` a no-op.  Two additions, both needed for ConvLogic blocks, which the reference
cannot run packed: a 4-D bool input ``[B, C, H, W]`` is packed to ``.t`` of shape
``[C, H, W, words]`` (so that ``flatten`` onto ``[C*H*W, words]`` is a free view in the same
feature order as ``nn.Flatten`` on NCHW), and the sample-major input is packed in one pass
without the transposed copy.
"""

import numpy as np
import torch

from . import ops


class PackBitsTensor:
    def __init__(self, t: torch.Tensor, bit_count: int = 32):
        assert t.dim() in (2, 4), t.shape
        self.bit_count = bit_count
        if not t.is_cuda:
            raise NotImplementedError(f"PackBitsTensor only supports CUDA tensors, but got {t.device}.")
        t = t.contiguous()
        flat = t.reshape(t.shape[0], -1)
        packed, self.pad_len = ops.pack_bits(flat, bit_count, sample_major=True)
        self.t = packed.view(*t.shape[1:], packed.shape[-1]) if t.dim() == 4 else packed
        self.slab = False

    @classmethod
    def from_packed(cls, t, pad_len, slab=False):
        """``slab=True``: ``t`` is a conv activation in the slab layout [C, U, H, W, 16 // itemsize]
        (see ``ops.packed_to_slab``) instead of [C, H, W, words]."""
        self = cls.__new__(cls)
        self.t, self.pad_len, self.bit_count, self.slab = t, pad_len, t.element_size() * 8, slab
        return self

    @classmethod
    def from_pixels(cls, pixels, thresholds, slab=None):
        """Thermometer-encode and pack images in one kernel: ``pixels`` [N, C, H, W] float32 / uint8,
        ``thresholds`` float32 [L] -> the packed ``[L*C, H, W, words]`` activation of
        ``cat([(x > t) for t in thresholds], dim=1)`` (the reference's input transform, data.py:46-50).
        ``slab=None`` picks the slab layout when the batch fills whole 128-sample units."""
        if slab is None:
            slab = (-(-pixels.shape[0] // 64)) % 2 == 0
        t, pad = ops.thermometer_pack(pixels, thresholds, slab)
        return cls.from_packed(t, pad, slab=slab)

    def rows(self):
        """The tensor in the rows layout [..., words] (converts a slab-layout activation)."""
        return ops.packed_to_rows(self.t) if self.slab else self.t

    @property
    def is_cuda(self):
        return self.t.is_cuda

    @property
    def device(self):
        return self.t.device

    def contiguous(self):
        return self

    def group_sum(self, k):
        t = self.rows()
        return ops.group_popcount(t.reshape(-1, t.shape[-1]), self.pad_len, k)

    def flatten(self, start_dim=0, end_dim=-1, **kwargs):
        """Returns the tensor itself viewed as [features, words]; arguments are ignored."""
        if self.slab or self.t.dim() != 2:
            t = self.rows()
            return PackBitsTensor.from_packed(t.reshape(-1, t.shape[-1]), self.pad_len)
        return self

    def _get_member_repr(self, member):
        rows = [np.binary_repr(int(v) & ((1 << self.bit_count) - 1), width=self.bit_count)[::-1] for v in member]
        if len(rows) <= 4:
            return " ".join(rows)
        return f"{' '.join(rows[:3])} ... {rows[-1]}"

    def __repr__(self):
        t2 = self.rows()
        t2 = t2.reshape(-1, t2.shape[-1]).cpu()
        return "\n".join(self._get_member_repr(item.tolist()) for item in t2)
