"""TreeLogicLayer: one pairwise gate level on the trailing dimension
(src/convlogic/treelogic_layer.py:33-130).  ``weights`` is ``[channels, input_bits // 2, 16]``."""

import torch
from torch import nn

from ._lib import W_ARGMAX, W_SOFTMAX
from .functional import GradFactor, TreeLogicFunction


class TreeLogicLayer(nn.Module):
    def __init__(self, channels, input_bits, residual_init=False, implementation="cuda", grad_factor=1.0):
        super().__init__()
        assert input_bits % 2 == 0, "input_bits must be even"
        if implementation != "cuda":
            raise ValueError(f"convlogic_b200 only provides the CUDA implementation, got {implementation!r}")
        self.channels, self.input_bits = channels, input_bits
        self.implementation, self.grad_factor = implementation, grad_factor
        if residual_init:
            w = torch.zeros(channels, input_bits // 2, 16)
            w[..., 3] = 5.0
        else:
            w = torch.randn(channels, input_bits // 2, 16)
        self.weights = nn.Parameter(w)

    def forward(self, x):
        assert x.shape[-1] == self.input_bits, (
            f"Expected input last dimension to be {self.input_bits}, but got {x.shape[-1]}")
        x = x.contiguous()
        if self.grad_factor != 1.0:
            x = GradFactor.apply(x, self.grad_factor)
        w = self.weights if self.weights.dtype == x.dtype else self.weights.to(x.dtype)
        return TreeLogicFunction.apply(x, w, W_SOFTMAX if self.training else W_ARGMAX)

    def extra_repr(self):
        return f"channels={self.channels}, input_bits={self.input_bits}"
