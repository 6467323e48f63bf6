"""Vectorised CPU restatement of the ConvLogic block (gather, 8->4->2->1 gate tree, 2x2 pool).

TEST INFRASTRUCTURE ONLY (see the package docstring).

Follows the reference:
  * selection word layout ``(channel << 16) | (row << 8) | col``:
    src/convlogic/convlogic_layer.py:175-179, 450-451;
  * tap gather with zeros outside the image, output size
    ``(H + 2*pad - kernel) // stride + 1``: convlogic_layer.py:248-282;
  * taps (2p, 2p+1) feed first-level gate p; gate slots 0-3 (conv), 4-5 (tree 1), 6 (tree 2),
    pairing of tree inputs by even/odd position: convlogic_layer.py:237-239, 286-314;
  * soft mode = softmax of the logits, hard mode = one-hot of their arg-max:
    convlogic_layer.py:252-257;
  * 2x2 pool keeps the FIRST maximum in the scan order (0,0),(0,1),(1,0),(1,1) and reports
    the flat index ``in_y * W_out + in_x``: src/convlogic/cuda/full_convlogic_kernel.cu:94-144.

Every function is differentiable through torch autograd, which is how the reference's own
CPU path obtains gradients; the backward oracle is ``torch.autograd.grad`` of these.
"""

import torch
import torch.nn.functional as F

from .logic_ops import bin_op_s


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def unpack_selection(sel):
    """int32 selection words -> (channel, row, col) tensors of the same shape."""
    sel = sel.to(torch.int64)
    return (sel >> 16) & 0xFFFF, (sel >> 8) & 0xFF, sel & 0xFF


def out_size(h, w, stride, padding, kernel):
    (sh, sw), (ph, pw), (kh, kw) = _pair(stride), _pair(padding), _pair(kernel)
    return (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1


def gather_taps(x, sel, stride=1, padding=1, kernel=3):
    """x [N, Ci, H, W] -> taps [N, C, Ho, Wo, 8]; taps falling outside the image read 0."""
    (sh, sw), (ph, pw) = _pair(stride), _pair(padding)
    n, _, h, w = x.shape
    ho, wo = out_size(h, w, stride, padding, kernel)
    ch, r, s = unpack_selection(sel)  # [C, 8]
    iy = torch.arange(ho).view(1, ho, 1, 1) * sh + r.view(-1, 1, 1, 8) - ph  # [C, Ho, 1, 8]
    ix = torch.arange(wo).view(1, 1, wo, 1) * sw + s.view(-1, 1, 1, 8) - pw  # [C, 1, Wo, 8]
    valid = (iy >= 0) & (iy < h) & (ix >= 0) & (ix < w)  # [C, Ho, Wo, 8]
    iyc = iy.clamp(0, h - 1).expand(-1, ho, wo, 8)
    ixc = ix.clamp(0, w - 1).expand(-1, ho, wo, 8)
    chb = ch.view(-1, 1, 1, 8).expand(-1, ho, wo, 8)
    taps = x[:, chb, iyc, ixc]  # [N, C, Ho, Wo, 8]
    return taps * valid.to(x.dtype)


def gate_probabilities(weights, training):
    """Logits [..., 16] -> gate mixture: softmax when training, one-hot(arg-max) otherwise."""
    if training:
        return F.softmax(weights, dim=-1)
    return F.one_hot(weights.argmax(-1), num_classes=16).to(weights.dtype)


def conv_stage(x, w_prob, sel, stride=1, padding=1, kernel=3):
    """First gate level only: [N, Ci, H, W] -> [N, C, Ho, Wo, 4]; ``w_prob`` is [C, 4, 16]."""
    taps = gather_taps(x, sel, stride, padding, kernel)
    c = sel.shape[0]
    return bin_op_s(taps[..., 0::2], taps[..., 1::2], w_prob.view(1, c, 1, 1, 4, 16))


def tree_stage(x, w_prob):
    """One pairwise reduction level: [N, C, H, W, 2X] -> [N, C, H, W, X]; ``w_prob`` [C, X, 16]
    (src/convlogic/treelogic_layer.py:110-127)."""
    c, xo = w_prob.shape[0], w_prob.shape[1]
    return bin_op_s(x[..., 0::2], x[..., 1::2], w_prob.view(1, c, 1, 1, xo, 16))


def pool_first_max(z):
    """2x2/stride-2 max pool of [N, C, Ho, Wo]; returns (y, idx) with idx int32 [N, C, I]."""
    n, c, ho, wo = z.shape
    hp, wp = ho // 2, wo // 2
    zz = z[:, :, : 2 * hp, : 2 * wp].reshape(n, c, hp, 2, wp, 2).permute(0, 1, 2, 4, 3, 5)
    cand = zz.reshape(n, c, hp, wp, 4)  # scan order (dy, dx) = (0,0),(0,1),(1,0),(1,1)
    # torch.max along a dim reports the first maximal element, i.e. strict '>' scanning.
    y, k = cand.max(dim=-1)
    py = torch.arange(hp).view(1, 1, hp, 1)
    px = torch.arange(wp).view(1, 1, 1, wp)
    idx = (2 * py + k // 2) * wo + (2 * px + k % 2)
    return y, idx.reshape(n, c, hp * wp).to(torch.int32)


def pool_at(z, idx):
    """The pooled output taken at GIVEN flat positions ``idx`` [N, C, I] (``in_y * W_out + in_x``) instead of at
    the maximum: the gradient then flows through exactly those positions, which is what the reference's backward
    kernels do with the ``indices`` tensor they are handed (full_convlogic_kernel.cu:365-461)."""
    n, c, ho, wo = z.shape
    y = z.reshape(n, c, ho * wo).gather(2, idx.to(torch.int64))
    return y.reshape(n, c, ho // 2, wo // 2)


def full_convlogic(x, w_prob, sel, stride=1, padding=1, kernel=3, forced_idx=None):
    """Fused block: returns (y [N,C,Ho/2,Wo/2], x2 [N,C,Ho,Wo,4], x3 [N,C,Ho,Wo,2], idx).
    With ``forced_idx`` the pool keeps those positions (see ``pool_at``) and returns them as idx."""
    ho, wo = out_size(x.shape[2], x.shape[3], stride, padding, kernel)
    if ho <= 0 or wo <= 0 or ho % 2 or wo % 2:
        raise ValueError(f"conv output {ho}x{wo} must be positive and even for the 2x2 pool")
    x2 = conv_stage(x, w_prob[:, 0:4], sel, stride, padding, kernel)
    x3 = tree_stage(x2, w_prob[:, 4:6])
    z = tree_stage(x3, w_prob[:, 6:7])[..., 0]
    if forced_idx is not None:
        return pool_at(z, forced_idx), x2, x3, forced_idx
    y, idx = pool_first_max(z)
    return y, x2, x3, idx
