"""CPU restatement (numpy, integer/bit arithmetic) of the packed inference path.

TEST INFRASTRUCTURE ONLY (see the package docstring).

Follows the reference:
  * bit packing along the batch, sample ``bits * word + i`` in bit ``i`` (LSB first), pad bits
    zero, ``pad_len = (bits - B % bits) % bits``: src/difflogic/cuda/difflogic_kernel.cu:335-413;
  * packed gate evaluation ``y[j] = op_j(x[a_j], x[b_j])`` word by word:
    difflogic_kernel.cu:272-293 with the bitwise gates of src/common/cuda_utils.cuh:162-199;
  * per-class bit counts, int32 ``[B, k]``, pad samples dropped: difflogic_kernel.cu:418-482;
  * thermometer input encoding ``cat([x > t_i])`` with ``t_i = i / (L + 1)``:
    src/convlogic/data.py:46-59.

The reference has no packed ConvLogic block (its ``forward_cuda_eval`` for the conv layer
refers to attributes and a binding that do not exist, convlogic_layer.py:357-372), so
``packed_convtree`` is defined by the eval-mode float block on {0,1} inputs: one-hot gates
give exactly 0.0 / 1.0 and the 2x2 max pool is a bitwise OR.  Tests check that identity.
"""

import numpy as np

from .logic_ops import bin_op_bits

_DTYPES = {8: np.int8, 16: np.int16, 32: np.int32, 64: np.int64}
_UDTYPES = {8: np.uint8, 16: np.uint16, 32: np.uint32, 64: np.uint64}


def pack_bits(t, bit_count=32):
    """bool [F, B] -> (intN [F, ceil(B / bits)], pad_len)."""
    t = np.asarray(t).astype(bool)
    f, b = t.shape
    words = -(-b // bit_count)
    pad_len = (bit_count - b % bit_count) % bit_count
    padded = np.zeros((f, words * bit_count), dtype=bool)
    padded[:, :b] = t
    acc = np.zeros((f, words), dtype=_UDTYPES[bit_count])
    lanes = padded.reshape(f, words, bit_count)
    for i in range(bit_count):
        acc |= lanes[:, :, i].astype(_UDTYPES[bit_count]) << _UDTYPES[bit_count](i)
    return acc.view(_DTYPES[bit_count]), pad_len


def unpack_bits(packed, n_samples):
    """intN [..., words] -> bool [..., n_samples]."""
    packed = np.asarray(packed)
    bits = packed.dtype.itemsize * 8
    u = packed.view(_UDTYPES[bits])
    shifts = np.arange(bits, dtype=_UDTYPES[bits])
    lanes = (u[..., None] >> shifts) & _UDTYPES[bits](1)
    return lanes.reshape(*packed.shape[:-1], -1)[..., :n_samples].astype(bool)


def packed_logic(x, idx_a, idx_b, ops):
    """x intN [in, words]; ops uint8 [out] gate ids -> intN [out, words]."""
    x = np.asarray(x)
    a = x[np.asarray(idx_a, dtype=np.int64)]
    b = x[np.asarray(idx_b, dtype=np.int64)]
    ops = np.asarray(ops)
    y = np.zeros_like(a)
    for i in range(16):
        m = ops == i
        if m.any():
            y[m] = bin_op_bits(a[m], b[m], i)
    return y


def packed_group_sum(x, pad_len, k):
    """x intN [F, words] -> int32 [B, k] with B = words * bits - pad_len."""
    x = np.asarray(x)
    f, words = x.shape
    if f % k:
        raise ValueError(f"in_dim ({f}) has to be divisible by k ({k}) but it is not")
    bits = x.dtype.itemsize * 8
    b = words * bits - pad_len
    lanes = unpack_bits(x, b)  # [F, B]
    return lanes.reshape(k, f // k, b).sum(1).T.astype(np.int32)


def packed_convtree(x, ops, sel, stride=1, padding=1, kernel=3):
    """Packed ConvLogic block.  x intN [Ci, H, W, words]; ops uint8 [C, 7]; sel int32 [C, 8]
    -> intN [C, Ho/2, Wo/2, words]."""
    x = np.asarray(x)
    sel = np.asarray(sel).astype(np.int64)
    pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)  # noqa: E731
    (sh, sw), (ph, pw), (kh, kw) = pair(stride), pair(padding), pair(kernel)
    ci, h, w, words = x.shape
    ho, wo = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    c = sel.shape[0]
    ch, r, s = (sel >> 16) & 0xFFFF, (sel >> 8) & 0xFF, sel & 0xFF
    out = np.zeros((c, ho // 2, wo // 2, words), dtype=x.dtype)
    oy = np.arange(ho)[:, None]
    ox = np.arange(wo)[None, :]
    for co in range(c):
        taps = []
        for t in range(8):
            iy = oy * sh + r[co, t] - ph
            ix = ox * sw + s[co, t] - pw
            valid = (iy >= 0) & (iy < h) & (ix >= 0) & (ix < w)
            v = x[ch[co, t], np.clip(iy, 0, h - 1), np.clip(ix, 0, w - 1)]  # [Ho, Wo, words]
            taps.append(np.where(valid[..., None], v, np.zeros_like(v)))
        g = [bin_op_bits(taps[2 * p], taps[2 * p + 1], ops[co, p]) for p in range(4)]
        t0 = bin_op_bits(g[0], g[1], ops[co, 4])
        t1 = bin_op_bits(g[2], g[3], ops[co, 5])
        z = bin_op_bits(t0, t1, ops[co, 6])
        z = z[: 2 * (ho // 2), : 2 * (wo // 2)]
        out[co] = z[0::2, 0::2] | z[0::2, 1::2] | z[1::2, 0::2] | z[1::2, 1::2]
    return out


def thermometer(pixels, levels):
    """float [N, Cp, H, W] in [0, 1) -> bool [N, levels * Cp, H, W], threshold-major:
    channel ``(i - 1) * Cp + c`` holds ``pixels[:, c] > i / (levels + 1)``."""
    pixels = np.asarray(pixels, dtype=np.float32)
    th = np.arange(1, levels + 1, dtype=np.float32) / np.float32(levels + 1)
    return np.concatenate([pixels > t for t in th], axis=1)
