"""The 16 two-input gates: real-valued relaxations and their bitwise twins.

TEST INFRASTRUCTURE ONLY (see the package docstring).

Follows the reference:
  * real-valued forms and the 0..15 accumulation order of the weighted sum:
    src/difflogic/functional.py:27-71 (``bin_op``, ``bin_op_s``);
  * truth table: src/common/cuda_utils.cuh:143-160;
  * bitwise forms: src/common/cuda_utils.cuh:162-199 (``bin_op_eval``);
  * the 4-term basis {ab, a, b, 1} every gate decomposes into:
    src/convlogic/cuda/full_convlogic_kernel.cu:692-696 and
    src/difflogic/cuda/difflogic_kernel.cu:164-168 (``coefs_T``).
"""

import numpy as np
import torch

# op id -> outputs for (a, b) = (0,0), (0,1), (1,0), (1,1); id bit 3 is f(0,0), bit 0 is f(1,1).
TRUTH = [[(i >> 3) & 1, (i >> 2) & 1, (i >> 1) & 1, i & 1] for i in range(16)]

# Real-valued relaxation of each gate, in the algebraic form the reference evaluates
# (probabilistic t-norm: AND = ab, OR = a + b - ab, XOR = a + b - 2ab, NOT = 1 - .).
_REAL = [
    lambda a, b: torch.zeros_like(a),
    lambda a, b: a * b,
    lambda a, b: a - a * b,
    lambda a, b: a,
    lambda a, b: b - a * b,
    lambda a, b: b,
    lambda a, b: a + b - 2 * a * b,
    lambda a, b: a + b - a * b,
    lambda a, b: 1 - (a + b - a * b),
    lambda a, b: 1 - (a + b - 2 * a * b),
    lambda a, b: 1 - b,
    lambda a, b: 1 - b + a * b,
    lambda a, b: 1 - a,
    lambda a, b: 1 - a + a * b,
    lambda a, b: 1 - a * b,
    lambda a, b: torch.ones_like(a),
]


def bin_op(a, b, i):
    """Relaxed gate ``i`` applied element-wise (functional.py:27-62)."""
    return _REAL[int(i)](a, b)


def bin_op_s(a, b, w):
    """Sum over the 16 gates of ``w[..., i] * op_i(a, b)``, accumulated i = 0..15 from zero
    (functional.py:66-71)."""
    acc = torch.zeros_like(a)
    for i in range(16):
        acc = acc + w[..., i] * _REAL[i](a, b)
    return acc


def _coefs():
    # op_i(a, b) = k_ab * ab + k_a * a + k_b * b + k_1 ; derive the integer coefficients
    # from the truth table (multilinear interpolation), rows ordered (ab, a, b, 1).
    c = np.zeros((4, 16), dtype=np.int64)
    for i, (f00, f01, f10, f11) in enumerate(TRUTH):
        c[3, i] = f00
        c[1, i] = f10 - f00
        c[2, i] = f01 - f00
        c[0, i] = f11 - f10 - f01 + f00
    return c


COEFS_T = _coefs()  # [4, 16], equals the reference's ``coefs_T`` table


def bin_op_bits(a, b, i):
    """Bitwise gate ``i`` on integer numpy arrays (every bit lane is one sample)."""
    i = int(i)
    f00, f01, f10, f11 = TRUTH[i]
    ones = ~np.zeros_like(a)
    out = np.zeros_like(a)
    if f11:
        out |= a & b
    if f10:
        out |= a & ~b
    if f01:
        out |= ~a & b
    if f00:
        out |= ~a & ~b
    return out & ones
