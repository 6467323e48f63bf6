"""CPU restatement of the flat LogicLayer and GroupSum.  TEST INFRASTRUCTURE ONLY.

Follows the reference:
  * gather of two input features per neuron and the weighted 16-gate sum:
    src/difflogic/difflogic.py:112-123 (``LogicLayer.forward_python``);
  * GroupSum, float input: ``reshape(..., k, F // k).sum(-1) / tau``: difflogic.py:203-208;
  * the consumer lists (CSR) used by the input-gradient kernel: difflogic.py:71-87.
"""

import numpy as np
import torch

from .logic_ops import bin_op_s


def logic_layer(x, idx_a, idx_b, w_prob):
    """x [B, in] -> [B, out]; ``w_prob`` [out, 16] is the gate mixture of every neuron."""
    a, b = x[..., idx_a.long()], x[..., idx_b.long()]
    return bin_op_s(a, b, w_prob)


def group_sum(x, k, tau=1.0):
    if x.shape[-1] % k:
        raise ValueError((tuple(x.shape), k))
    return x.reshape(*x.shape[:-1], k, x.shape[-1] // k).sum(-1) / tau


def inverse_connections(idx_a, idx_b, in_dim):
    """For every input feature, the neurons that read it, ordered by neuron index with a
    neuron listed twice when both of its inputs are that feature.
    Returns (start [in_dim + 1], consumers [2 * out]) as int64 numpy arrays."""
    a = np.asarray(idx_a, dtype=np.int64)
    b = np.asarray(idx_b, dtype=np.int64)
    out = a.shape[0]
    feat = np.stack([a, b], 1).reshape(-1)  # neuron-major, a before b
    neuron = np.repeat(np.arange(out, dtype=np.int64), 2)
    order = np.argsort(feat, kind="stable")
    counts = np.bincount(feat, minlength=in_dim)
    start = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    return start, neuron[order]
