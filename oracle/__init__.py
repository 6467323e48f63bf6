"""CPU oracle for the logic-gate hot path.  TEST INFRASTRUCTURE ONLY.

This package restates, on the CPU (PyTorch CPU tensors and numpy, vectorised), the
arithmetic of the reference's ConvLogicLayer / TreeLogicLayer / LogicLayer / GroupSum /
packed-inference path.  It exists so that the CUDA kernels can be checked against an
independent implementation of the same maths.

Only the test-suite, the repository's smoke check and the benchmark's CPU-baseline leg may
import it; the product package (``convlogic_b200``) never does and has no CPU fallback.

Pinning: the restatement is compared, in ``tests/test_oracle_golden.py``, with golden
tensors that were produced by running the reference's own ``implementation="python"``
modules (``tests/golden/make_golden.py`` holds the generating script), and with the
reference tests' known-answer vectors (the 16-operator truth table).
"""

from .logic_ops import COEFS_T, bin_op, bin_op_s, bin_op_bits  # noqa: F401
from .conv_oracle import (  # noqa: F401
    unpack_selection,
    gather_taps,
    conv_stage,
    tree_stage,
    pool_first_max,
    pool_at,
    full_convlogic,
    gate_probabilities,
)
from .flat_oracle import logic_layer, group_sum, inverse_connections  # noqa: F401
from .packed_oracle import (  # noqa: F401
    pack_bits,
    unpack_bits,
    packed_logic,
    packed_group_sum,
    packed_convtree,
    thermometer,
)
