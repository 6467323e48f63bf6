"""convlogic_b200: the ConvLogic / difflogic layer API on hand-written sm_100a CUDA kernels.

Public names mirror the reference packages ``convlogic`` and ``difflogic``
(src/convlogic/__init__.py:1-4, src/difflogic/__init__.py:1-3).
"""

from .convlogic_layer import ConvLogicLayer, PoolLogicLayer  # noqa: F401
from .treelogic_layer import TreeLogicLayer  # noqa: F401
from .difflogic import (  # noqa: F401
    FusedLogicLayers,
    GroupSum,
    GroupSumCrossEntropy,
    LogicLayer,
    fuse_logic_layers,
    get_unique_connections,
)
from .dp import FlatAdam, GradBucket  # noqa: F401
from .packbitstensor import PackBitsTensor  # noqa: F401
from .functional import (  # noqa: F401
    ConvLogicFunction,
    FullConvLogicFunction,
    GradFactor,
    LogicLayerCudaFunction,
    TreeLogicFunction,
)
from .model import ConvLogicCifarModel, ConvLogicMnistModel  # noqa: F401
from .compiled_model import CompiledLogicNet  # noqa: F401
from ._lib import LIB_PATH, W_ARGMAX, W_PROB, W_SOFTMAX  # noqa: F401

__all__ = [
    "ConvLogicLayer", "PoolLogicLayer", "TreeLogicLayer", "LogicLayer", "GroupSum", "PackBitsTensor",
    "ConvLogicFunction", "FullConvLogicFunction", "TreeLogicFunction", "LogicLayerCudaFunction", "GradFactor",
    "ConvLogicCifarModel", "ConvLogicMnistModel", "get_unique_connections", "CompiledLogicNet", "FusedLogicLayers", "fuse_logic_layers",
    "GroupSumCrossEntropy", "FlatAdam", "GradBucket",
]
