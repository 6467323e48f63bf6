"""The reference's two layer stacks (src/convlogic/model.py:11-109), as plain nn.Modules.

Only the shapes are the reference's: four (CIFAR) or three (MNIST) fused ConvLogic blocks,
Flatten, three LogicLayers, GroupSum.  The Lightning training module around them is out of scope.
"""

import torch.nn as nn

from .convlogic_layer import ConvLogicLayer
from .difflogic import GroupSum, LogicLayer


class ConvLogicCifarModel(nn.Module):
    def __init__(self, k_param=32, input_channels=3, input_size=32, tau=20, implementation="cuda"):
        super().__init__()
        self.input_size, self.k_param = input_size, k_param
        self.extra_layers = 2 if k_param >= 1024 else 1
        channels = [input_channels, k_param, 4 * k_param, 16 * k_param, 32 * k_param]
        layers = [ConvLogicLayer(i, o, padding=1, groups=1, residual_init=True, complete=True,
                                 implementation=implementation) for i, o in zip(channels[:-1], channels[1:])]
        side = input_size // 2 ** (len(channels) - 1)
        flat = channels[-1] * side * side
        e = self.extra_layers
        dims = [flat, e * flat * 10, e * flat * 5, e * (flat * 10) // 4]
        layers.append(nn.Flatten())
        layers += [LogicLayer(i, o, grad_factor=1, residual_init=True, implementation=implementation)
                   for i, o in zip(dims[:-1], dims[1:])]
        layers.append(GroupSum(k=10, tau=tau))
        self.network = nn.Sequential(*layers)

    def forward(self, x):
        return self.network(x)


class ConvLogicMnistModel(nn.Module):
    def __init__(self, input_channels=1, input_size=28, k_param=32, tau=6.5, implementation="cuda"):
        super().__init__()
        k = k_param
        conv = dict(residual_init=True, complete=True, implementation=implementation)
        fc = dict(residual_init=True, implementation=implementation)
        self.network = nn.Sequential(
            ConvLogicLayer(input_channels, k, kernel=5, padding=0, **conv),
            ConvLogicLayer(k, 3 * k, kernel=3, padding=1, **conv),
            ConvLogicLayer(3 * k, 9 * k, kernel=3, padding=1, **conv),
            nn.Flatten(),
            LogicLayer(81 * k, 1280 * k, **fc),
            LogicLayer(1280 * k, 640 * k, **fc),
            LogicLayer(640 * k, 320 * k, **fc),
            GroupSum(k=10, tau=tau),
        )

    def forward(self, x):
        return self.network(x)
