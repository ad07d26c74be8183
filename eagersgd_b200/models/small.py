"""Small networks: MNIST LeNet-style nets and CIFAR Wide-ResNet (deep500/networks/pytorch_mnist.py,
pytorch_deep_mnist.py, pytorch_wide_resnet.py)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class MnistNet(nn.Module):
    """Two dense layers on flattened 28x28 digits."""

    def __init__(self, hidden: int = 100, classes: int = 10):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(784, hidden), nn.Linear(hidden, classes)

    def forward(self, x):
        return self.fc2(F.relu(self.fc1(torch.flatten(x, 1))))


class SimpleCNN(nn.Module):
    """conv5(10) - pool - conv5(20) - pool - fc50 - fc for square images of any size and channel count: the
    'simple_cnn' the reference's samples train on MNIST and CIFAR (deep500/networks/pytorch_mnist.py:18-36)."""

    def __init__(self, in_channels: int = 1, size: int = 28, classes: int = 10):
        super().__init__()
        self.conv1, self.conv2 = nn.Conv2d(in_channels, 10, 5), nn.Conv2d(10, 20, 5)
        self.side = (((size - 4) // 2) - 4) // 2                 # what two valid 5x5 convolutions and two poolings leave
        self.fc1, self.fc2 = nn.Linear(self.side * self.side * 20, 50), nn.Linear(50, classes)

    def forward(self, x):
        x = F.relu(F.max_pool2d(self.conv1(x), 2))
        x = F.relu(F.max_pool2d(self.conv2(x), 2))
        return self.fc2(F.relu(self.fc1(torch.flatten(x, 1))))


class DeepMnistNet(nn.Module):
    """conv5-pool-conv5-pool-fc1024-fc10 (the 'deep MNIST' tutorial network)."""

    def __init__(self, classes: int = 10):
        super().__init__()
        self.c1, self.c2 = nn.Conv2d(1, 32, 5, padding=2), nn.Conv2d(32, 64, 5, padding=2)
        self.f1, self.f2 = nn.Linear(7 * 7 * 64, 1024), nn.Linear(1024, classes)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.c1(x)), 2)
        x = F.max_pool2d(F.relu(self.c2(x)), 2)
        return self.f2(F.relu(self.f1(torch.flatten(x, 1))))


class _WideBlock(nn.Module):
    def __init__(self, cin, cout, stride, dropout):
        super().__init__()
        self.bn1, self.c1 = nn.BatchNorm2d(cin), nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.bn2, self.c2 = nn.BatchNorm2d(cout), nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.short = nn.Conv2d(cin, cout, 1, stride, bias=False) if (stride != 1 or cin != cout) else None
        self.dropout = dropout

    def forward(self, x):
        o = F.relu(self.bn1(x))
        y = self.c1(o)
        y = F.dropout(F.relu(self.bn2(y)), self.dropout, self.training) if self.dropout else F.relu(self.bn2(y))
        y = self.c2(y)
        return y + (self.short(o) if self.short is not None else x)


class WideResNet(nn.Module):
    """WRN-depth-widen for CIFAR (depth = 6n + 4)."""

    def __init__(self, depth: int = 16, widen: int = 4, classes: int = 10, dropout: float = 0.0):
        super().__init__()
        n = (depth - 4) // 6
        w = [16, 16 * widen, 32 * widen, 64 * widen]
        self.stem = nn.Conv2d(3, w[0], 3, 1, 1, bias=False)
        blocks, cin = [], w[0]
        for i, stride in enumerate((1, 2, 2)):
            for j in range(n):
                blocks.append(_WideBlock(cin, w[i + 1], stride if j == 0 else 1, dropout))
                cin = w[i + 1]
        self.blocks = nn.Sequential(*blocks)
        self.bn, self.fc = nn.BatchNorm2d(cin), nn.Linear(cin, classes)

    def forward(self, x):
        x = F.relu(self.bn(self.blocks(self.stem(x))))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))
