"""Plain PyTorch ResNet (torch.nn modules only) for the synchronous data-parallel baseline arm.

Nothing of this framework is on its path: ``nn.Conv2d`` / ``nn.BatchNorm2d`` / ``nn.Linear`` in
channels_last under bf16 autocast, i.e. cuDNN and cuBLAS, wrapped by ``DistributedDataParallel`` over NCCL.
It is what a PyTorch user would write for the model the reference trains (bottleneck ResNet v1.5:
official/resnet/resnet_model.py:51-554 with the stride on the 3x3 convolution; zero-initialised last
batch-norm gamma of every block), and the role Horovod + TensorFlow play in the reference's comparison
(official/resnet/resnet_run_loop_hvd_imagenet_300.py:374-377).
"""
from __future__ import annotations

import torch
import torch.nn as nn


class Bottleneck(nn.Module):
    def __init__(self, cin: int, width: int, stride: int):
        super().__init__()
        cout = width * 4
        self.conv1 = nn.Conv2d(cin, width, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = nn.Conv2d(width, width, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = nn.Conv2d(width, cout, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(cout)
        nn.init.zeros_(self.bn3.weight)
        self.relu = nn.ReLU(inplace=True)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride=stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        idt = x if self.down is None else self.down(x)
        y = self.relu(self.bn1(self.conv1(x)))
        y = self.relu(self.bn2(self.conv2(y)))
        y = self.bn3(self.conv3(y))
        return self.relu(y + idt)


class BasicBlock(nn.Module):
    def __init__(self, cin: int, cout: int, stride: int):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, cout, 3, stride=stride, padding=1, bias=False)
        self.bn1 = nn.BatchNorm2d(cout)
        self.conv2 = nn.Conv2d(cout, cout, 3, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(cout)
        nn.init.zeros_(self.bn2.weight)
        self.relu = nn.ReLU(inplace=True)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride=stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        idt = x if self.down is None else self.down(x)
        y = self.relu(self.bn1(self.conv1(x)))
        y = self.bn2(self.conv2(y))
        return self.relu(y + idt)


class TorchResNet50(nn.Module):
    def __init__(self, classes: int = 1000):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, 64, 7, stride=2, padding=3, bias=False), nn.BatchNorm2d(64),
                                  nn.ReLU(inplace=True), nn.MaxPool2d(3, stride=2, padding=1))
        layers, cin = [], 64
        for width, blocks, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
            for b in range(blocks):
                layers.append(Bottleneck(cin, width, stride if b == 0 else 1))
                cin = width * 4
        self.layers = nn.Sequential(*layers)
        self.pool = nn.AdaptiveAvgPool2d(1)
        self.fc = nn.Linear(cin, classes)

    def forward(self, x):
        return self.fc(torch.flatten(self.pool(self.layers(self.stem(x))), 1))


class TorchResNetCifar(nn.Module):
    """6n+2 layers, 16/32/64 channels (official/resnet/cifar10_main.py:179-219)."""

    def __init__(self, depth: int = 32, classes: int = 10):
        super().__init__()
        n = (depth - 2) // 6
        self.stem = nn.Sequential(nn.Conv2d(3, 16, 3, padding=1, bias=False), nn.BatchNorm2d(16), nn.ReLU(inplace=True))
        layers, cin = [], 16
        for cout, stride in ((16, 1), (32, 2), (64, 2)):
            for b in range(n):
                layers.append(BasicBlock(cin, cout, stride if b == 0 else 1))
                cin = cout
        self.layers = nn.Sequential(*layers)
        self.pool = nn.AdaptiveAvgPool2d(1)
        self.fc = nn.Linear(cin, classes)

    def forward(self, x):
        return self.fc(torch.flatten(self.pool(self.layers(self.stem(x))), 1))


class TorchLSTMClassifier(nn.Module):
    """Frame features -> 2-layer cuDNN LSTM -> linear on the last hidden state."""

    def __init__(self, features: int = 2048, hidden: int = 2048, layers: int = 2, classes: int = 101):
        super().__init__()
        self.lstm = nn.LSTM(features, hidden, layers, batch_first=True)
        self.fc = nn.Linear(hidden, classes)

    def forward(self, x):
        y, _ = self.lstm(x)
        return self.fc(y[:, -1])
