"""ResNet v1 / v1.5 / v2 for CIFAR (6n+2) and ImageNet (18 … 200).

Architecture, initialisation and *variable creation order* follow the reference
model so that checkpoints can be exported in its layout
(test-models/.../official/resnet/resnet_model.py:51-554, cifar10_main.py:179-219,
imagenet_main_eagersgd.py:290-330; PyTorch variants in
deep500/networks/pytorch_resnet.py): fixed padding for strided convolutions,
batch-norm momentum 0.997 / eps 1e-5, zero-initialised gamma on the last
batch-norm of every residual block, projection shortcuts created before the
main path, the stride on the 3x3 convolution of a bottleneck ("v1.5").
Activations are NHWC (channels_last) bf16 on GPUs.
"""
from __future__ import annotations

from typing import List, Tuple

import torch.nn as nn

from ..ops import functional as ops

BN_MOMENTUM_TF = 0.997  # tf decay; torch momentum = 1 - decay
BN_EPS = 1e-5

IMAGENET_BLOCKS = {
    18: ("building", [2, 2, 2, 2]), 34: ("building", [3, 4, 6, 3]), 50: ("bottleneck", [3, 4, 6, 3]),
    101: ("bottleneck", [3, 4, 23, 3]), 152: ("bottleneck", [3, 8, 36, 3]), 200: ("bottleneck", [3, 24, 36, 3]),
}


class BatchNormAct(nn.BatchNorm2d):
    """Batch norm fused with an optional residual add and ReLU (one kernel pass each way)."""

    # Ghost batch norm: statistics over consecutive groups of this many samples instead of the whole batch
    # (the reference's --virtual_batch_size, official/resnet/resnet_model.py:45-60); None: the whole batch.
    virtual_batch_size = None

    def forward(self, y, relu: bool = True, residual=None, stats=None):  # noqa: D102
        v = self.virtual_batch_size
        if v and self.training and y.shape[0] > v:
            import torch
            outs = [ops.bn_act(y[i:i + v], self.weight, self.bias, self.running_mean, self.running_var, self.momentum,
                               relu, None if residual is None else residual[i:i + v], None, True)
                    for i in range(0, y.shape[0], v)]
            return torch.cat(outs)
        return ops.bn_act(y, self.weight, self.bias, self.running_mean, self.running_var, self.momentum, relu,
                          residual, stats, self.training)


def _bn(ch: int, zero_gamma: bool = False) -> BatchNormAct:
    bn = BatchNormAct(ch, eps=BN_EPS, momentum=1.0 - BN_MOMENTUM_TF)
    if zero_gamma:
        nn.init.zeros_(bn.weight)
    return bn


class _Conv(nn.Conv2d):
    """conv2d_fixed_padding: explicit symmetric padding when strided (resnet_model.py:63-101).

    ``forward`` returns ``(y, stats)`` where ``stats`` holds the per-channel sum and sum of
    squares of ``y`` when the kernel produced them in its epilogue (else ``None``).
    """

    def __init__(self, cin, cout, k, stride):
        super().__init__(cin, cout, k, stride=stride, padding=(k - 1) // 2, bias=False)
        # variance_scaling_initializer() of the reference: fan-in scaling
        nn.init.kaiming_normal_(self.weight, mode="fan_in", nonlinearity="linear")

    def forward(self, x, tap_input: bool = False):  # noqa: D102
        return ops.conv2d(x, self.weight, self.stride[0], self.padding[0], want_stats=self.training,
                          tap_input=tap_input)


class _Block(nn.Module):
    def __init__(self, cin, filters, stride, kind, version, project, registry):
        super().__init__()
        self.kind, self.version = kind, version
        cout = filters * 4 if kind == "bottleneck" else filters
        self.proj = self.proj_bn = None
        if version == 2:
            self.pre_bn = _bn(cin)
            registry.append(("bn", self.pre_bn))
        if project:
            self.proj = _Conv(cin, cout, 1, stride)
            registry.append(("conv", self.proj))
            if version == 1:
                self.proj_bn = _bn(cout)
                registry.append(("bn", self.proj_bn))
        convs, bns = [], []
        if kind == "bottleneck":
            spec = [(cin, filters, 1, 1), (filters, filters, 3, stride), (filters, cout, 1, 1)]
        else:
            spec = [(cin, filters, 3, stride), (filters, filters, 3, 1)]
        for idx, (ci, co, k, s) in enumerate(spec):
            conv = _Conv(ci, co, k, s)
            convs.append(conv)
            registry.append(("conv", conv))
            last = idx == len(spec) - 1
            if version == 1 or not last:
                bn = _bn(co, zero_gamma=(last and version == 1))
                bns.append(bn)
                registry.append(("bn", bn))
        self.convs = nn.ModuleList(convs)
        self.bns = nn.ModuleList(bns)
        self.cout = cout

    def forward(self, x):
        n = len(self.convs)
        if self.version == 1:
            # The shortcut branches off the first convolution's tapped input: both gradients of x then meet
            # inside that convolution's data-gradient kernel instead of in a separate addition.
            yc, st, shortcut = self.convs[0](x, tap_input=True)
            if self.proj is not None:
                ys, sts = self.proj(shortcut)
                shortcut = self.proj_bn(ys, relu=False, stats=sts)
            y = x
            for i in range(n):
                if i > 0:
                    yc, st = self.convs[i](y)
                # the last batch norm also adds the shortcut and applies the block's final ReLU
                y = self.bns[i](yc, relu=True, residual=shortcut if i == n - 1 else None, stats=st)
            return y
        pre = self.pre_bn(x, relu=True)
        shortcut = self.proj(pre)[0] if self.proj is not None else x
        y = pre
        for i in range(n):
            yc, st = self.convs[i](y)
            y = self.bns[i](yc, relu=True, stats=st) if i < n - 1 else yc
        return y + shortcut


class ResNet(nn.Module):
    def __init__(self, kind: str, blocks: List[int], num_classes: int, num_filters: int, first_kernel: int,
                 first_stride: int, first_pool: bool, block_strides: List[int], version: int = 1):
        super().__init__()
        assert version in (1, 2)
        self.version = version
        self.registry: List[Tuple[str, nn.Module]] = []  # creation order, for the tf-models variable names
        self.stem = _Conv(3, num_filters, first_kernel, first_stride)
        self.registry.append(("conv", self.stem))
        self.stem_bn = None
        if version == 1:
            self.stem_bn = _bn(num_filters)
            self.registry.append(("bn", self.stem_bn))
        self.first_pool = first_pool
        layers = []
        cin = num_filters
        for i, nb in enumerate(blocks):
            filters = num_filters * (2 ** i)
            for j in range(nb):
                blk = _Block(cin, filters, block_strides[i] if j == 0 else 1, kind, version, j == 0, self.registry)
                layers.append(blk)
                cin = blk.cout
        self.blocks = nn.ModuleList(layers)
        self.final_bn = None
        if version == 2:
            self.final_bn = _bn(cin)
            self.registry.append(("bn", self.final_bn))
        self.fc = nn.Linear(cin, num_classes)
        self.registry.append(("dense", self.fc))
        self.feature_dim = cin

    def features(self, x):
        x, st = self.stem(x)
        if self.stem_bn is not None:
            x = self.stem_bn(x, relu=True, stats=st)
        if self.first_pool:
            x = ops.max_pool_3x3_s2(x)
        for blk in self.blocks:
            x = blk(x)
        if self.final_bn is not None:
            x = self.final_bn(x, relu=True)
        return ops.global_avg_pool(x)

    def forward(self, x):
        """Logits (fp32 on the native path)."""
        return ops.linear(self.features(x), self.fc.weight, self.fc.bias)


def imagenet_resnet(size: int = 50, version: int = 1, num_classes: int = 1001) -> ResNet:
    """ImagenetModel (imagenet_main_eagersgd.py:290-330).  ``version=1`` is the
    reference's v1 with the stride on the 3x3 convolution, i.e. "ResNet v1.5"."""
    kind, blocks = IMAGENET_BLOCKS[size]
    return ResNet(kind, blocks, num_classes, 64, 7, 2, True, [1, 2, 2, 2], version)


def cifar_resnet(size: int = 32, version: int = 1, num_classes: int = 10) -> ResNet:
    """Cifar10Model: 6n+2 layers, 16/32/64 filters, building blocks (cifar10_main.py:179-219)."""
    if size % 6 != 2:
        raise ValueError("resnet_size must be 6n + 2")
    n = (size - 2) // 6
    return ResNet("building", [n] * 3, num_classes, 16, 3, 1, False, [1, 2, 2], version)


def count_parameters(model: nn.Module) -> Tuple[int, int]:
    ps = [p for p in model.parameters() if p.requires_grad]
    return len(ps), sum(p.numel() for p in ps)
