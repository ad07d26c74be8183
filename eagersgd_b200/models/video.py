"""Video classifier: a convolutional network per frame, an LSTM over the frame features, a linear layer per
time step and the mean of its outputs over time.

This is the reference's UCF101 model (deep500 samples/ucf101_resnetlstm.py:18-59): ResNet-50 without its
classification layer gives 2048 features per frame, a 2-layer LSTM with hidden size 256 and dropout 0.5
between the layers runs over the frames (batch first), a fully connected layer maps every hidden state to
the classes and the logits are averaged over time.  Here the frame network is this framework's ResNet
(tcgen05 convolutions, fused batch norm) and the recurrent part its LSTM kernels; frames of all clips of a
batch go through the frame network as one batch.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as ops
from .lstm import LSTMClassifier
from .resnet import imagenet_resnet


class ResNetLSTM(nn.Module):
    def __init__(self, num_classes: int = 101, resnet_size: int = 50, hidden: int = 256, layers: int = 2,
                 dropout: float = 0.5, frame_chunk: int = 64, frame_net: nn.Module = None, feature_dim: int = None):
        super().__init__()
        self.frame_net = frame_net if frame_net is not None else imagenet_resnet(resnet_size, 1, 1000)
        if feature_dim is None:
            feature_dim = self.frame_net.fc.in_features
        self.feature_dim, self.frame_chunk = feature_dim, frame_chunk
        # the LSTM stack of the sequence classifier, with a head applied at every time step instead of the last
        self.rnn = LSTMClassifier(feature_dim, hidden, layers, num_classes, dropout=dropout)

    def compute_dtype_(self, dtype):
        self.rnn.compute_dtype_(dtype)
        return self

    def features(self, frames: torch.Tensor) -> torch.Tensor:
        """[N, 3, H, W] -> [N, feature_dim]: the frame network up to its pooled features."""
        net = self.frame_net
        if hasattr(net, "features"):
            return net.features(frames)
        feats = []
        hook = net.fc.register_forward_pre_hook(lambda m, inp: feats.append(inp[0]))
        try:
            net(frames)
        finally:
            hook.remove()
        return feats[0]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: [B, T, 3, H, W] (left-padded clips) -> logits [B, classes], the mean over time of per-step logits."""
        b, t = x.shape[:2]
        flat = x.reshape(b * t, *x.shape[2:])
        if flat.is_cuda:
            flat = flat.contiguous(memory_format=torch.channels_last)
        chunks = [self.features(flat[i:i + self.frame_chunk]) for i in range(0, b * t, self.frame_chunk)]
        f = torch.cat(chunks).reshape(b, t, self.feature_dim)
        h = self.rnn.hidden_states(f)                               # [T, B, hidden]
        logits = ops.linear(h.reshape(t * b, -1), self.rnn.fc.weight, self.rnn.fc.bias).reshape(t, b, -1)
        return logits.float().mean(0)
