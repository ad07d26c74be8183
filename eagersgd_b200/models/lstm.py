"""Sequence classifier: stacked LSTM over per-frame feature vectors, linear head on the last state.

The reference's video model feeds per-frame ResNet-50 features (2048-d) to a 2-layer LSTM and a
fully connected layer (deep500 samples/ucf101_resnetlstm.py:18-59: hidden 256, dropout 0.5,
batch-first input, variable-length clips left-padded by the loader).  Hidden size and depth are
parameters; the benchmark configuration uses hidden 2048, 101 classes, batch 16.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import functional as ops
from ..ops.lstm import lstm_layer


class LSTMClassifier(nn.Module):
    def __init__(self, input_dim: int = 2048, hidden: int = 2048, layers: int = 2, num_classes: int = 101,
                 dropout: float = 0.0):
        super().__init__()
        self.hidden, self.layers, self.dropout = hidden, layers, dropout
        self.w_ih = nn.ParameterList()
        self.w_hh = nn.ParameterList()
        self.bias = nn.ParameterList()
        k = 1.0 / math.sqrt(hidden)
        for l in range(layers):
            inp = input_dim if l == 0 else hidden
            self.w_ih.append(nn.Parameter(torch.empty(4 * hidden, inp).uniform_(-k, k)))
            self.w_hh.append(nn.Parameter(torch.empty(4 * hidden, hidden).uniform_(-k, k)))
            self.bias.append(nn.Parameter(torch.zeros(4 * hidden)))
        self.fc = nn.Linear(hidden, num_classes)

    def compute_dtype_(self, dtype):
        """Low-precision weights for the projections; biases stay fp32."""
        for p in list(self.w_ih) + list(self.w_hh):
            p.data = p.data.to(dtype)
        self.fc.to(dtype)
        return self

    def hidden_states(self, x):
        """x: [B, T, input_dim] (batch first, left-padded) -> the top layer's hidden states [T, B, hidden]."""
        h = x.transpose(0, 1).contiguous()                 # [T, B, I]
        for l in range(self.layers):
            h = lstm_layer(h, self.w_ih[l], self.w_hh[l], self.bias[l])
            if self.dropout > 0 and self.training and l < self.layers - 1:
                h = torch.nn.functional.dropout(h, self.dropout)
        return h

    def forward(self, x):
        """x: [B, T, input_dim] -> logits [B, classes] from the last hidden state."""
        return ops.linear(self.hidden_states(x)[-1], self.fc.weight, self.fc.bias)
