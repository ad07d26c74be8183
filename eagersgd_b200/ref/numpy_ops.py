"""NumPy restatements of every operator, used as oracles (NCHW, float64 internally).

Same set as the reference's python operators (deep500/frameworks/reference/custom_operators/python/
*.py: add, sum, relu, reshape, squeeze, unsqueeze, matmul, gemm, conv, batch-norm inference /
training, max / average / global-average pool, softmax, cross-entropy, softmax cross-entropy, mean
squared error), each with its gradient where the training path needs one.
"""
from __future__ import annotations

import numpy as np


def add(a, b): return a + b
def sum_(*xs): return np.sum(np.stack(xs), axis=0)
def relu(x): return np.maximum(x, 0)
def relu_grad(x, dy): return dy * (x > 0)
def reshape(x, shape): return np.reshape(x, shape)
def squeeze(x, axes): return np.squeeze(x, axis=tuple(axes))
def unsqueeze(x, axes):
    for a in sorted(axes):
        x = np.expand_dims(x, a)
    return x
def matmul(a, b): return a @ b


def gemm(a, b, c=None, alpha=1.0, beta=1.0, trans_a=False, trans_b=False):
    a = a.T if trans_a else a
    b = b.T if trans_b else b
    y = alpha * (a @ b)
    return y + beta * c if c is not None else y


def _pad(x, p):
    return np.pad(x, ((0, 0), (0, 0), (p, p), (p, p))) if p else x


def conv2d(x, w, stride=1, pad=0):
    """Cross-correlation, x [N,C,H,W], w [K,C,R,S]."""
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    xp = _pad(x.astype(np.float64), pad)
    ho, wo = (h + 2 * pad - r) // stride + 1, (wd + 2 * pad - s) // stride + 1
    y = np.zeros((n, k, ho, wo))
    for i in range(r):
        for j in range(s):
            patch = xp[:, :, i:i + stride * ho:stride, j:j + stride * wo:stride]
            y += np.einsum("nchw,kc->nkhw", patch, w[:, :, i, j].astype(np.float64))
    return y


def conv2d_grad(x, w, dy, stride=1, pad=0):
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    xp = _pad(x.astype(np.float64), pad)
    dxp = np.zeros_like(xp)
    dw = np.zeros(w.shape)
    ho, wo = dy.shape[2], dy.shape[3]
    for i in range(r):
        for j in range(s):
            patch = xp[:, :, i:i + stride * ho:stride, j:j + stride * wo:stride]
            dw[:, :, i, j] = np.einsum("nkhw,nchw->kc", dy, patch)
            dxp[:, :, i:i + stride * ho:stride, j:j + stride * wo:stride] += np.einsum(
                "nkhw,kc->nchw", dy, w[:, :, i, j].astype(np.float64))
    dx = dxp[:, :, pad:pad + h, pad:pad + wd] if pad else dxp
    return dx, dw


def batchnorm_inference(x, gamma, beta, mean, var, eps=1e-5):
    sh = (1, -1, 1, 1)
    return (x - mean.reshape(sh)) / np.sqrt(var.reshape(sh) + eps) * gamma.reshape(sh) + beta.reshape(sh)


def batchnorm_training(x, gamma, beta, running_mean, running_var, momentum=0.1, eps=1e-5):
    """Returns y, new running mean / var (unbiased variance in the running estimate), and the
    saved batch mean / inverse std."""
    ax = (0, 2, 3)
    m = x.shape[0] * x.shape[2] * x.shape[3]
    mean, var = x.mean(ax), x.var(ax)
    invstd = 1.0 / np.sqrt(var + eps)
    sh = (1, -1, 1, 1)
    y = (x - mean.reshape(sh)) * invstd.reshape(sh) * gamma.reshape(sh) + beta.reshape(sh)
    rm = (1 - momentum) * running_mean + momentum * mean
    rv = (1 - momentum) * running_var + momentum * var * m / max(m - 1, 1)
    return y, rm, rv, mean, invstd


def batchnorm_training_grad(x, gamma, mean, invstd, dy):
    ax = (0, 2, 3)
    m = x.shape[0] * x.shape[2] * x.shape[3]
    sh = (1, -1, 1, 1)
    xhat = (x - mean.reshape(sh)) * invstd.reshape(sh)
    dbeta, dgamma = dy.sum(ax), (dy * xhat).sum(ax)
    dx = gamma.reshape(sh) * invstd.reshape(sh) * (dy - dbeta.reshape(sh) / m - xhat * dgamma.reshape(sh) / m)
    return dx, dgamma, dbeta


def _windows(x, k, stride, pad, fill):
    n, c, h, w = x.shape
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)), constant_values=fill)
    ho, wo = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    out = np.empty((n, c, ho, wo, k * k), dtype=x.dtype)
    for i in range(k):
        for j in range(k):
            out[..., i * k + j] = xp[:, :, i:i + stride * ho:stride, j:j + stride * wo:stride]
    return out


def maxpool(x, k=3, stride=2, pad=1): return _windows(x, k, stride, pad, -np.inf).max(-1)
def averagepool(x, k=2, stride=2, pad=0): return _windows(x, k, stride, pad, 0.0).mean(-1)
def globalaveragepool(x): return x.mean((2, 3))


def softmax(x, axis=-1):
    e = np.exp(x - x.max(axis, keepdims=True))
    return e / e.sum(axis, keepdims=True)


def cross_entropy(probs, labels):
    return float(-np.log(probs[np.arange(len(labels)), labels]).mean())


def softmax_cross_entropy(logits, labels):
    """Mean loss and its gradient w.r.t. the logits."""
    p = softmax(logits.astype(np.float64))
    loss = cross_entropy(p, labels)
    g = p.copy()
    g[np.arange(len(labels)), labels] -= 1
    return loss, g / len(labels)


def mean_squared_error(pred, target):
    d = pred - target
    return float((d * d).mean()), 2 * d / d.size


def momentum_sgd(w, g, acc, lr, momentum=0.9, weight_decay=0.0):
    """acc = m*acc + g + wd*w ; w -= lr*acc (deep500/frameworks/reference/optimizers.py:39-46)."""
    acc = momentum * acc + g + weight_decay * w
    return w - lr * acc, acc


def lstm_cell(x_proj, h_proj, bias, c_prev):
    pre = x_proj + h_proj + bias
    i, f, g, o = np.split(pre, 4, axis=-1)
    sig = lambda v: 1 / (1 + np.exp(-v))
    c = sig(f) * c_prev + sig(i) * np.tanh(g)
    return sig(o) * np.tanh(c), c
