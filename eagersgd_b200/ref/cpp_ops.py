"""ctypes front end of the C++ oracle library (``ref/cpp/ops.cpp``, ``ops_more.cpp``), built on first use."""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess
import tempfile

import numpy as np

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpp")
_SRCS = [os.path.join(_DIR, "ops.cpp"), os.path.join(_DIR, "ops_more.cpp")]
_lib = None


def lib():
    global _lib
    if _lib is None:
        h = hashlib.sha256(b"".join(open(f, "rb").read() for f in _SRCS)).hexdigest()[:12]
        d = os.path.join(tempfile.gettempdir(), "eagersgd_ops")
        os.makedirs(d, exist_ok=True)
        so = os.path.join(d, "libref_ops_%s.so" % h)
        if not os.path.exists(so):
            subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fopenmp"] + _SRCS + ["-o", so + ".tmp"], check=True)
            os.replace(so + ".tmp", so)
        _lib = C.CDLL(so)
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def conv2d(x, w, stride=1, pad=0):
    x, w = _f(x), _f(w)
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    y = np.empty((n, k, (h + 2 * pad - r) // stride + 1, (wd + 2 * pad - s) // stride + 1), dtype=np.float32)
    lib().ref_conv2d_fwd(_p(x), _p(w), _p(y), n, c, h, wd, k, r, s, stride, pad)
    return y


def conv2d_grads(x, w, dy, stride=1, pad=0):
    x, w, dy = _f(x), _f(w), _f(dy)
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    dx, dw = np.empty_like(x), np.empty_like(w)
    lib().ref_conv2d_dgrad(_p(dy), _p(w), _p(dx), n, c, h, wd, k, r, s, stride, pad)
    lib().ref_conv2d_wgrad(_p(x), _p(dy), _p(dw), n, c, h, wd, k, r, s, stride, pad)
    return dx, dw


def batchnorm_training(x, gamma, beta, rm, rv, momentum=0.1, eps=1e-5):
    x, gamma, beta = _f(x), _f(gamma), _f(beta)
    rm, rv = _f(rm).copy(), _f(rv).copy()
    n, c, h, w = x.shape
    y, mean, invstd = np.empty_like(x), np.empty(c, np.float32), np.empty(c, np.float32)
    lib().ref_batchnorm_train_fwd(_p(x), _p(gamma), _p(beta), _p(y), _p(rm), _p(rv), _p(mean), _p(invstd), n, c, h * w,
                                  C.c_float(momentum), C.c_float(eps))
    return y, rm, rv, mean, invstd


def batchnorm_training_grad(x, gamma, mean, invstd, dy):
    x, gamma, mean, invstd, dy = map(_f, (x, gamma, mean, invstd, dy))
    n, c, h, w = x.shape
    dx, dg, db = np.empty_like(x), np.empty(c, np.float32), np.empty(c, np.float32)
    lib().ref_batchnorm_train_bwd(_p(x), _p(gamma), _p(mean), _p(invstd), _p(dy), _p(dx), _p(dg), _p(db), n, c, h * w)
    return dx, dg, db


def gemm(a, b, c=None, alpha=1.0, beta=0.0, trans_a=False, trans_b=False):
    a, b = _f(a), _f(b)
    m = a.shape[1] if trans_a else a.shape[0]
    k = a.shape[0] if trans_a else a.shape[1]
    n = b.shape[0] if trans_b else b.shape[1]
    out = _f(c).copy() if c is not None else np.zeros((m, n), np.float32)
    lib().ref_gemm(_p(a), _p(b), _p(out), m, n, k, int(trans_a), int(trans_b), C.c_float(alpha), C.c_float(beta))
    return out


def softmax(x):
    x = _f(x)
    y = np.empty_like(x)
    lib().ref_softmax(_p(x), _p(y), x.shape[0], x.shape[1])
    return y


def maxpool(x, k=3, stride=2, pad=1):
    x = _f(x)
    n, c, h, w = x.shape
    y = np.empty((n, c, (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1), np.float32)
    lib().ref_maxpool(_p(x), _p(y), n, c, h, w, k, stride, pad)
    return y


def global_avgpool(x):
    x = _f(x)
    n, c, h, w = x.shape
    y = np.empty((n, c), np.float32)
    lib().ref_global_avgpool(_p(x), _p(y), n, c, h * w)
    return y


def relu(x):
    x = _f(x)
    y = np.empty_like(x)
    lib().ref_relu(_p(x), _p(y), C.c_int64(x.size))
    return y


# ---- operators of ops_more.cpp: forward and backward ---------------------------------------------------------------
def add(a, b):
    a, b = _f(a), _f(b)
    y = np.empty_like(a)
    lib().ref_add_fwd(_p(a), _p(b), _p(y), C.c_int64(a.size))
    return y


def add_grad(dy):
    dy = _f(dy)
    da, db = np.empty_like(dy), np.empty_like(dy)
    lib().ref_add_bwd(_p(dy), _p(da), _p(db), C.c_int64(dy.size))
    return da, db


def sum_n(inputs):
    arrs = [_f(a) for a in inputs]
    y = np.empty_like(arrs[0])
    ptrs = (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])
    lib().ref_sum_fwd(ptrs, len(arrs), _p(y), C.c_int64(y.size))
    return y


def sum_n_grad(dy, num_inputs):
    dy = _f(dy)
    outs = [np.empty_like(dy) for _ in range(num_inputs)]
    ptrs = (C.c_void_p * num_inputs)(*[a.ctypes.data for a in outs])
    lib().ref_sum_bwd(_p(dy), ptrs, num_inputs, C.c_int64(dy.size))
    return outs


def reshape(x, shape):
    x = _f(x)
    y = np.empty(x.size, np.float32)
    lib().ref_reshape_fwd(_p(x), _p(y), C.c_int64(x.size))
    return y.reshape(shape)


def reshape_grad(dy, in_shape):
    dy = _f(dy)
    dx = np.empty(dy.size, np.float32)
    lib().ref_reshape_bwd(_p(dy), _p(dx), C.c_int64(dy.size))
    return dx.reshape(in_shape)


def relu_grad(x, dy):
    x, dy = _f(x), _f(dy)
    dx = np.empty_like(x)
    lib().ref_relu_bwd(_p(x), _p(dy), _p(dx), C.c_int64(x.size))
    return dx


def matmul(a, b):
    a, b = _f(a), _f(b)
    y = np.empty((a.shape[0], b.shape[1]), np.float32)
    lib().ref_matmul_fwd(_p(a), _p(b), _p(y), a.shape[0], b.shape[1], a.shape[1])
    return y


def matmul_grad(a, b, dy):
    a, b, dy = _f(a), _f(b), _f(dy)
    da, db = np.empty_like(a), np.empty_like(b)
    lib().ref_matmul_bwd(_p(a), _p(b), _p(dy), _p(da), _p(db), a.shape[0], b.shape[1], a.shape[1])
    return da, db


def gemm_grad(a, b, dy, alpha=1.0, beta=0.0, trans_a=False, trans_b=False):
    a, b, dy = _f(a), _f(b), _f(dy)
    m, n = dy.shape
    k = a.shape[0] if trans_a else a.shape[1]
    da, db, dc = np.empty_like(a), np.empty_like(b), np.empty_like(dy)
    lib().ref_gemm_bwd(_p(a), _p(b), _p(dy), _p(da), _p(db), _p(dc), m, n, k, int(trans_a), int(trans_b),
                       C.c_float(alpha), C.c_float(beta))
    return da, db, dc


def softmax_grad(y, dy):
    y, dy = _f(y), _f(dy)
    dx = np.empty_like(y)
    lib().ref_softmax_bwd(_p(y), _p(dy), _p(dx), y.shape[0], y.shape[1])
    return dx


def maxpool_grad(x, dy, k=3, stride=2, pad=1):
    x, dy = _f(x), _f(dy)
    n, c, h, w = x.shape
    dx = np.empty_like(x)
    lib().ref_maxpool_bwd(_p(x), _p(dy), _p(dx), n, c, h, w, k, stride, pad)
    return dx


def avgpool(x, k=2, stride=2, pad=0, count_include_pad=False):
    x = _f(x)
    n, c, h, w = x.shape
    y = np.empty((n, c, (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1), np.float32)
    lib().ref_avgpool_fwd(_p(x), _p(y), n, c, h, w, k, stride, pad, int(count_include_pad))
    return y


def avgpool_grad(dy, in_shape, k=2, stride=2, pad=0, count_include_pad=False):
    dy = _f(dy)
    n, c, h, w = in_shape
    dx = np.empty(in_shape, np.float32)
    lib().ref_avgpool_bwd(_p(dy), _p(dx), n, c, h, w, k, stride, pad, int(count_include_pad))
    return dx


def global_avgpool_grad(dy, in_shape):
    dy = _f(dy)
    n, c, h, w = in_shape
    dx = np.empty(in_shape, np.float32)
    lib().ref_global_avgpool_bwd(_p(dy), _p(dx), n, c, h * w)
    return dx


def batchnorm_inference(x, gamma, beta, mean, var, eps=1e-5):
    x = _f(x)
    n, c, h, w = x.shape
    y = np.empty_like(x)
    lib().ref_batchnorm_infer_fwd(_p(x), _p(_f(gamma)), _p(_f(beta)), _p(_f(mean)), _p(_f(var)), _p(y), n, c, h * w,
                                  C.c_float(eps))
    return y


def batchnorm_inference_grad(x, gamma, mean, var, dy, eps=1e-5):
    x, dy = _f(x), _f(dy)
    n, c, h, w = x.shape
    dx, dg, db = np.empty_like(x), np.empty(c, np.float32), np.empty(c, np.float32)
    lib().ref_batchnorm_infer_bwd(_p(x), _p(_f(gamma)), _p(_f(mean)), _p(_f(var)), _p(dy), _p(dx), _p(dg), _p(db), n, c,
                                  h * w, C.c_float(eps))
    return dx, dg, db
