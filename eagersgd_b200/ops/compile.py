"""Run-time compilation of user operators written in C++ or CUDA, and their use from PyTorch.

``compile_custom_op`` writes / takes a source file, builds a shared library (g++, or nvcc pinned to
sm_100a for ``.cu``), loads it with ctypes and returns a ``CustomCPPOp``; ``custom_op`` turns that
into a differentiable PyTorch function.  Same capability as the reference's operator pipeline
(deep500/lv0/operators/op_compiler.py:57-114 ``compile_custom_cppop[_inline]``, cmake_wrapper.py,
operator_interface.py ``CustomCPPOp``; PyTorch glue deep500/frameworks/pytorch/custom_operators/
pytorch.py:71-113) without CMake and Jinja: one compiler invocation, one C ABI
(``ops/include/eagersgd/op.h``).
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess
import tempfile
from typing import List, Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
INCLUDE_DIR = os.path.join(_HERE, "include")
_TYPE_CODES = {torch.float32: 0, torch.float64: 1, torch.int32: 2, torch.int64: 3, torch.bfloat16: 4, torch.float16: 5}


class TensorDescriptor:
    """Shape and dtype of an operator input or output (deep500/utils/tensor_desc.py)."""

    def __init__(self, dtype: torch.dtype, shape: Sequence[int]):
        self.dtype, self.shape = dtype, tuple(int(s) for s in shape)

    @staticmethod
    def from_tensor(t: torch.Tensor) -> "TensorDescriptor":
        return TensorDescriptor(t.dtype, t.shape)


def desc_from_tensor(t: torch.Tensor) -> TensorDescriptor:
    return TensorDescriptor.from_tensor(t)


class _CTensor(C.Structure):
    _fields_ = [("type", C.c_int32), ("dims", C.c_int32), ("sizes", C.c_int64 * 8)]


def _c_descs(descs: Sequence[TensorDescriptor]):
    arr = (_CTensor * max(len(descs), 1))()
    for i, d in enumerate(descs):
        arr[i].type = _TYPE_CODES[d.dtype]
        arr[i].dims = len(d.shape)
        for j, s in enumerate(d.shape):
            arr[i].sizes[j] = s
    return arr


class CompilableOp:
    """Metadata of an operator to compile: name, source, tensor descriptors, build flags."""

    def __init__(self, name: str, source_files: Sequence[str], input_descs: Sequence[TensorDescriptor],
                 output_descs: Sequence[TensorDescriptor], has_backward: bool = True, additional_flags=(),
                 defines=None):
        self.name, self.files = name, list(source_files)
        self.input_descs, self.output_descs = list(input_descs), list(output_descs)
        self.has_backward = has_backward
        self.flags = list(additional_flags)
        self.defines = dict(defines or {})


def _build(op: CompilableOp, output_dir: Optional[str]) -> str:
    blob = hashlib.sha256()
    for f in op.files:
        blob.update(open(f, "rb").read())
    blob.update(repr((op.flags, sorted(op.defines.items()))).encode())
    out_dir = output_dir or os.path.join(tempfile.gettempdir(), "eagersgd_ops")
    os.makedirs(out_dir, exist_ok=True)
    lib = os.path.join(out_dir, "lib%s_%s.so" % (op.name, blob.hexdigest()[:12]))
    if os.path.exists(lib):
        return lib
    is_cuda = any(f.endswith(".cu") for f in op.files)
    defs = ["-D%s=%s" % kv for kv in op.defines.items()]
    if is_cuda:
        from .._build import CUDA_ARCH_FLAGS, nvcc_path
        cmd = [nvcc_path(), "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-I", INCLUDE_DIR] + \
            CUDA_ARCH_FLAGS + defs + op.flags + op.files + ["-o", lib + ".tmp"]
    else:
        cmd = ["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-fopenmp", "-I", INCLUDE_DIR] + defs + op.flags + \
            op.files + ["-o", lib + ".tmp"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("compiling operator %s failed:\n%s" % (op.name, res.stderr[-4000:]))
    os.replace(lib + ".tmp", lib)
    return lib


class CustomCPPOp:
    """A loaded operator library and one operator instance created from it."""

    def __init__(self, library: str, op: CompilableOp):
        self.lib = C.CDLL(library)
        self.desc = op
        self.lib.create_new_op.restype = C.c_void_p
        self.lib.create_new_op.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        for fn in ("delete_op", "is_cuda_supported"):
            getattr(self.lib, fn).argtypes = [C.c_void_p]
        self.lib.report.restype = C.c_int64
        self.lib.report.argtypes = [C.c_void_p, C.c_void_p]
        self.lib.forward_op.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        self.lib.backward_op.argtypes = [C.c_void_p] * 5
        self.lib.forward_op_cuda.argtypes = [C.c_void_p] * 4
        self.lib.backward_op_cuda.argtypes = [C.c_void_p] * 6
        self.handle = C.c_void_p(self.lib.create_new_op(_c_descs(op.input_descs), len(op.input_descs),
                                                       _c_descs(op.output_descs), len(op.output_descs)))
        self.supports_cuda = bool(self.lib.is_cuda_supported(self.handle))

    def report(self) -> int:
        return int(self.lib.report(self.handle, None))

    @staticmethod
    def _ptrs(tensors: Sequence[torch.Tensor]):
        return (C.c_void_p * max(len(tensors), 1))(*[t.data_ptr() for t in tensors])

    def forward(self, *inputs: torch.Tensor) -> List[torch.Tensor]:
        dev = inputs[0].device if inputs else torch.device("cpu")
        inputs = [t.contiguous() for t in inputs]
        outs = [torch.empty(d.shape, dtype=d.dtype, device=dev) for d in self.desc.output_descs]
        if dev.type == "cuda":
            if not self.supports_cuda:
                raise RuntimeError("operator %s has no CUDA implementation" % self.desc.name)
            self.lib.forward_op_cuda(self.handle, self._ptrs(inputs), self._ptrs(outs),
                                     C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        else:
            self.lib.forward_op(self.handle, self._ptrs(inputs), self._ptrs(outs))
        return outs

    def backward(self, grads, fwd_inputs, fwd_outputs) -> List[torch.Tensor]:
        dev = grads[0].device
        grads = [g.contiguous() for g in grads]
        igrads = [torch.zeros(d.shape, dtype=d.dtype, device=dev) for d in self.desc.input_descs]
        args = (self._ptrs(grads), self._ptrs(fwd_inputs), self._ptrs(fwd_outputs), self._ptrs(igrads))
        if dev.type == "cuda":
            self.lib.backward_op_cuda(self.handle, *args, C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        else:
            self.lib.backward_op(self.handle, *args)
        return igrads

    def __del__(self):
        try:
            self.lib.delete_op(self.handle)
        except Exception:
            pass


def compile_custom_op(name: str, source: str, input_descs, output_descs, is_file: bool = False,
                      cuda: bool = False, additional_flags=(), defines=None, output_dir: Optional[str] = None,
                      has_backward: bool = True) -> CustomCPPOp:
    """Compile ``source`` (a path when ``is_file`` else the code itself) and instantiate the operator."""
    if is_file:
        files = [source]
    else:
        d = output_dir or os.path.join(tempfile.gettempdir(), "eagersgd_ops", name + "_src")
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, name + (".cu" if cuda else ".cpp"))
        if not os.path.exists(path) or open(path).read() != source:
            with open(path, "w") as f:
                f.write(source)
        files = [path]
    op = CompilableOp(name, files, input_descs, output_descs, has_backward, additional_flags, defines)
    return CustomCPPOp(_build(op, output_dir), op)


compile_custom_cppop_inline = compile_custom_op   # the reference's name for the inline variant


def custom_op(op: CustomCPPOp):
    """A differentiable PyTorch callable around a compiled operator."""

    class _Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *inputs):
            outs = op.forward(*inputs)
            ctx.save_for_backward(*inputs, *outs)
            ctx.nin = len(inputs)
            return outs[0] if len(outs) == 1 else tuple(outs)

        @staticmethod
        def backward(ctx, *grads):
            saved = ctx.saved_tensors
            ins, outs = list(saved[:ctx.nin]), list(saved[ctx.nin:])
            return tuple(op.backward(list(grads), ins, outs))

    return _Fn.apply


def custom_python_op(forward_fn, backward_fn):
    """Operator defined by two Python callables on tensors (deep500 ``CustomPythonOp``)."""

    class _Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *inputs):
            out = forward_fn(*inputs)
            outs = out if isinstance(out, (tuple, list)) else (out,)
            ctx.save_for_backward(*inputs, *outs)
            ctx.nin = len(inputs)
            return out

        @staticmethod
        def backward(ctx, *grads):
            saved = ctx.saved_tensors
            g = backward_fn(list(grads), list(saved[:ctx.nin]), list(saved[ctx.nin:]))
            return tuple(g) if isinstance(g, (tuple, list)) else g

    return _Fn.apply
