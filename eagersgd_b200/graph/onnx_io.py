"""Read and write ``.onnx`` files without the ``onnx`` package: a small protobuf wire-format codec for the
messages a model file is made of (ModelProto, GraphProto, NodeProto, AttributeProto, TensorProto,
ValueInfoProto), mapped onto ``graph.ir.Graph``.

``load_onnx(path)`` is the counterpart of the reference's ``load_and_parse_model``
(deep500/utils/onnx_interop/parser.py:1-59, onnx_objects.py: OnnxModel / OnnxGraph / OnnxNode / OnnxTensor):
nodes become ``Operation`` objects with their attributes as Python values, initializers become numpy arrays,
graph inputs that are initializers are not listed as inputs.  ``save_onnx(graph, path)`` writes a file other
ONNX tools can read (IR version 7, default opset 13).  Field numbers are those of onnx.proto3.
"""
from __future__ import annotations

import struct
from typing import Any, Dict, Iterator, List, Optional, Tuple

import numpy as np

from .ir import Graph, Operation

# TensorProto.DataType -> numpy
_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 4: np.uint16, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_,
           10: np.float16, 11: np.float64, 12: np.uint32, 13: np.uint64}
_DTYPE_IDS = {np.dtype(v): k for k, v in _DTYPES.items()}
_BFLOAT16 = 16
# AttributeProto.AttributeType
_A_FLOAT, _A_INT, _A_STRING, _A_TENSOR, _A_FLOATS, _A_INTS, _A_STRINGS = 1, 2, 3, 4, 6, 7, 8


# ---- wire format ---------------------------------------------------------------------------------------------
def _varint(buf: bytes, pos: int) -> Tuple[int, int]:
    result = shift = 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7
        if shift > 70:
            raise ValueError("malformed varint")


def _fields(buf: bytes) -> Iterator[Tuple[int, int, Any]]:
    """Yield (field number, wire type, value) of one message; length-delimited values come as bytes."""
    pos, end = 0, len(buf)
    while pos < end:
        key, pos = _varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == 0:
            val, pos = _varint(buf, pos)
        elif wt == 1:
            val, pos = buf[pos:pos + 8], pos + 8
        elif wt == 2:
            n, pos = _varint(buf, pos)
            val, pos = buf[pos:pos + n], pos + n
        elif wt == 5:
            val, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ValueError("unsupported protobuf wire type %d" % wt)
        yield num, wt, val


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_varints(val, wt) -> List[int]:
    if wt == 0:
        return [_signed(val)]
    out, pos = [], 0
    while pos < len(val):
        v, pos = _varint(val, pos)
        out.append(_signed(v))
    return out


def _enc_varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _enc_field(num: int, wt: int, payload: bytes) -> bytes:
    key = _enc_varint((num << 3) | wt)
    return key + (_enc_varint(len(payload)) + payload if wt == 2 else payload)


def _enc_str(num: int, s: str) -> bytes:
    return _enc_field(num, 2, s.encode())


def _enc_int(num: int, v: int) -> bytes:
    return _enc_field(num, 0, _enc_varint(v))


# ---- decoding ------------------------------------------------------------------------------------------------------
def _parse_tensor(buf: bytes) -> Tuple[str, np.ndarray]:
    dims: List[int] = []
    dtype_id, name, raw = 1, "", None
    floats: List[float] = []
    ints: List[int] = []
    doubles: List[float] = []
    for num, wt, val in _fields(buf):
        if num == 1:
            dims += _packed_varints(val, wt)
        elif num == 2:
            dtype_id = val
        elif num == 4:      # float_data (packed or not)
            floats += list(struct.unpack("<%df" % (len(val) // 4), val)) if wt == 2 else [struct.unpack("<f", val)[0]]
        elif num in (5, 7):  # int32_data / int64_data
            ints += _packed_varints(val, wt)
        elif num == 8:
            name = val.decode()
        elif num == 9:
            raw = val
        elif num == 10:
            doubles += list(struct.unpack("<%dd" % (len(val) // 8), val)) if wt == 2 else [struct.unpack("<d", val)[0]]
    if dtype_id == _BFLOAT16:
        src = np.frombuffer(raw, dtype=np.uint16) if raw is not None else np.asarray(ints, dtype=np.uint16)
        arr = (src.astype(np.uint32) << 16).view(np.float32)
    else:
        if dtype_id not in _DTYPES:
            raise ValueError("tensor %r: unsupported ONNX data type %d" % (name, dtype_id))
        dt = np.dtype(_DTYPES[dtype_id])
        if raw is not None:
            arr = np.frombuffer(raw, dtype=dt.newbyteorder("<")).astype(dt)
        elif dtype_id == 10 and ints:         # float16 travels as uint16 bit patterns in int32_data
            arr = np.asarray(ints, dtype=np.uint16).view(np.float16)
        elif floats:
            arr = np.asarray(floats, dtype=dt)
        elif doubles:
            arr = np.asarray(doubles, dtype=dt)
        else:
            arr = np.asarray(ints, dtype=dt)
    return name, arr.reshape(dims) if dims or arr.size == 1 else arr


def _parse_attribute(buf: bytes) -> Tuple[str, Any]:
    name, atype = "", 0
    f = i = s = t = None
    floats: List[float] = []
    ints: List[int] = []
    strings: List[str] = []
    for num, wt, val in _fields(buf):
        if num == 1:
            name = val.decode()
        elif num == 2:
            f = struct.unpack("<f", val)[0]
        elif num == 3:
            i = _signed(val)
        elif num == 4:
            s = val
        elif num == 5:
            t = _parse_tensor(val)[1]
        elif num == 7:
            floats += list(struct.unpack("<%df" % (len(val) // 4), val)) if wt == 2 else [struct.unpack("<f", val)[0]]
        elif num == 8:
            ints += _packed_varints(val, wt)
        elif num == 9:
            strings.append(val.decode())
        elif num == 20:
            atype = val
    if atype == _A_FLOAT or (atype == 0 and f is not None):
        return name, f
    if atype == _A_INT or (atype == 0 and i is not None):
        return name, i
    if atype == _A_STRING or (atype == 0 and s is not None):
        return name, s.decode(errors="replace") if s is not None else ""
    if atype == _A_TENSOR or (atype == 0 and t is not None):
        return name, t
    if atype == _A_FLOATS or (atype == 0 and floats):
        return name, floats
    if atype == _A_STRINGS or (atype == 0 and strings):
        return name, strings
    return name, ints


def _parse_node(buf: bytes) -> Operation:
    inputs, outputs, attrs = [], [], {}
    name, op_type = None, ""
    for num, wt, val in _fields(buf):
        if num == 1:
            inputs.append(val.decode())
        elif num == 2:
            outputs.append(val.decode())
        elif num == 3:
            name = val.decode() or None
        elif num == 4:
            op_type = val.decode()
        elif num == 5:
            k, v = _parse_attribute(val)
            attrs[k] = v
    from .onnx_ops import make_operation
    return make_operation(op_type, inputs, outputs, name, **attrs)


def _value_info_name_shape(buf: bytes) -> Tuple[str, Optional[List[Any]]]:
    name, shape = "", None
    for num, wt, val in _fields(buf):
        if num == 1:
            name = val.decode()
        elif num == 2:                                   # TypeProto
            for n2, _, v2 in _fields(val):
                if n2 == 1:                              # tensor_type
                    for n3, _, v3 in _fields(v2):
                        if n3 == 2:                      # TensorShapeProto
                            shape = []
                            for n4, _, v4 in _fields(v3):
                                if n4 == 1:              # Dimension
                                    dim: Any = None
                                    for n5, _, v5 in _fields(v4):
                                        dim = _signed(v5) if n5 == 1 else v5.decode() if n5 == 2 else dim
                                    shape.append(dim)
    return name, shape


def parse_onnx(data: bytes) -> Graph:
    """Decode the bytes of a ModelProto into a ``Graph`` (``graph.meta`` keeps ir / opset / producer / shapes)."""
    graph_buf = None
    meta: Dict[str, Any] = {"opsets": {}}
    for num, wt, val in _fields(data):
        if num == 1:
            meta["ir_version"] = val
        elif num == 2:
            meta["producer_name"] = val.decode()
        elif num == 7:
            graph_buf = val
        elif num == 8:                                    # OperatorSetIdProto
            dom, ver = "", 0
            for n2, _, v2 in _fields(val):
                dom, ver = (v2.decode(), ver) if n2 == 1 else (dom, v2) if n2 == 2 else (dom, ver)
            meta["opsets"][dom] = ver
    if graph_buf is None:
        raise ValueError("not an ONNX model: no graph")
    g = Graph()
    shapes: Dict[str, Any] = {}
    declared_inputs: List[str] = []
    for num, wt, val in _fields(graph_buf):
        if num == 1:
            g.ops.append(_parse_node(val))
        elif num == 2:
            g.name = val.decode() or "graph"
        elif num == 5:
            n, arr = _parse_tensor(val)
            g.initializers[n] = arr
        elif num == 11:
            n, shp = _value_info_name_shape(val)
            declared_inputs.append(n)
            shapes[n] = shp
        elif num == 12:
            n, shp = _value_info_name_shape(val)
            g.outputs.append(n)
            shapes[n] = shp
        elif num == 13:
            n, shp = _value_info_name_shape(val)
            shapes[n] = shp
    g.inputs = [n for n in declared_inputs if n not in g.initializers]   # old exporters list weights as inputs too
    seen = set()
    for op in g.ops:                                                     # node names must be unique for our tools
        if op.name in seen:
            op.name = "%s_%d" % (op.name, len(seen))
        seen.add(op.name)
    meta["shapes"] = shapes
    g.meta = meta
    _normalise_for_executor(g)
    return g


def _normalise_for_executor(g: Graph) -> None:
    """Bring opset differences to the attribute form ``graph.executor`` reads: Reshape / Squeeze / Unsqueeze /
    ReduceX take their shape or axes from an attribute here, newer opsets pass them as a constant input."""
    consts = dict(g.initializers)
    for op in g.ops:
        if op.op_type == "Constant" and "value" in op.attrs:
            consts[op.outputs[0]] = np.asarray(op.attrs["value"])
    for op in g.ops:
        if op.op_type == "Reshape" and "shape" not in op.attrs and len(op.inputs) > 1 and op.inputs[1] in consts:
            op.attrs["shape"] = [int(v) for v in consts[op.inputs[1]].reshape(-1)]
        if op.op_type in ("Squeeze", "Unsqueeze", "ReduceMean", "ReduceSum") and "axes" not in op.attrs and \
                len(op.inputs) > 1 and op.inputs[1] in consts:
            op.attrs["axes"] = [int(v) for v in consts[op.inputs[1]].reshape(-1)]


def load_onnx(path: str) -> Graph:
    with open(path, "rb") as f:
        return parse_onnx(f.read())


# ---- encoding ------------------------------------------------------------------------------------------------------
def _enc_tensor(name: str, arr: np.ndarray) -> bytes:
    arr = np.asarray(arr, order="C")          # not ascontiguousarray: that turns a scalar into a vector of one
    if arr.dtype not in _DTYPE_IDS:
        arr = arr.astype(np.float32)
    out = b"".join(_enc_int(1, int(d)) for d in arr.shape)
    out += _enc_int(2, _DTYPE_IDS[arr.dtype]) + _enc_str(8, name)
    out += _enc_field(9, 2, arr.astype(arr.dtype.newbyteorder("<")).tobytes())
    return out


def _enc_attribute(name: str, value: Any) -> bytes:
    out = _enc_str(1, name)
    if isinstance(value, bool):
        value = int(value)
    if isinstance(value, float):
        return out + _enc_field(2, 5, struct.pack("<f", value)) + _enc_int(20, _A_FLOAT)
    if isinstance(value, (int, np.integer)):
        return out + _enc_int(3, int(value)) + _enc_int(20, _A_INT)
    if isinstance(value, str):
        return out + _enc_str(4, value) + _enc_int(20, _A_STRING)
    if isinstance(value, np.ndarray):
        return out + _enc_field(5, 2, _enc_tensor("", value)) + _enc_int(20, _A_TENSOR)
    seq = list(value)
    if seq and all(isinstance(v, str) for v in seq):
        return out + b"".join(_enc_str(9, v) for v in seq) + _enc_int(20, _A_STRINGS)
    if seq and any(isinstance(v, float) for v in seq):
        return out + b"".join(_enc_field(7, 5, struct.pack("<f", float(v))) for v in seq) + _enc_int(20, _A_FLOATS)
    return out + b"".join(_enc_int(8, int(v)) for v in seq) + _enc_int(20, _A_INTS)


def _enc_value_info(name: str, shape=None, elem_type: int = 1) -> bytes:
    tensor_type = _enc_int(1, elem_type)
    if shape is not None:
        dims = b""
        for d in shape:
            dims += _enc_field(1, 2, _enc_str(2, d) if isinstance(d, str) else _enc_int(1, int(d if d is not None else 0)))
        tensor_type += _enc_field(2, 2, dims)
    return _enc_str(1, name) + _enc_field(2, 2, _enc_field(1, 2, tensor_type))


def dump_onnx(graph: Graph, opset: int = 13, producer: str = "eagersgd_b200") -> bytes:
    shapes = getattr(graph, "meta", {}).get("shapes", {}) if hasattr(graph, "meta") else {}
    g = b""
    for op in graph.ops:
        node = b"".join(_enc_str(1, i) for i in op.inputs) + b"".join(_enc_str(2, o) for o in op.outputs)
        node += _enc_str(3, op.name) + _enc_str(4, op.op_type)
        node += b"".join(_enc_field(5, 2, _enc_attribute(k, v)) for k, v in op.attrs.items())
        g += _enc_field(1, 2, node)
    g += _enc_str(2, graph.name)
    for name, arr in graph.initializers.items():
        g += _enc_field(5, 2, _enc_tensor(name, np.asarray(arr)))
    for name in graph.inputs:
        g += _enc_field(11, 2, _enc_value_info(name, shapes.get(name)))
    for name in graph.outputs:
        g += _enc_field(12, 2, _enc_value_info(name, shapes.get(name)))
    model = _enc_int(1, 7) + _enc_str(2, producer) + _enc_field(7, 2, g)
    model += _enc_field(8, 2, _enc_str(1, "") + _enc_int(2, opset))
    return model


def save_onnx(graph: Graph, path: str, opset: int = 13) -> None:
    with open(path, "wb") as f:
        f.write(dump_onnx(graph, opset))
