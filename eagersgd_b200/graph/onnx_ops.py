"""The ONNX operator set as classes: one ``Operation`` subclass per standard operator, with its attributes
(names and defaults) and the number of inputs it takes.

The reference ships 115 operator classes generated from the ONNX schema
(deep500/utils/onnx_interop/generated_operators.py, built by generate_operators.py) so that parsed models become
typed objects for its visitors.  Here the classes are made at import time from the table below: ``op.pads`` reads an
attribute (or its default), ``op.validate()`` rejects attributes the operator does not have and wrong input counts,
``isinstance(op, operator_class("Conv"))`` works for graphs built in code and for parsed ``.onnx`` files alike
(``Graph.add`` makes the right class).  Operators outside the table stay plain ``Operation`` objects.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

REQUIRED = object()      # marks an attribute without a default
INF = 1 << 30

# name: (attributes {name: default}, min inputs, max inputs)
SCHEMA: Dict[str, Tuple[Dict[str, Any], int, int]] = {}


def _op(name: str, lo: int, hi: int, **attrs) -> None:
    SCHEMA[name] = (attrs, lo, hi)


# ---- elementwise, unary -----------------------------------------------------------------------------------------
for _n in ("Abs", "Acos", "Acosh", "Asin", "Asinh", "Atan", "Atanh", "Ceil", "Cos", "Cosh", "Erf", "Exp", "Floor",
           "Identity", "IsNaN", "Log", "Neg", "Not", "Reciprocal", "Relu", "Round", "Sigmoid", "Sign", "Sin", "Sinh",
           "Softplus", "Softsign", "Sqrt", "Tan", "Tanh", "NonZero", "Shape", "Size"):
    _op(_n, 1, 1)
_op("LeakyRelu", 1, 1, alpha=0.01)
_op("Elu", 1, 1, alpha=1.0)
_op("Selu", 1, 1, alpha=1.67326319217681884765625, gamma=1.05070102214813232421875)
_op("Celu", 1, 1, alpha=1.0)
_op("HardSigmoid", 1, 1, alpha=0.2, beta=0.5)
_op("ThresholdedRelu", 1, 1, alpha=1.0)
_op("Shrink", 1, 1, bias=0.0, lambd=0.5)
_op("PRelu", 2, 2)
_op("Clip", 1, 3, min=None, max=None)
_op("IsInf", 1, 1, detect_negative=1, detect_positive=1)
_op("Cast", 1, 1, to=REQUIRED)
_op("Softmax", 1, 1, axis=-1)
_op("LogSoftmax", 1, 1, axis=-1)
_op("Hardmax", 1, 1, axis=-1)
_op("Dropout", 1, 3, seed=None, ratio=0.5)
_op("LRN", 1, 1, alpha=0.0001, beta=0.75, bias=1.0, size=REQUIRED)
_op("LpNormalization", 1, 1, axis=-1, p=2)
_op("MeanVarianceNormalization", 1, 1, axes=[0, 2, 3])
_op("CumSum", 2, 2, exclusive=0, reverse=0)
# ---- elementwise, binary / variadic ---------------------------------------------------------------------------------
for _n in ("Add", "Sub", "Mul", "Div", "Pow", "And", "Or", "Xor", "Equal", "Greater", "GreaterOrEqual", "Less",
           "LessOrEqual"):
    _op(_n, 2, 2)
_op("BitShift", 2, 2, direction=REQUIRED)
_op("Mod", 2, 2, fmod=0)
for _n in ("Sum", "Mean", "Max", "Min"):
    _op(_n, 1, INF)
_op("Where", 3, 3)
# ---- matrix products ---------------------------------------------------------------------------------------------
_op("MatMul", 2, 2)
_op("MatMulInteger", 2, 4)
_op("Gemm", 2, 3, alpha=1.0, beta=1.0, transA=0, transB=0)
_op("Einsum", 1, INF, equation=REQUIRED)
# ---- convolutions, pooling, normalisation ------------------------------------------------------------------------
_op("Conv", 2, 3, auto_pad="NOTSET", dilations=None, group=1, kernel_shape=None, pads=None, strides=None)
_op("ConvInteger", 2, 4, auto_pad="NOTSET", dilations=None, group=1, kernel_shape=None, pads=None, strides=None)
_op("ConvTranspose", 2, 3, auto_pad="NOTSET", dilations=None, group=1, kernel_shape=None, output_padding=None,
    output_shape=None, pads=None, strides=None)
_op("MaxPool", 1, 1, auto_pad="NOTSET", ceil_mode=0, dilations=None, kernel_shape=REQUIRED, pads=None, storage_order=0,
    strides=None)
_op("AveragePool", 1, 1, auto_pad="NOTSET", ceil_mode=0, count_include_pad=0, kernel_shape=REQUIRED, pads=None,
    strides=None)
_op("LpPool", 1, 1, auto_pad="NOTSET", kernel_shape=REQUIRED, p=2, pads=None, strides=None)
_op("MaxUnpool", 2, 3, kernel_shape=REQUIRED, pads=None, strides=None)
_op("MaxRoiPool", 2, 2, pooled_shape=REQUIRED, spatial_scale=1.0)
_op("RoiAlign", 3, 3, mode="avg", output_height=1, output_width=1, sampling_ratio=0, spatial_scale=1.0)
for _n in ("GlobalAveragePool", "GlobalMaxPool"):
    _op(_n, 1, 1)
_op("GlobalLpPool", 1, 1, p=2)
_op("BatchNormalization", 5, 5, epsilon=1e-5, momentum=0.9, training_mode=0, spatial=1)
_op("InstanceNormalization", 3, 3, epsilon=1e-5)
# ---- reductions ------------------------------------------------------------------------------------------------------
for _n in ("ReduceL1", "ReduceL2", "ReduceLogSum", "ReduceLogSumExp", "ReduceMax", "ReduceMean", "ReduceMin",
           "ReduceProd", "ReduceSumSquare"):
    _op(_n, 1, 1, axes=None, keepdims=1)
_op("ReduceSum", 1, 2, axes=None, keepdims=1, noop_with_empty_axes=0)
_op("ArgMax", 1, 1, axis=0, keepdims=1, select_last_index=0)
_op("ArgMin", 1, 1, axis=0, keepdims=1, select_last_index=0)
_op("TopK", 2, 2, axis=-1, largest=1, sorted=1)
# ---- shapes and data movement --------------------------------------------------------------------------------------
_op("Reshape", 1, 2, allowzero=0, shape=None)
_op("Flatten", 1, 1, axis=1)
_op("Squeeze", 1, 2, axes=None)
_op("Unsqueeze", 1, 2, axes=None)
_op("Transpose", 1, 1, perm=None)
_op("Concat", 1, INF, axis=REQUIRED)
_op("Split", 1, 2, axis=0, split=None)
_op("Slice", 3, 5)
_op("Gather", 2, 2, axis=0)
_op("GatherElements", 2, 2, axis=0)
_op("GatherND", 2, 2, batch_dims=0)
_op("Scatter", 3, 3, axis=0)
_op("ScatterElements", 3, 3, axis=0)
_op("ScatterND", 3, 3)
_op("Expand", 2, 2)
_op("Tile", 2, 2)
_op("Pad", 1, 3, mode="constant", pads=None, value=0.0)
_op("DepthToSpace", 1, 1, blocksize=REQUIRED, mode="DCR")
_op("SpaceToDepth", 1, 1, blocksize=REQUIRED)
_op("Resize", 1, 4, coordinate_transformation_mode="half_pixel", cubic_coeff_a=-0.75, exclude_outside=0,
    extrapolation_value=0.0, mode="nearest", nearest_mode="round_prefer_floor")
_op("Upsample", 1, 2, mode="nearest", scales=None)
_op("Compress", 2, 2, axis=None)
_op("OneHot", 3, 3, axis=-1)
_op("ReverseSequence", 2, 2, batch_axis=1, time_axis=0)
_op("Unique", 1, 1, axis=None, sorted=1)
_op("Trilu", 1, 2, upper=1)
_op("EyeLike", 1, 1, dtype=None, k=0)
_op("Range", 3, 3)
# ---- constants and random ------------------------------------------------------------------------------------------
_op("Constant", 0, 0, value=None, value_float=None, value_floats=None, value_int=None, value_ints=None,
    value_string=None, value_strings=None, sparse_value=None)
_op("ConstantOfShape", 1, 1, value=None)
_op("RandomNormal", 0, 0, dtype=1, mean=0.0, scale=1.0, seed=None, shape=REQUIRED)
_op("RandomNormalLike", 1, 1, dtype=None, mean=0.0, scale=1.0, seed=None)
_op("RandomUniform", 0, 0, dtype=1, high=1.0, low=0.0, seed=None, shape=REQUIRED)
_op("RandomUniformLike", 1, 1, dtype=None, high=1.0, low=0.0, seed=None)
_op("Multinomial", 1, 1, dtype=6, sample_size=1, seed=None)
# ---- recurrent -----------------------------------------------------------------------------------------------------------
_RNN = dict(activation_alpha=None, activation_beta=None, activations=None, clip=None, direction="forward",
            hidden_size=None)
_op("RNN", 3, 6, **_RNN)
_op("GRU", 3, 6, linear_before_reset=0, **_RNN)
_op("LSTM", 3, 8, input_forget=0, **_RNN)
# ---- quantisation, control flow, sequences, text ------------------------------------------------------------------------
_op("QuantizeLinear", 2, 3, axis=1)
_op("DequantizeLinear", 2, 3, axis=1)
_op("DynamicQuantizeLinear", 1, 1)
_op("QLinearConv", 8, 9, auto_pad="NOTSET", dilations=None, group=1, kernel_shape=None, pads=None, strides=None)
_op("QLinearMatMul", 8, 8)
_op("If", 1, 1, else_branch=REQUIRED, then_branch=REQUIRED)
_op("Loop", 2, INF, body=REQUIRED)
_op("Scan", 1, INF, body=REQUIRED, num_scan_inputs=REQUIRED, scan_input_axes=None, scan_input_directions=None,
    scan_output_axes=None, scan_output_directions=None)
_op("NonMaxSuppression", 2, 5, center_point_box=0)
_op("TfIdfVectorizer", 1, 1, max_gram_length=REQUIRED, max_skip_count=REQUIRED, min_gram_length=REQUIRED, mode=REQUIRED,
    ngram_counts=REQUIRED, ngram_indexes=REQUIRED, pool_int64s=None, pool_strings=None, weights=None)
_op("StringNormalizer", 1, 1, case_change_action="NONE", is_case_sensitive=0, locale=None, stopwords=None)
_op("Det", 1, 1)
_op("NegativeLogLikelihoodLoss", 2, 3, ignore_index=None, reduction="mean")
_op("SoftmaxCrossEntropyLoss", 2, 3, ignore_index=None, reduction="mean")
for _n in ("SequenceConstruct", "ConcatFromSequence", "SequenceAt", "SequenceEmpty", "SequenceErase", "SequenceInsert",
           "SequenceLength", "SplitToSequence"):
    _op(_n, 0, INF)
SCHEMA["ConcatFromSequence"] = ({"axis": REQUIRED, "new_axis": 0}, 1, 1)
SCHEMA["SplitToSequence"] = ({"axis": 0, "keepdims": 1}, 1, 2)
SCHEMA["SequenceEmpty"] = ({"dtype": None}, 0, 0)
# ---- this framework's additions (losses and gradient extensions of the reference's object model) ---------------------
for _n in ("SoftmaxCrossEntropy", "CrossEntropy", "MeanSquaredError"):
    _op(_n, 2, 2)
# ---- the experimental operators of the ONNX release the reference generated its classes from (deep500/utils/
# onnx_interop/generated_operators.py has a class for each; later ONNX releases dropped them) -------------------------
_op("Affine", 1, 1, alpha=1.0, beta=0.0)                        # alpha * x + beta
_op("Scale", 1, 1, scale=1.0)
_op("ScaledTanh", 1, 1, alpha=1.0, beta=1.0)                    # alpha * tanh(beta * x)
_op("ParametricSoftplus", 1, 1, alpha=1.0, beta=1.0)            # alpha * log(exp(beta * x) + 1)
_op("ImageScaler", 1, 1, bias=None, scale=1.0)                  # x * scale + bias[channel]
_op("Crop", 1, 1, border=None, scale=None)                      # border = left, top, right, bottom; or scale = height, width
_op("ConstantFill", 0, 1, dtype=1, extra_shape=None, input_as_shape=0, shape=None, value=0.0)
_op("GivenTensorFill", 0, 1, extra_shape=None, input_as_shape=0, shape=None, values=None)
_op("GRUUnit", 4, 4, drop_states=0)                             # hidden_prev, gates, seq_lengths, t
_op("LoopIndexTensor", 2, 2, axis=0)
_op("StopGradient", 1, 1)
_op("AllReduceGradients", 1, 1)
_op("ConsistentParameterServerGradients", 1, 1)
_op("InconsistentParameterServerGradients", 1, 1)

_op("ATen", 0, INF, operator=None)                              # a call into the exporting framework: any attributes
ANY_ATTRIBUTES = {"ATen"}

_CLASSES: Dict[str, type] = {}


def _make_class(op_type: str):
    from .ir import Operation
    attrs, lo, hi = SCHEMA[op_type]
    open_ended = op_type in ANY_ATTRIBUTES

    def validate(self) -> None:
        unknown = sorted(set(self.attrs) - set(attrs))
        if unknown and not open_ended:
            raise ValueError("%s has no attribute %s (it has: %s)" % (op_type, ", ".join(unknown), ", ".join(sorted(attrs)) or "none"))
        missing = sorted(a for a, d in attrs.items() if d is REQUIRED and a not in self.attrs)
        if missing:
            raise ValueError("%s needs the attribute %s" % (op_type, ", ".join(missing)))
        n = len([i for i in self.inputs if i != ""])
        if not (lo <= len(self.inputs) and n <= hi):
            raise ValueError("%s takes %s inputs, not %d" % (op_type, lo if lo == hi else "%d to %s" % (lo, "any number of" if hi >= INF else hi), n))

    def __getattr__(self, name):          # attribute access with the schema's defaults
        if name.startswith("_") or name in ("attrs", "inputs", "outputs", "op_type", "name"):
            raise AttributeError(name)
        if name in self.__dict__.get("attrs", {}):
            return self.attrs[name]
        if name in attrs:
            d = attrs[name]
            if d is REQUIRED:
                raise AttributeError("%s: required attribute %r is not set" % (op_type, name))
            return d
        raise AttributeError("%s has no attribute %r" % (op_type, name))

    return type(op_type, (Operation,), {"ATTRIBUTES": dict(attrs), "MIN_INPUTS": lo, "MAX_INPUTS": hi,
                                        "validate": validate, "__getattr__": __getattr__,
                                        "__doc__": "ONNX operator %s (attributes: %s)" % (op_type, ", ".join(sorted(attrs)) or "none")})


def operator_class(op_type: str) -> Optional[type]:
    """The class of a standard operator, or None for an operator outside the table."""
    if op_type not in SCHEMA:
        return None
    if op_type not in _CLASSES:
        _CLASSES[op_type] = _make_class(op_type)
    return _CLASSES[op_type]


def make_operation(op_type: str, inputs, outputs, name=None, **attrs):
    """An operation object of the operator's own class (plain ``Operation`` for unknown operators)."""
    from .ir import Operation
    cls = operator_class(op_type)
    return (cls or Operation)(op_type, inputs, outputs, name=name, **attrs)


def operator_names():
    return sorted(SCHEMA)
