"""Model graphs (ONNX-shaped object model, visitors) and their execution with this framework's operators."""
from .ir import Graph, Operation, Visitor, EmptyVisitor, OpCounter, STANDARD_OPS, LOSS_OPS, EXTENSION_OPS  # noqa: F401
from .executor import GraphNetwork, from_torch_resnet  # noqa: F401
from .onnx_io import load_onnx, save_onnx, parse_onnx, dump_onnx  # noqa: F401
from .reference_executor import ReferenceGraphExecutor  # noqa: F401
from .onnx_ops import operator_class, operator_names, make_operation  # noqa: F401
from .from_torch import from_torch_module, export_network  # noqa: F401
from .onnx_test import OnnxTestParser, OnnxTestData, OnnxTest, write_case, load_tensor_pb, save_tensor_pb  # noqa: F401
