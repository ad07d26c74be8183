"""Write an operator in C++, compile it at run time, use it with autograd and validate it.

    python samples/custom_operator.py

The operator ABI is ``eagersgd/op.h``; the compile pipeline and the validation harness mirror the
reference's operator tutorial (deep500 tutorials/operator.md, samples/custom_operator*.py).
"""
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from eagersgd_b200.ops.compile import TensorDescriptor, compile_custom_op, custom_op  # noqa: E402
from eagersgd_b200.ops.validation import test_op_forward, test_op_gradient  # noqa: E402

SOURCE = r'''
#include <eagersgd/op.h>
#include <cmath>
// y = x * sigmoid(BETA * x)   (swish), with its gradient
class Swish : public eagersgd::CustomOperator {
  int64_t n;
 public:
  Swish(const eagersgd::tensor_t* in, int, const eagersgd::tensor_t*, int) : n(in[0].numel()) {}
  void forward(void** in, void** out) override {
    const float* x = (const float*)in[0]; float* y = (float*)out[0];
    for (int64_t i = 0; i < n; ++i) y[i] = x[i] / (1.0f + std::exp(-BETA * x[i]));
  }
  void backward(void** g, void** in, void**, void** ig) override {
    const float* dy = (const float*)g[0]; const float* x = (const float*)in[0]; float* dx = (float*)ig[0];
    for (int64_t i = 0; i < n; ++i) {
      const float s = 1.0f / (1.0f + std::exp(-BETA * x[i]));
      dx[i] = dy[i] * (s + BETA * x[i] * s * (1.0f - s));
    }
  }
};
ESGD_REGISTER_OP(Swish)
'''


def main():
    d = TensorDescriptor(torch.float32, (4, 8))
    with tempfile.TemporaryDirectory() as tmp:
        op = compile_custom_op("swish", SOURCE, [d], [d], defines={"BETA": "1.5f"}, output_dir=tmp)
        swish = custom_op(op)
        x = torch.randn(4, 8)
        test_op_forward(swish, [x], x * torch.sigmoid(1.5 * x))
        test_op_gradient(swish, [x], eps=1e-2, rtol=2e-2, atol=2e-2)
        y = swish(x.requires_grad_())
        y.sum().backward()
        print("swish ok: forward and numerical-gradient checks passed; |dx| = %.4f" % x.grad.norm())


if __name__ == "__main__":
    main()
