// C++ interface of user-defined operators compiled at run time.
//
// An operator is a class with forward(...) and backward(...) methods over raw pointers (and
// optionally forward_cuda / backward_cuda taking a stream).  ESGD_REGISTER_OP exports the C entry
// points the Python loader binds with ctypes: create_new_op, delete_op, forward_op, backward_op,
// is_cuda_supported and report.  The pointer lists are flat arrays in declaration order (inputs
// first, then outputs; for backward: next-gradients, forward inputs, forward outputs, then the
// input gradients to produce).  Same role as the reference's deep500.h (CustomOperator, tensor_t,
// D500_REGISTER_OP, D500_EXPORTED create_new_op: deep500/lv0/operators/include/deep500/deep500.h:43-124).
#pragma once
#include <stdint.h>

namespace eagersgd {

enum tensortype_t : int32_t { T_FLOAT = 0, T_DOUBLE = 1, T_INT32 = 2, T_INT64 = 3, T_BF16 = 4, T_HALF = 5 };

struct tensor_t {
  int32_t type;
  int32_t dims;
  int64_t sizes[8];
  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < dims; ++i) n *= sizes[i];
    return n;
  }
};

class CustomOperator {
 public:
  virtual ~CustomOperator() {}
  virtual bool supports_cuda() { return false; }
  virtual int64_t report(void* /*data*/) { return 0; }   // e.g. bytes communicated
  virtual void forward(void** /*inputs*/, void** /*outputs*/) {}
  virtual void backward(void** /*nextop_grads*/, void** /*fwd_inputs*/, void** /*fwd_outputs*/, void** /*input_grads*/) {}
  virtual void forward_cuda(void** in, void** out, void* /*stream*/) { forward(in, out); }
  virtual void backward_cuda(void** g, void** in, void** out, void** ig, void* /*stream*/) { backward(g, in, out, ig); }
};

}  // namespace eagersgd

#define ESGD_EXPORTED extern "C" __attribute__((visibility("default")))

// ESGD_REGISTER_OP(ClassName): the class needs a constructor
//   ClassName(const eagersgd::tensor_t* inputs, int ninputs, const eagersgd::tensor_t* outputs, int noutputs)
#define ESGD_REGISTER_OP(cls)                                                                                      \
  ESGD_EXPORTED void* create_new_op(const eagersgd::tensor_t* in, int nin, const eagersgd::tensor_t* out,          \
                                    int nout) {                                                                    \
    return new cls(in, nin, out, nout);                                                                            \
  }                                                                                                                \
  ESGD_EXPORTED void delete_op(void* h) { delete static_cast<eagersgd::CustomOperator*>(h); }                      \
  ESGD_EXPORTED int is_cuda_supported(void* h) { return static_cast<eagersgd::CustomOperator*>(h)->supports_cuda(); } \
  ESGD_EXPORTED int64_t report(void* h, void* d) { return static_cast<eagersgd::CustomOperator*>(h)->report(d); }   \
  ESGD_EXPORTED void forward_op(void* h, void** in, void** out) {                                                  \
    static_cast<eagersgd::CustomOperator*>(h)->forward(in, out);                                                   \
  }                                                                                                                \
  ESGD_EXPORTED void backward_op(void* h, void** g, void** in, void** out, void** ig) {                            \
    static_cast<eagersgd::CustomOperator*>(h)->backward(g, in, out, ig);                                           \
  }                                                                                                                \
  ESGD_EXPORTED void forward_op_cuda(void* h, void** in, void** out, void* s) {                                    \
    static_cast<eagersgd::CustomOperator*>(h)->forward_cuda(in, out, s);                                           \
  }                                                                                                                \
  ESGD_EXPORTED void backward_op_cuda(void* h, void** g, void** in, void** out, void** ig, void* s) {              \
    static_cast<eagersgd::CustomOperator*>(h)->backward_cuda(g, in, out, ig, s);                                   \
  }
