// Entry points of the operator library.
//
// Role parity: csrc/core/registration.h:5-26 of the reference, which emits an
// empty Python module init so that the shared object can also be imported as a
// module.  The operators themselves are reached through torch.ops after
// torch.ops.load_library().
#pragma once

#include <Python.h>
#include <torch/library.h>

namespace pplx {

void register_all_to_all_ops(torch::Library& m);
void register_symmetric_memory_ops(torch::Library& m);
// Operators beyond the reference's surface: block quantisation, grouped GEMM,
// fused MoE layer.
void register_extension_ops(torch::Library& m);

}  // namespace pplx

#define PPLX_CONCAT_(a, b) a##b
#define PPLX_CONCAT(a, b) PPLX_CONCAT_(a, b)
#define PPLX_STRINGIFY_(x) #x
#define PPLX_STRINGIFY(x) PPLX_STRINGIFY_(x)

#define PPLX_REGISTER_EXTENSION(NAME)                                                  \
  extern "C" PyMODINIT_FUNC PPLX_CONCAT(PyInit_, NAME)() {                             \
    static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, PPLX_STRINGIFY(NAME),   \
                                        nullptr, 0, nullptr};                          \
    return PyModule_Create(&module);                                                   \
  }
