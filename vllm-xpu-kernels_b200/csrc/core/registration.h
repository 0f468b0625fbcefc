// Glue for loading the op library with a plain `import`.
//
// The shared object is a CPython extension only so that `import vllm_xpu_kernels._C`
// maps it into the process; mapping it runs the static TORCH_LIBRARY initialisers,
// which is where the ops are registered.  The module object itself stays empty.
// Same contract as the reference's csrc/core/registration.h:21-34.
#pragma once
#include <Python.h>

#define KVC_PP_CAT_(a, b) a##b
#define KVC_PP_CAT(a, b) KVC_PP_CAT_(a, b)
#define KVC_PP_STR_(a) #a
#define KVC_PP_STR(a) KVC_PP_STR_(a)

// TORCH_LIBRARY with a namespace that is itself a macro (TORCH_EXTENSION_NAME-derived).
#define KVC_TORCH_LIBRARY(ns, m) TORCH_LIBRARY(ns, m)
#define KVC_TORCH_LIBRARY_IMPL(ns, key, m) TORCH_LIBRARY_IMPL(ns, key, m)

// Emits PyInit_<name>, returning an empty module.  Limited-API only, so the object can
// be named <name>.abi3.so and serve every CPython 3 minor version.
#define KVC_DEFINE_EMPTY_PYMODULE(name)                                               \
  extern "C" __attribute__((visibility("default"))) PyObject* KVC_PP_CAT(PyInit_, name)(void) { \
    static PyModuleDef def = {PyModuleDef_HEAD_INIT, KVC_PP_STR(name), nullptr, 0, nullptr,     \
                              nullptr,               nullptr,          nullptr, nullptr};       \
    return PyModule_Create(&def);                                                     \
  }
