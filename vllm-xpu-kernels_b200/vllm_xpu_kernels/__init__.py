"""B200-native KV-cache write ops behind the ``vllm_xpu_kernels`` plugin interface.

``import vllm_xpu_kernels._C`` maps the op library and registers
``torch.ops._C_cache_ops.reshape_and_cache`` and ``reshape_and_cache_flash`` for
CUDA tensors, with the schemas of the reference plugin
(csrc/torch_bindings.cpp:107-124 there).  There is no CPU or eager fallback: if
the compiled objects are missing the import fails.

``vllm_xpu_kernels.cabi`` binds the same kernels through their C ABI (ctypes),
and ``vllm_xpu_kernels.ops`` holds the thin Python wrappers the reference keeps
in tests/register_ops.py:79-120.
"""
import torch  # noqa: F401  (libtorch must be mapped before the op library)

__version__ = "0.1.0"
