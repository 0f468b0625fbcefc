"""B200-native KV-cache write ops behind the ``vllm_xpu_kernels`` plugin interface.

``import vllm_xpu_kernels._C`` maps the op library and registers, for CUDA tensors and with
the schemas of the reference plugin (csrc/torch_bindings.cpp:61-139 and
csrc/flash_attn/flash_api.cpp:179-193 there):

* ``torch.ops._C_cache_ops``: ``reshape_and_cache``, ``reshape_and_cache_flash``,
  ``concat_and_cache_mla``, ``gather_cache`` and, without a counterpart there,
  ``rotary_embedding_and_cache_flash``;
* ``torch.ops._C``: ``rotary_embedding``, ``static_scaled_fp8_quant``,
  ``dynamic_scaled_fp8_quant``, ``dynamic_per_token_scaled_fp8_quant``;
* ``torch.ops._vllm_fa2_C``: ``varlen_fwd`` and ``paged_decode_attention`` (the latter for fp8 caches).

There is no CPU or eager fallback: if the compiled objects are missing the import fails.

``vllm_xpu_kernels.cabi`` binds the same kernels through their C ABI (ctypes),
and ``vllm_xpu_kernels.ops`` holds the thin Python wrappers the reference keeps
in tests/register_ops.py:79-120.
"""
import torch  # noqa: F401  (libtorch must be mapped before the op library)

__version__ = "0.1.0"
