"""Loads the op library, which registers ``torch.ops._vllm_fa2_C.varlen_fwd`` (paged decode case) and
``torch.ops._vllm_fa2_C.paged_decode_attention``.  The reference ships a separate compiled module of this
name (vllm_xpu_kernels/flash_attn_interface.py:7-13 there); here all ops live in one shared object."""
from . import _C  # noqa: F401
