"""``scaled_fp8_quant``: the convenience wrapper the reference keeps in tests/ops/fp8_quant_op.py:13-79
(itself vLLM's ``ops.scaled_fp8_quant``), over ``torch.ops._C.{static,dynamic,dynamic_per_token}_scaled_fp8_quant``."""
from typing import Optional, Union

import torch

from . import _C  # noqa: F401  (registers the ops; raises ImportError if not built)


def scaled_fp8_quant(
    input: torch.Tensor,
    scale: Optional[torch.Tensor] = None,
    num_token_padding: Optional[int] = None,
    scale_ub: Optional[torch.Tensor] = None,
    use_per_token_if_dynamic: bool = False,
    output: Optional[torch.Tensor] = None,
    fp8_dtype: torch.dtype = torch.float8_e5m2,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantise a 2-D tensor to fp8; returns (quantised, scale).

    With ``scale`` given the quantisation is static; without it the scale is the tensor's (or, with
    ``use_per_token_if_dynamic``, each row's) absmax / fp8_max, optionally capped through ``scale_ub``.
    ``num_token_padding`` pads the first dim of the output for consumers that want it."""
    assert input.ndim == 2
    shape: Union[tuple[int, int], torch.Size] = input.shape
    if num_token_padding:
        shape = (max(num_token_padding, input.shape[0]), shape[1])
    if output is None:
        output = torch.empty(shape, device=input.device, dtype=fp8_dtype)
    else:
        assert num_token_padding is None, "padding not supported if output passed in"
        assert output.dtype == fp8_dtype
    if scale is None:
        if use_per_token_if_dynamic:
            scale = torch.zeros((shape[0], 1), device=input.device, dtype=torch.float32)
            torch.ops._C.dynamic_per_token_scaled_fp8_quant(output, input.contiguous(), scale, scale_ub)
        else:
            scale = torch.zeros(1, device=input.device, dtype=torch.float32)
            torch.ops._C.dynamic_scaled_fp8_quant(output, input, scale)
    else:
        assert scale.numel() == 1, f"{scale.shape}"
        torch.ops._C.static_scaled_fp8_quant(output, input, scale)
    return output, scale
