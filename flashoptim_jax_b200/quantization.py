"""Group-wise int8 / uint8 codecs for optimizer moments, on the GPU.

Same names and meaning as the reference module flashoptim_jax/quantization.py:
`values` keeps the tensor's shape, `scales` holds one fp16 absmax per `group_size`
consecutive elements of the row-major flattening (the last group may be short).
"""

from __future__ import annotations

from typing import NamedTuple

import torch

from . import _lib
from ._dev import as_tensor, require_cuda, stream_ptr


class QuantizedArray(NamedTuple):
    """Quantized values paired with per-group scales (flashoptim_jax/quantization.py:9-12)."""

    values: torch.Tensor
    scales: torch.Tensor


def _num_groups(n: int, group_size: int) -> int:
    return (n + group_size - 1) // group_size


def _quantize(x, group_size: int, variance: bool) -> QuantizedArray:
    x = as_tensor(x)
    require_cuda(x, "x")
    xf = x.to(torch.float32).contiguous()
    n = xf.numel()
    values = torch.empty(x.shape, dtype=torch.uint8 if variance else torch.int8, device=x.device)
    scales = torch.empty((_num_groups(n, group_size),), dtype=torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        fn = _lib.lib().fo_quantize_variance if variance else _lib.lib().fo_quantize_momentum
        _lib.check(fn(xf.data_ptr(), values.data_ptr(), scales.data_ptr(), n, int(group_size), 0, stream_ptr(x.device)))
    return QuantizedArray(values=values, scales=scales)


def _dequantize(q: QuantizedArray, group_size: int, variance: bool) -> torch.Tensor:
    values, scales = q.values, q.scales
    require_cuda(values, "values")
    values = values.contiguous()
    scales = scales.to(torch.float16).contiguous()
    out = torch.empty(values.shape, dtype=torch.float32, device=values.device)
    with torch.cuda.device(values.device):
        fn = _lib.lib().fo_dequantize_variance if variance else _lib.lib().fo_dequantize_momentum
        _lib.check(fn(values.data_ptr(), scales.data_ptr(), out.data_ptr(), values.numel(), int(group_size), stream_ptr(values.device)))
    return out


def quantize_momentum(x, group_size: int = 32) -> QuantizedArray:
    """int8 soft-sign codes + fp16 group absmax (flashoptim_jax/quantization.py:37-46)."""
    return _quantize(x, group_size, variance=False)


def dequantize_momentum(x: QuantizedArray, group_size: int = 32) -> torch.Tensor:
    """Inverse of quantize_momentum up to quantization error (flashoptim_jax/quantization.py:49-56)."""
    return _dequantize(x, group_size, variance=False)


def quantize_variance(x, group_size: int = 32) -> QuantizedArray:
    """uint8 codes of sqrt(x) + fp16 group max (flashoptim_jax/quantization.py:59-68)."""
    return _quantize(x, group_size, variance=True)


def dequantize_variance(x: QuantizedArray, group_size: int = 32) -> torch.Tensor:
    """(code/255 * scale)^2 (flashoptim_jax/quantization.py:71-77)."""
    return _dequantize(x, group_size, variance=True)
