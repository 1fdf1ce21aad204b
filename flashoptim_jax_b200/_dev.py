"""Tensor plumbing between PyTorch and the C ABI: dtype codes, pointers, streams.

PyTorch is used for device memory and streams only; every computation is a call into
libflashoptim_b200.so on the current CUDA stream.
"""

from __future__ import annotations

import torch

from . import _lib

DTYPE_CODE = {torch.float32: _lib.FO_F32, torch.bfloat16: _lib.FO_BF16, torch.float16: _lib.FO_F16}
LOW_PRECISION = (torch.bfloat16, torch.float16)
FUSED_PARAM_DTYPES = (torch.float32, torch.bfloat16, torch.float16)
ECC_BITS_OF = {torch.int8: 8, torch.int16: 16}

_DTYPE_NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16"}


def dtype_name(dt) -> str:
    return _DTYPE_NAME.get(dt, str(dt).replace("torch.", ""))


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{what} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise RuntimeError(
            f"{what} lives on {t.device}; flashoptim_jax_b200 computes on CUDA devices only (there is no CPU path)"
        )


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)  # the handle without a Stream object around it


def stream_ptr(device: torch.device) -> int:
    """Handle of torch's current stream on `device` (what every launch of this package runs on)."""
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


def as_tensor(x, dtype=None, device=None) -> torch.Tensor:
    if isinstance(x, torch.Tensor):
        t = x
        if dtype is not None and t.dtype != dtype:
            t = t.to(dtype)
        if device is not None and t.device != torch.device(device):
            t = t.to(device)
        return t
    return torch.as_tensor(x, dtype=dtype, device=device)
