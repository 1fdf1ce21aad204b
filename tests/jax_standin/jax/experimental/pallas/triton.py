"""`plgpu.load` / `plgpu.store` with masks, on the NumPy refs of the interpreter."""
from __future__ import annotations

import numpy as _np

from . import Ref, _View


class CompilerParams:
    def __init__(self, **kwargs):
        self.kwargs = kwargs


def load(src, mask=None, other=None):
    if isinstance(src, Ref):
        return src.data[()] if src.data.ndim == 0 else src.data.copy()
    assert isinstance(src, _View)
    data, idx = src.ref.data, _np.asarray(src.idx)
    if mask is None:
        return data[idx]
    safe = _np.where(mask, idx, 0)
    got = data[safe] if data.size else _np.zeros(idx.shape, dtype=data.dtype)
    fill = _np.asarray(0 if other is None else other).astype(data.dtype)
    return _np.where(mask, got, fill)


def store(dst, value, mask=None):
    if isinstance(dst, Ref):
        dst.data[...] = value
        return
    assert isinstance(dst, _View)
    data, idx = dst.ref.data, _np.asarray(dst.idx)
    value = _np.asarray(value)
    if value.dtype != data.dtype:
        raise TypeError(f"store of {value.dtype} into a {data.dtype} ref")
    if mask is None:
        data[idx] = value
    else:
        data[idx[mask]] = value[mask]
