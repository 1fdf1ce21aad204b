"""A NumPy interpreter for the subset of Pallas the reference's four kernels use.

`pallas_call(kernel, out_shape=..., grid=(n,), input_output_aliases=...)` returns a callable that
runs `kernel(*input_refs, *output_refs)` once per program id, eagerly, on NumPy buffers.  An output
that aliases an input starts as a copy of it.  Every program reads its inputs from a snapshot
taken before the first program runs, which is what a GPU launch over disjoint blocks observes.
This executes the kernel text under strict IEEE fp32 (no FMA contraction, true division); what
Triton's code generator would do to that text on a GPU is not modelled.
"""
from __future__ import annotations

import numpy as _np

no_block_spec = None
_program_ids = [0]


def program_id(axis: int) -> int:
    return _program_ids[axis]


class _At:
    def __init__(self, ref):
        self._ref = ref

    def __getitem__(self, idx):
        return _View(self._ref, idx)


class _View:
    def __init__(self, ref, idx):
        self.ref = ref
        self.idx = idx


class Ref:
    """A kernel operand: `shape`, `dtype`, `.at[offsets]`."""

    def __init__(self, data):
        self.data = data

    @property
    def shape(self):
        return self.data.shape

    @property
    def dtype(self):
        return self.data.dtype

    @property
    def at(self):
        return _At(self)


def pallas_call(kernel, out_shape, grid, in_specs=None, out_specs=None, compiler_params=None,
                debug=False, name=None, input_output_aliases=None, interpret=False):
    aliases = dict(input_output_aliases or {})
    single = not isinstance(out_shape, (list, tuple))
    shapes = [out_shape] if single else list(out_shape)

    def run(*operands):
        ins = [_np.array(op, copy=True) for op in operands]
        outs = [None] * len(shapes)
        for i_in, i_out in aliases.items():
            want = shapes[i_out]
            src = ins[i_in]
            if tuple(src.shape) != tuple(want.shape) or src.dtype != _np.dtype(want.dtype):
                raise ValueError(f"alias {i_in}->{i_out}: operand {src.shape} {src.dtype} "
                                 f"does not match output {want.shape} {want.dtype}")
            outs[i_out] = src.copy()
        for j, s in enumerate(shapes):
            if outs[j] is None:
                outs[j] = _np.zeros(s.shape, dtype=s.dtype)
        in_refs = [Ref(a) for a in ins]
        out_refs = [Ref(a) for a in outs]
        (n,) = grid
        for pid in range(n):
            _program_ids[0] = pid
            kernel(*in_refs, *out_refs)
        _program_ids[0] = 0
        return outs[0] if single else outs

    return run


from . import triton  # noqa: E402,F401
