"""A leaf longer than 2^31 elements: fo_step cuts it into pieces of 2^31 (the 32-group kernels
use 32-bit element offsets).  The one-call result must equal two calls on hand-made views that
are each short enough to go in uncut, and the region around the cut must equal the oracle."""

import pytest

from oracle import c_oracle as C
from oracle import flashoptim_oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

CUT = 1 << 31
N = CUT + 3 * 2048 + 37  # two pieces; the second ends in a ragged chunk


def _filled(n, dtype, seed, scale):
    """n pseudo-random values, generated in slabs so that no fp32 temporary of the full length exists."""
    import torch

    out = torch.empty(n, dtype=dtype, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(seed)
    slab = 1 << 28
    for lo in range(0, n, slab):
        m = min(slab, n - lo)
        out[lo:lo + m] = (torch.randn(m, device="cuda", generator=gen) * scale).to(dtype)
    return out


def _state(n, param):
    import torch

    G = (n + 31) // 32
    return H.LeafArrays(param, torch.zeros(n, dtype=torch.int16, device="cuda"),
                        torch.zeros(n, dtype=torch.int8, device="cuda"), torch.zeros(G, dtype=torch.float16, device="cuda"),
                        torch.zeros(n, dtype=torch.uint8, device="cuda"), torch.zeros(G, dtype=torch.float16, device="cuda"))


def _view(leaf, lo, hi):
    g0, g1 = lo // 32, (hi + 31) // 32
    return H.LeafArrays(leaf.param[lo:hi], leaf.ecc[lo:hi], leaf.mu[lo:hi], leaf.mu_scales[g0:g1], leaf.nu[lo:hi], leaf.nu_scales[g0:g1])


def test_leaf_over_2_31_elements_equals_two_hand_cut_calls():
    import torch

    free, _ = torch.cuda.mem_get_info()
    if free < 70 * (1 << 30):
        pytest.skip("needs about 60 GB of device memory")
    grad = _filled(N, torch.bfloat16, 1, 1e-3)
    whole = _state(N, _filled(N, torch.bfloat16, 2, 0.02))
    parts = _state(N, whole.param.clone())
    for t in range(1, 3):
        hp = H.hyper_tuple(C.ADAM, O.FUSED, t, lr=1e-3, wd=1e-2)
        H.abi_step(C.ADAM, [grad], [whole], C.STATE_QUANT, 32, [hp], [0], 1, 1, 16)
        H.abi_step(C.ADAM, [grad[:CUT], grad[CUT:]], [_view(parts, 0, CUT), _view(parts, CUT, N)], C.STATE_QUANT, 32, [hp], [0, 0], 1, 1, 16)
    torch.cuda.synchronize()
    for f in whole.fields():
        assert torch.equal(getattr(whole, f), getattr(parts, f)), f
    # the second piece really was updated, up to its last element
    assert int(whole.mu[CUT:].ne(0).sum()) > (N - CUT) // 2 and int(whole.nu[-37:].ne(0).sum()) > 0

    # oracle on a window across the cut (whole groups on both sides), from the same start
    lo, hi = CUT - 4096, CUT + 4096
    p0 = _filled(N, torch.bfloat16, 2, 0.02)[lo:hi]
    ref = H.fresh_leaf(H.to_numpy(p0), C.ADAM, C.STATE_QUANT, 16)
    g = H.to_numpy(grad[lo:hi])
    for t in range(1, 3):
        H.oracle_step(C.ADAM, g, ref, C.STATE_QUANT, 32, H.hyper_tuple(C.ADAM, O.FUSED, t, lr=1e-3, wd=1e-2))
    H.assert_leaf_equal(_view(whole, lo, hi).to_host(), ref, "window across the cut")
