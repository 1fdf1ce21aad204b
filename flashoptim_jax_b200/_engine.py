"""The multi-tensor step: from pytrees to fo_step() calls.

The reference loops over leaves in Python and issues one device call per leaf
(flashoptim_jax/adamw.py:522-540, lion.py:168-188, sgd.py:193-217).  Here the loop only
fills descriptor tables; leaves that share the kernel's compile-time switches (param
dtype, grad dtype, ECC width, state kind, group size) form a bucket and each bucket is one
fo_step() call that covers all its leaves in a single launch.
"""

from __future__ import annotations

import contextlib
import ctypes
import threading
from typing import Any, Dict, List, NamedTuple, Optional, Tuple

import numpy as np
import torch

from . import _lib
from . import tree as pytree
from ._dev import DTYPE_CODE, ECC_BITS_OF, as_tensor, require_cuda, stream_ptr
from .quantization import QuantizedArray
from .utils import (
    _group_config_for_path,
    _is_quantized_leaf,
    _tree_leaves_with_paths,
    _use_ecc_leaf,
    _validate_fused_group_size,
    _validate_master_weight_bits,
    _validate_meaningful_master_weight_bits,
    _validate_param_dtypes,
    no_ecc_leaf,
    no_state_leaf,
)

LEAF_DTYPE = np.dtype(
    [("grad", "<u8"), ("param", "<u8"), ("ecc", "<u8"), ("mu", "<u8"), ("mu_scales", "<u8"), ("nu", "<u8"),
     ("nu_scales", "<u8"), ("n", "<u8"), ("hyper", "<u4"), ("reserved", "<u4")]
)
HYPER_DTYPE = np.dtype(
    [("lr", "<f4"), ("wd", "<f4"), ("b1", "<f4"), ("b2", "<f4"), ("one_minus_b1", "<f4"), ("one_minus_b2", "<f4"),
     ("eps", "<f4"), ("bc1", "<f4"), ("bc2", "<f4"), ("flags", "<u4"), ("dev_scalars", "<u8")]
)
assert LEAF_DTYPE.itemsize == ctypes.sizeof(_lib.FoLeaf) and HYPER_DTYPE.itemsize == ctypes.sizeof(_lib.FoHyper)

F32 = np.float32


def one_minus(beta: float, fused: bool) -> np.float32:
    """(1 - beta): in fp32 as the fused kernel text does (adamw.py:99-100), or in Python
    floats rounded once as the jnp text does (adamw.py:394-395)."""
    if fused:
        return F32(F32(1.0) - F32(beta))
    return F32(1.0 - float(beta))


def bias_correction(beta: float, count: int) -> np.float32:
    """1 - f32(beta) ** f32(count) (adamw.py:527-528); the power is taken in float64 and
    rounded once to fp32."""
    return F32(F32(1.0) - F32(float(F32(beta)) ** float(count)))


class LeafWork(NamedTuple):
    """Device buffers of one leaf for one step (updated in place) plus its hyper-parameters."""

    bucket: Tuple[Any, ...]  # (device index, param dtype code, grad dtype code, ecc bits, state kind, group size)
    grad: torch.Tensor
    param: torch.Tensor
    ecc: Optional[torch.Tensor]
    mu: Optional[torch.Tensor]
    mu_scales: Optional[torch.Tensor]
    nu: Optional[torch.Tensor]
    nu_scales: Optional[torch.Tensor]
    hyper: Tuple[Any, ...]  # (lr, wd, b1, b2, omb1, omb2, eps, bc1, bc2, flags)


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


# ---- global-norm clipping folded into the step ---------------------------------------------------

_clip = threading.local()


@contextlib.contextmanager
def grad_clip(sq_norm: torch.Tensor, max_norm: float):
    """While active, every launch rescales its gradients as optax.clip_by_global_norm does
    (examples/train_gpt2_pretrain.py:56-70): `sq_norm` is a one-element float64 device tensor with the
    sum of squares of all gradients of the step (see sq_norm_of)."""
    if sq_norm.dtype != torch.float64 or sq_norm.numel() != 1 or not sq_norm.is_cuda:
        raise ValueError("sq_norm must be a one-element float64 CUDA tensor")
    previous = getattr(_clip, "value", None)
    _clip.value = (sq_norm, float(max_norm))
    try:
        yield
    finally:
        _clip.value = previous


_workspaces: Dict[int, torch.Tensor] = {}


def sq_norm_of(tensors: List[torch.Tensor], out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """Sum of squares of the given CUDA tensors (fp32 / bf16 / fp16, one device) into a one-element
    float64 tensor, on the current stream, without a host round trip (fo_sq_norm, one call per dtype)."""
    tensors = [t for t in tensors if t.numel() > 0]
    if not tensors and out is None:
        raise ValueError("sq_norm_of needs a tensor or an output to tell the device")
    device = tensors[0].device if tensors else out.device
    if out is None:
        out = torch.zeros(1, dtype=torch.float64, device=device)
    lib = _lib.lib()
    ws = _workspaces.get(device.index)
    if ws is None:
        ws = _workspaces[device.index] = torch.empty(_lib.FO_SQ_NORM_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
    by_dtype: Dict[torch.dtype, List[torch.Tensor]] = {}
    for t in tensors:
        if t.dtype not in DTYPE_CODE:
            raise ValueError(f"sq_norm_of: unsupported dtype {t.dtype}")
        if t.device != device:
            raise ValueError("sq_norm_of: tensors on several devices")
        by_dtype.setdefault(t.dtype, []).append(t.contiguous())
    first = True
    with torch.cuda.device(device):
        for dtype, ts in by_dtype.items() or [(torch.float32, [])]:
            table = (_lib.FoArray * max(1, len(ts)))()
            for i, t in enumerate(ts):
                table[i].data, table[i].n = t.data_ptr(), t.numel()
            _lib.check(lib.fo_sq_norm(table, len(ts), DTYPE_CODE[dtype], int(accumulate or not first), out.data_ptr(),
                                      ws.data_ptr(), stream_ptr(device)))
            first = False
    return out


# ---- per-step scalars on the device (graph-capturable steps) ---------------------------------------


def mean_sq_norm(grad_slice: torch.Tensor, mean_out: torch.Tensor, peer_grad_offsets: List[int], out: torch.Tensor,
                 accumulate: bool) -> torch.Tensor:
    """mean_out <- this rank's slice of the gradient averaged over the ranks (own value, then the same elements
    `peer_grad_offsets` bytes away in the peers' buffers), and the sum of its squares into `out` (a one-element
    float64 tensor), in one sweep over NVLink (fo_mean_sq_norm)."""
    device = grad_slice.device
    if grad_slice.numel() != mean_out.numel() or grad_slice.dtype != mean_out.dtype:
        raise ValueError("mean_sq_norm: slice and output differ")
    ws = _workspaces.get(device.index)
    if ws is None:
        ws = _workspaces[device.index] = torch.empty(_lib.FO_SQ_NORM_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
    peers = np.asarray(peer_grad_offsets, dtype=np.int64)
    with torch.cuda.device(device):
        _lib.check(_lib.lib().fo_mean_sq_norm(grad_slice.data_ptr(), mean_out.data_ptr(), grad_slice.numel(), DTYPE_CODE[grad_slice.dtype],
                                             peers.ctypes.data if len(peers) else None, len(peers), int(accumulate), out.data_ptr(),
                                             ws.data_ptr(), stream_ptr(device)))
    return out


def step_scalars(count: torch.Tensor, learning_rate: Any, b1: float, b2: float, write_count: bool) -> torch.Tensor:
    """float32[3] = {lr, 1 - b1^(count+1), 1 - b2^(count+1)} formed on the device from the device counter
    (adamw.py:510, 526-528); `learning_rate` is a number or a 0-d float32 CUDA tensor.  With `write_count`
    the counter is advanced in place.  The result is what FoHyper.dev_scalars points to."""
    if not (count.is_cuda and count.dtype == torch.int32 and count.numel() == 1):
        raise ValueError("a capturable step keeps `count` as a 0-d int32 CUDA tensor")
    from .schedules import DeviceSchedule

    if isinstance(learning_rate, DeviceSchedule):  # evaluated on the device at the zero-based count (adamw.py:526)
        out = torch.empty(3, dtype=torch.float32, device=count.device)
        params = (ctypes.c_float * 3)(*learning_rate.device_params())
        with torch.cuda.device(count.device):
            _lib.check(_lib.lib().fo_step_scalars_schedule(count.data_ptr(), learning_rate.kind, params, float(b1), float(b2),
                                                           out.data_ptr(), count.data_ptr() if write_count else 0,
                                                           stream_ptr(count.device)))
        return out
    lr_ptr, lr_const = 0, 0.0
    if isinstance(learning_rate, torch.Tensor):
        if not (learning_rate.is_cuda and learning_rate.dtype == torch.float32 and learning_rate.numel() == 1):
            raise ValueError("a tensor learning rate must be a 0-d float32 CUDA tensor")
        lr_ptr = learning_rate.data_ptr()
    elif callable(learning_rate):
        raise ValueError("a capturable step cannot call a schedule on the host: pass a schedule from "
                         "flashoptim_jax_b200.schedules, or a CUDA tensor that you update yourself")
    else:
        lr_const = float(learning_rate)
    out = torch.empty(3, dtype=torch.float32, device=count.device)
    with torch.cuda.device(count.device):
        _lib.check(_lib.lib().fo_step_scalars(count.data_ptr(), lr_ptr, lr_const, float(b1), float(b2), out.data_ptr(),
                                              count.data_ptr() if write_count else 0, stream_ptr(count.device)))
    return out


def device_step_scalars(count: Any, leaves: List[torch.Tensor], configs: List[Dict[str, Any]]):
    """For a capturable step: advance the device counter and form each hyper-parameter group's scalars on the
    device.  Returns (counter tensor, per-leaf pointer to its group's float32[3], tensors to keep alive until the
    launch has been issued)."""
    count = as_tensor(count, dtype=torch.int32)
    if not count.is_cuda:
        count = count.to(leaves[0].device)  # first step after an init on the host
    keys = [tuple(sorted(((k, id(v) if isinstance(v, torch.Tensor) else v) for k, v in c.items()), key=lambda kv: kv[0]))
            for c in configs]
    distinct = list(dict.fromkeys(keys))
    scalars = {}
    for i, key in enumerate(distinct):
        c = configs[keys.index(key)]
        scalars[key] = step_scalars(count, c["learning_rate"], c.get("b1", 0.0), c.get("b2", 0.0), write_count=i == len(distinct) - 1)
    return count, [scalars[key].data_ptr() for key in keys], list(scalars.values())


# ---- observing launches (benchmarks time every fo_step call with CUDA events) ----------------------

_observer = None


def set_launch_observer(fn) -> None:
    """`fn(bucket_key, n_params)` must return a context manager; every fo_step call of this module then
    runs inside it.  None switches observation off."""
    global _observer
    _observer = fn


def _observed(key, n_params):
    return contextlib.nullcontext() if _observer is None else _observer(key, n_params)


class PreparedLaunch:
    """The fo_step calls of a fixed list of leaves, with their descriptor tables built once.

    The buffers of a sharded optimizer never move, so only the hyper-parameter values change from step
    to step: `run` writes them into the prepared tables (one entry per distinct hyper-parameter group)
    and issues the calls.  The host cost of a step is then proportional to the number of calls and
    groups, not to the number of leaves (the per-leaf Python loop of the reference,
    flashoptim_jax/adamw.py:522-540, runs once)."""

    def __init__(self, opt: int, work: List[LeafWork], group_ids: List[int], peer_param_offsets: Optional[List[int]] = None,
                 peer_grad_offsets: Optional[List[int]] = None, mc_param_offset: int = 0, mc_grad_offset: int = 0):
        self.peers = np.asarray(peer_param_offsets or [], dtype=np.int64)
        self.grad_peers = np.asarray(peer_grad_offsets or [], dtype=np.int64)
        if len(self.peers) and len(self.grad_peers) and len(self.peers) != len(self.grad_peers):
            raise ValueError("peer_param_offsets and peer_grad_offsets must name the same peers")
        n_peers = max(len(self.peers), len(self.grad_peers))
        buckets: Dict[Tuple[Any, ...], List[Tuple[LeafWork, int]]] = {}
        for i, (w, gid) in enumerate(zip(work, group_ids)):
            buckets.setdefault(w.bucket, []).append((w, gid, i))
        self.calls: List[Dict[str, Any]] = []
        for key, items in buckets.items():
            dev_index, pdt, gdt, ecc_bits, state, group_size = key
            start = 0
            while start < len(items):
                slots: Dict[int, int] = {}
                end = start
                while end < len(items) and (items[end][1] in slots or len(slots) < _lib.FO_MAX_HYPERS):  # noqa: E501
                    slots.setdefault(items[end][1], len(slots))
                    end += 1
                part = items[start:end]
                ws = [w for w, _, _ in part]
                leaves = np.zeros(len(part), dtype=LEAF_DTYPE)
                leaves["grad"] = [w.grad.data_ptr() for w in ws]
                leaves["param"] = [w.param.data_ptr() for w in ws]
                for name in ("ecc", "mu", "mu_scales", "nu", "nu_scales"):
                    leaves[name] = [_ptr(getattr(w, name)) for w in ws]
                leaves["n"] = [w.param.numel() for w in ws]
                leaves["hyper"] = [slots[gid] for _, gid, _ in part]
                hypers = np.zeros(len(slots), dtype=HYPER_DTYPE)
                desc = _lib.FoStepDesc(
                    struct_size=ctypes.sizeof(_lib.FoStepDesc), opt=opt, param_dtype=pdt, grad_dtype=gdt, ecc_bits=ecc_bits,
                    state=state, group_size=group_size, n_leaves=len(part), n_hypers=len(slots),
                    leaves=leaves.ctypes.data, hypers=hypers.ctypes.data, n_peers=n_peers,
                    peer_param_offsets=self.peers.ctypes.data if len(self.peers) else None,
                    peer_grad_offsets=self.grad_peers.ctypes.data if len(self.grad_peers) else None,
                )
                desc.mc_param_offset, desc.mc_grad_offset = int(mc_param_offset), int(mc_grad_offset)
                self.calls.append({"key": key, "desc": desc, "leaves": leaves, "hypers": hypers, "slots": list(slots.items()),
                                   "device": torch.device("cuda", dev_index), "n_params": int(leaves["n"].sum()),
                                   "index": np.asarray([i for _, _, i in part], dtype=np.int64),
                                   "keep": ws})  # the tensors stay alive as long as their addresses are in the tables
                start = end

    def set_grads(self, grad_ptrs: np.ndarray, keep: List[torch.Tensor]) -> None:
        """New gradient buffers for the same leaves (addresses in the order of the work list this was built from)."""
        for call in self.calls:
            call["leaves"]["grad"] = grad_ptrs[call["index"]]
        self._grads_alive = keep

    def run(self, hyper_of_group: Dict[int, Tuple[Any, ...]]) -> int:
        lib = _lib.lib()
        clip = getattr(_clip, "value", None)
        for call in self.calls:
            hypers = call["hypers"]
            for gid, slot in call["slots"]:
                hp = hyper_of_group[gid]
                hypers[slot] = hp if len(hp) == len(HYPER_DTYPE.names) else hp + (0,)
            desc = call["desc"]
            if clip is not None:
                desc.grad_sq_norm, desc.max_grad_norm = clip[0].data_ptr(), clip[1]
            else:
                desc.grad_sq_norm, desc.max_grad_norm = None, 0.0
            device = call["device"]
            if _observer is None and torch.cuda.current_device() == device.index:
                # the common case, without the two context managers (a few microseconds each on a launch-bound step)
                _lib.check(lib.fo_step(ctypes.byref(desc), stream_ptr(device)))
            else:
                with torch.cuda.device(device), _observed(call["key"], call["n_params"]):
                    _lib.check(lib.fo_step(ctypes.byref(desc), stream_ptr(device)))
        return len(self.calls)


class DonatedStepCache:
    """The functional tx.step for callers that donate their buffers and hand each step's outputs to the
    next: the parameter and state tensors are then the same objects step after step, and only the gradients
    and the scalars change.  After one step through the general path this remembers the prepared launch of
    that step, keyed on the identity and the addresses of every tensor of the returned trees; a later call
    whose trees consist of exactly those tensors skips the per-leaf host work (path normalisation, param-group
    matching, validation, table building: about 12 us per leaf) and replays the launch with new gradient
    addresses and hyper-parameter values.  Anything else (other tensors, other gradient dtypes, non-contiguous
    gradients) falls back to the general path, which then re-primes the cache.  A replayed step keeps the
    param-group membership of the remembered call: selectors are functions of the path and of the leaf's
    shape / dtype in every use the reference shows, and a selector that reads a leaf's *values* is not
    re-evaluated while the same tensors come back."""

    def __init__(self):
        self.entry = None

    @staticmethod
    def _tensors(params: Any, state_trees: List[Any]) -> Tuple[List[torch.Tensor], List[Any]]:
        """Every tensor of the trees in flattening order, and the trees' structural signature."""
        out, sig = pytree.tree_leaves_and_signature(params)
        sig.append(len(out))
        for tree in state_trees:
            leaves, s = pytree.tree_leaves_and_signature(tree, is_leaf=_is_quantized_leaf)
            sig.append(s)
            for leaf in leaves:
                if isinstance(leaf, QuantizedArray):
                    out.append(leaf.values)
                    out.append(leaf.scales)
                else:
                    out.append(leaf)
        return out, sig

    def remember(self, opt: int, work: List[LeafWork], configs: List[Dict[str, Any]], params_out: Any, state_trees_out: List[Any]) -> None:
        groups: List[Dict[str, Any]] = []
        gids = []
        for c in configs:
            for i, g in enumerate(groups):
                if g is c or g == c:
                    gids.append(i)
                    break
            else:
                groups.append(c)
                gids.append(len(groups) - 1)
        tensors, sig = self._tensors(params_out, state_trees_out)
        if not all(isinstance(t, torch.Tensor) for t in tensors):
            self.entry = None
            return
        self.entry = {
            "plan": PreparedLaunch(opt, work, gids), "groups": groups, "ids": [id(t) for t in tensors],
            "sig": sig,
            "ptrs": [t.data_ptr() for t in tensors], "alive": tensors, "params": params_out, "state": state_trees_out,
            "grad_spec": [(w.grad.dtype, w.grad.shape, w.grad.device) for w in work],
        }

    def replay(self, params: Any, state_trees: List[Any], grads: Any, hyper_of_group) -> Optional[Tuple[Any, List[Any]]]:
        """Runs the remembered launch if (params, state) are the remembered tensors; returns (params, state trees)
        or None.  `hyper_of_group(config)` gives the hyper-parameter tuple of a param group for this step."""
        e = self.entry
        if e is None:
            return None
        tensors, sig = self._tensors(params, state_trees)
        if len(tensors) != len(e["ids"]) or sig != e["sig"]:
            return None
        try:  # the same objects at the same addresses (C-level loops: this check runs on every step)
            if list(map(id, tensors)) != e["ids"] or list(map(torch.Tensor.data_ptr, tensors)) != e["ptrs"]:
                return None
        except TypeError:  # something that is not a tensor
            return None
        g_leaves = pytree.tree_leaves(grads)
        spec = e["grad_spec"]
        if len(g_leaves) != len(spec):
            return None
        ptrs = np.empty(len(spec), dtype=np.uint64)
        for k, (g, (dtype, shape, device)) in enumerate(zip(g_leaves, spec)):
            if not isinstance(g, torch.Tensor) or g.dtype != dtype or g.shape != shape or g.device != device or not g.is_contiguous():
                return None
            ptrs[k] = g.data_ptr()
        plan = e["plan"]
        plan.set_grads(ptrs, g_leaves)
        plan.run({gid: hyper_of_group(config) for gid, config in enumerate(e["groups"])})
        return e["params"], e["state"]


def launch(opt: int, work: List[LeafWork], peer_param_offsets: Optional[List[int]] = None,
           peer_grad_offsets: Optional[List[int]] = None, mc_param_offset: int = 0, mc_grad_offset: int = 0) -> int:
    """Issue one fo_step per bucket (per <=16 hyper sets); returns the number of calls.

    peer_param_offsets: byte distances from every param address to the same element of each peer
    GPU's replica; when given, the kernel also stores the updated parameters there.
    peer_grad_offsets: byte distances from every grad address to the same element of each peer GPU's
    gradient buffer; when given, the kernel averages the gradients over the ranks as it reads them.
    mc_param_offset / mc_grad_offset: byte distances to the multicast mappings of the same buffers; when
    non-zero the two exchanges go through the NVLink switch (one multicast store, one multicast load-reduce)."""
    flush_copies()  # the buffers of an undonated step get their contents now
    peers = np.asarray(peer_param_offsets or [], dtype=np.int64)
    grad_peers = np.asarray(peer_grad_offsets or [], dtype=np.int64)
    if len(peers) and len(grad_peers) and len(peers) != len(grad_peers):
        raise ValueError("peer_param_offsets and peer_grad_offsets must name the same peers")
    n_peers = max(len(peers), len(grad_peers))
    buckets: Dict[Tuple[Any, ...], List[LeafWork]] = {}
    for w in work:
        buckets.setdefault(w.bucket, []).append(w)
    calls = 0
    lib = _lib.lib()
    for key, items in buckets.items():
        dev_index, pdt, gdt, ecc_bits, state, group_size = key
        hyper_index: Dict[Tuple[Any, ...], int] = {}
        pending: List[Tuple[LeafWork, int]] = []

        def flush():
            nonlocal calls, hyper_index, pending
            if not pending:
                return
            leaves = np.zeros(len(pending), dtype=LEAF_DTYPE)
            ws = [w for w, _ in pending]
            leaves["grad"] = [w.grad.data_ptr() for w in ws]
            leaves["param"] = [w.param.data_ptr() for w in ws]
            leaves["ecc"] = [_ptr(w.ecc) for w in ws]
            leaves["mu"] = [_ptr(w.mu) for w in ws]
            leaves["mu_scales"] = [_ptr(w.mu_scales) for w in ws]
            leaves["nu"] = [_ptr(w.nu) for w in ws]
            leaves["nu_scales"] = [_ptr(w.nu_scales) for w in ws]
            leaves["n"] = [w.param.numel() for w in ws]
            leaves["hyper"] = [h for _, h in pending]
            hypers = np.zeros(len(hyper_index), dtype=HYPER_DTYPE)
            for hp, idx in hyper_index.items():
                hypers[idx] = hp if len(hp) == len(HYPER_DTYPE.names) else hp + (0,)
            desc = _lib.FoStepDesc(
                struct_size=ctypes.sizeof(_lib.FoStepDesc), opt=opt, param_dtype=pdt, grad_dtype=gdt, ecc_bits=ecc_bits,
                state=state, group_size=group_size, n_leaves=len(pending), n_hypers=len(hyper_index),
                leaves=leaves.ctypes.data, hypers=hypers.ctypes.data,
                n_peers=n_peers, peer_param_offsets=peers.ctypes.data if len(peers) else None,
                peer_grad_offsets=grad_peers.ctypes.data if len(grad_peers) else None,
            )
            desc.mc_param_offset, desc.mc_grad_offset = int(mc_param_offset), int(mc_grad_offset)
            clip = getattr(_clip, "value", None)
            if clip is not None:
                desc.grad_sq_norm, desc.max_grad_norm = clip[0].data_ptr(), clip[1]
            device = torch.device("cuda", dev_index)
            with torch.cuda.device(device), _observed(key, int(leaves["n"].sum())):
                _lib.check(lib.fo_step(ctypes.byref(desc), stream_ptr(device)))
            calls += 1
            hyper_index = {}
            pending = []

        for w in items:
            if w.hyper not in hyper_index and len(hyper_index) == _lib.FO_MAX_HYPERS:
                flush()
            idx = hyper_index.setdefault(w.hyper, len(hyper_index))
            pending.append((w, idx))
        flush()
    return calls


# ---- state initialisation (flashoptim_jax/utils.py:287-306, 337-358) -------------------------


def init_moment(param: torch.Tensor, group_size: int, quantize: bool, code_dtype: torch.dtype):
    """Zero moment: quantized zeros are code 0 / scale 0, which is what quantizing zeros gives."""
    if quantize:
        n = param.numel()
        return QuantizedArray(
            values=torch.zeros(param.shape, dtype=code_dtype, device=param.device),
            scales=torch.zeros(((n + group_size - 1) // group_size,), dtype=torch.float16, device=param.device),
        )
    return torch.zeros(param.shape, dtype=torch.float32, device=param.device)


def init_ecc(param: torch.Tensor, master_weight_bits: Optional[int]) -> torch.Tensor:
    if _use_ecc_leaf(param, master_weight_bits):
        return torch.zeros(param.shape, dtype=torch.int8 if master_weight_bits == 24 else torch.int16, device=param.device)
    return no_ecc_leaf(param.device)


def init_common(params: Any, defaults, param_groups, name: str, per_leaf_check=None):
    """Validation shared by the three init functions; yields (path, leaf tensor, config)."""
    _validate_param_dtypes(params, defaults, param_groups, name)
    _validate_meaningful_master_weight_bits(params, defaults, param_groups, name)
    path_leaves, treedef = _tree_leaves_with_paths(params)
    out = []
    for path, leaf in path_leaves:
        config = _group_config_for_path(path, leaf, defaults, param_groups)
        _validate_master_weight_bits(config["master_weight_bits"])
        _validate_fused_group_size(config["group_size"], quantize=config["quantize"], fused=config["fused"])
        if per_leaf_check is not None:
            per_leaf_check(config)
        out.append((path, as_tensor(leaf), config))
    return out, treedef


# ---- one step ----------------------------------------------------------------------------------


def _prep_grad(grad: Any, param: torch.Tensor) -> torch.Tensor:
    g = as_tensor(grad)
    if g.device != param.device:
        g = g.to(param.device)
    if g.dtype not in DTYPE_CODE:
        g = g.to(torch.float32)  # the reference upcasts every grad to fp32 first (adamw.py:531)
    if g.shape != param.shape:
        raise ValueError(f"gradient shape {tuple(g.shape)} does not match parameter shape {tuple(param.shape)}")
    return g.contiguous()


_copies = threading.local()  # (destination, source) pairs of the step being assembled on this thread


def _own(t: torch.Tensor, donate: bool) -> torch.Tensor:
    """The buffer the kernel may overwrite: the caller's own when donated, else a copy.  The copies of one
    step are collected and made together right before its launches (flush_copies): one multi-tensor copy
    per dtype instead of four to six small launches per leaf."""
    if donate and t.is_contiguous():
        return t
    dst = torch.empty_like(t, memory_format=torch.contiguous_format)
    pending = getattr(_copies, "pairs", None)
    if pending is None:
        pending = _copies.pairs = []
    pending.append((dst, t))
    return dst


def flush_copies() -> None:
    pending = getattr(_copies, "pairs", None)
    if pending:
        _copies.pairs = []
        groups: Dict[Tuple[Any, Any, Any], Tuple[List[torch.Tensor], List[torch.Tensor]]] = {}
        for d, s in pending:  # the multi-tensor kernel takes lists of one dtype on one device
            dst, src = groups.setdefault((d.dtype, s.dtype, d.device), ([], []))
            dst.append(d)
            src.append(s)
        for dst, src in groups.values():
            torch._foreach_copy_(dst, src)


def flatten_step_inputs(name: str, params, grads, state_trees: List[Any]):
    """Flatten params / grads / state trees and check that they line up (adamw.py:511-519)."""
    _copies.pairs = []  # a step that failed half-way leaves nothing behind
    param_pl, treedef = _tree_leaves_with_paths(params)
    # the usual case, all trees alike, is settled by the cheap structural signatures; anything else goes
    # through the structure objects below, which tell the cases apart for the error messages
    _, want = pytree.tree_leaves_and_signature(params)
    grad_leaves, sig = pytree.tree_leaves_and_signature(grads)
    alike = sig == want and len(grad_leaves) == len(param_pl)
    flat_states = []
    for st in state_trees:
        leaves, sig = pytree.tree_leaves_and_signature(st, is_leaf=_is_quantized_leaf)
        alike = alike and sig == want and len(leaves) == len(param_pl)
        flat_states.append(leaves)
    if alike:
        return param_pl, grad_leaves, flat_states, treedef
    grad_pl, grad_def = _tree_leaves_with_paths(grads)
    for st in state_trees:
        if pytree.tree_structure(st, is_leaf=_is_quantized_leaf) != treedef:
            raise ValueError(f"{name} state trees must match parameter structure")
    if grad_def != treedef:
        raise ValueError(f"{name} state trees must match parameter structure")
    if [p for p, _ in param_pl] != [p for p, _ in grad_pl]:
        raise ValueError(f"{name} gradients must match parameter paths")
    return param_pl, [g for _, g in grad_pl], flat_states, treedef


def make_work(
    param: torch.Tensor,
    grad: torch.Tensor,
    ecc_leaf: Any,
    mu_leaf: Any,
    nu_leaf: Any,
    config: Dict[str, Any],
    hyper: Tuple[Any, ...],
    donate: bool,
    has_nu: bool,
    use_momentum: bool = True,
):
    """Resolve one leaf into kernel buffers.  Returns (LeafWork, new param, new ecc, new mu, new nu)."""
    require_cuda(param, "parameter")
    g = _prep_grad(grad, param)
    p = _own(param, donate)
    use_ecc = _use_ecc_leaf(param, config["master_weight_bits"])
    ecc_out: Any
    ecc_buf = None
    ecc_bits = 0
    if use_ecc:
        want = torch.int8 if config["master_weight_bits"] == 24 else torch.int16
        e = as_tensor(ecc_leaf)
        if e.dim() == 0 and e.dtype == torch.int32:  # sentinel where a buffer is expected: start from zeros (utils.py:459-461)
            ecc_buf = torch.zeros(param.shape, dtype=want, device=param.device)
        else:
            ecc_buf = _own(e.to(want) if e.dtype != want else e, donate and e.dtype == want)
        ecc_bits = ECC_BITS_OF[want]
        ecc_out = ecc_buf
    else:
        ecc_out = ecc_leaf if isinstance(ecc_leaf, torch.Tensor) and ecc_leaf.dim() == 0 else no_ecc_leaf(param.device)

    group_size = int(config["group_size"])
    mu_buf = mu_sc = nu_buf = nu_sc = None
    mu_out: Any = mu_leaf
    nu_out: Any = nu_leaf
    if not use_momentum:
        state = _lib.FO_STATE_NONE
        mu_out = mu_leaf if isinstance(mu_leaf, torch.Tensor) else no_state_leaf(param.device)
    elif config["quantize"]:
        state = _lib.FO_STATE_QUANT
        if not isinstance(mu_leaf, QuantizedArray):
            raise ValueError("quantize=True expects QuantizedArray moments in the optimizer state")
        mu_buf, mu_sc = _own(mu_leaf.values, donate), _own(mu_leaf.scales, donate)
        mu_out = QuantizedArray(values=mu_buf, scales=mu_sc)
        if has_nu:
            nu_buf, nu_sc = _own(nu_leaf.values, donate), _own(nu_leaf.scales, donate)
            nu_out = QuantizedArray(values=nu_buf, scales=nu_sc)
    else:
        state = _lib.FO_STATE_FULL
        mu_buf = _own(as_tensor(mu_leaf, dtype=torch.float32), donate)
        mu_out = mu_buf
        if has_nu:
            nu_buf = _own(as_tensor(nu_leaf, dtype=torch.float32), donate)
            nu_out = nu_buf
    bucket = (param.device.index if param.device.index is not None else torch.cuda.current_device(),
              DTYPE_CODE[param.dtype], DTYPE_CODE[g.dtype], ecc_bits, state,
              group_size if state == _lib.FO_STATE_QUANT else 32)
    work = LeafWork(bucket, g, p, ecc_buf, mu_buf, mu_sc, nu_buf, nu_sc, hyper)
    return work, p, ecc_out, mu_out, nu_out
