"""ZeRO-1 sharding of the optimizer step across the GPUs of one node.

The reference replicates optimizer state on every device and all-reduces gradients
(examples/train_gpt2_pretrain.py:412-441).  Here each rank keeps the ECC and the
quantized moments of only its slice of every dtype bucket:

    reduce-scatter(mean) of the gradients  ->  fused step on the local slice
                                           ->  all-gather of the updated parameters

Every quantization group of 32 consecutive elements is an independent unit, so a slice
boundary that falls on a group boundary changes no result: the sharded step is
bit-identical to the single-device step whenever the averaged gradient is.

Layout.  All leaves of one parameter dtype live in one flat buffer, each leaf starting at a
multiple of 32 elements (a group boundary; also 16-byte alignment for the vector path).
The buffer is cut into n_slices slices of world_size pieces, a piece being a multiple of 4096
elements (one kernel chunk): rank r owns piece r of every slice; a leaf that straddles
pieces is cut at group boundaries.  One slice is the unit of the collectives, so that the
step of slice s runs while slice s+1 is still being reduce-scattered and the all-gathers
queue up behind the reduce-scatters on the communication stream.  The parameter and
gradient trees handed back to the caller are views into the flat buffers, so no copy sits
between backward and the collectives.
"""

from __future__ import annotations

import contextlib

from typing import Any, Callable, Dict, List, NamedTuple, Optional, Tuple

import torch
import torch.distributed as dist

from . import _engine as eng
from . import _lib
from . import tree as pytree
from . import utils
from ._dev import DTYPE_CODE, as_tensor
from .adamw import adam_hyper
from .lion import lion_hyper
from .sgd import sgd_hyper

LEAF_ALIGN = 32      # elements: one quantization group
SHARD_ALIGN = 4096   # elements: the largest kernel chunk (512-thread blocks x 8), so that a shard is whole chunks for every slice


class Segment(NamedTuple):
    """The part of one leaf that one rank owns."""

    leaf: int     # index into the flattened parameter list
    lo: int       # first element of the leaf in this segment (multiple of 32)
    hi: int       # one past the last element
    offset: int   # position of `lo` in the rank's shard
    slice: int = 0  # which slice of the bucket the segment lies in


class BucketLayout(NamedTuple):
    dtype: torch.dtype
    leaves: List[int]          # leaf indices in this bucket, in tree order
    starts: List[int]          # start of each leaf in the flat buffer
    sizes: List[int]
    total: int                 # padded length = n_slices * world_size * piece
    shard: int                 # elements one rank owns = n_slices * piece
    segments: List[List[Segment]]  # per rank, ordered by slice
    piece: int = 0             # elements of one rank in one slice
    n_slices: int = 1



def plan_bucket(dtype: torch.dtype, leaf_ids: List[int], sizes: List[int], world_size: int,
                n_slices: Optional[int] = None) -> BucketLayout:
    """Place leaves in a flat buffer and cut it into n_slices x world_size pieces."""
    starts, pos = [], 0
    for n in sizes:
        starts.append(pos)
        pos += -(-n // LEAF_ALIGN) * LEAF_ALIGN
    if n_slices is None:
        # Measured on 2 x B200 (Llama-3-8B pytree): 8 slices with the pipeline 51.9 ms per step, one slice
        # without it 46.2 ms: the persistent step kernel and NCCL's kernels slow each other down more than the
        # overlap gains.  One slice is therefore the default; more can be asked for.
        n_slices = 1
    piece = -(-pos // (world_size * n_slices * SHARD_ALIGN)) * SHARD_ALIGN if pos else SHARD_ALIGN
    slice_len = piece * world_size
    segments: List[List[Segment]] = []
    for r in range(world_size):
        segs = []
        for sl in range(n_slices):
            lo_r = sl * slice_len + r * piece
            hi_r = lo_r + piece
            for leaf, start, n in zip(leaf_ids, starts, sizes):
                lo, hi = max(start, lo_r), min(start + n, hi_r)
                if lo < hi:
                    segs.append(Segment(leaf, lo - start, hi - start, sl * piece + lo - lo_r, sl))
        segments.append(segs)
    return BucketLayout(dtype, list(leaf_ids), starts, list(sizes), slice_len * n_slices, piece * n_slices, segments, piece, n_slices)


def flat_position(layout: BucketLayout, rank: int, offset: int) -> int:
    """Position in the flat buffer of element `offset` of rank `rank`'s shard."""
    sl, within = divmod(offset, layout.piece)
    return (sl * (layout.total // layout.shard) + rank) * layout.piece + within


class ShardState(NamedTuple):
    """Optimizer state of one segment (same tensors as the unsharded state, for [lo, hi) only)."""

    ecc: Optional[torch.Tensor]
    mu: Optional[torch.Tensor]
    mu_scales: Optional[torch.Tensor]
    nu: Optional[torch.Tensor]
    nu_scales: Optional[torch.Tensor]


def _reduce_scatter_mean(out: torch.Tensor, full: torch.Tensor, group, world_size: int) -> None:
    """out <- mean over ranks of this rank's slice of `full` (the reference's pmean, train_gpt2_pretrain.py:429)."""
    if world_size == 1:
        if out.data_ptr() != full.data_ptr():
            out.copy_(full[: out.numel()])
        return
    backend = dist.get_backend(group)
    if backend == "nccl":
        dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.AVG, group=group)
        return
    # backends without a mean / low-precision reduce-scatter (gloo, used by the CPU tests)
    rank = dist.get_rank(group)
    acc = full.to(torch.float32)
    dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=group)
    n = out.numel()
    out.copy_((acc[rank * n:(rank + 1) * n] / world_size).to(out.dtype))


def _all_gather_inplace(full: torch.Tensor, shard: int, group, world_size: int) -> None:
    """Every rank's slice of `full` is sent to all others, in place."""
    if world_size == 1:
        return
    rank = dist.get_rank(group)
    mine = full[rank * shard:(rank + 1) * shard]
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(full, mine, group=group)
    else:
        parts = [torch.empty_like(mine) for _ in range(world_size)]
        dist.all_gather(parts, mine.clone(), group=group)
        for r, part in enumerate(parts):
            full[r * shard:(r + 1) * shard].copy_(part)


StepFn = Callable[..., int]  # (opt, work[, peer_param_offsets]) -> number of fo_step calls


class Zero1Optimizer:
    """flash_adamw / flash_adam / flash_lion / flash_sgd / flash_sgdw with sharded state.

    optimizer   one of "adamw", "adam", "lion", "sgd", "sgdw"
    params      pytree of tensors, identical on every rank; fp32 / bf16 / fp16 leaves
    hparams     the keyword arguments of the matching flash_* factory (param_groups included)
    group       torch.distributed process group (None = default group; no group = one rank)
    step_fn     how a list of LeafWork is executed; the default launches the CUDA kernels
    n_slices    slices per bucket (None: chosen from the bucket size; 1 disables the pipeline)
    fused_allgather
                fold the all-gather into the step kernel: the flat parameter buffers are allocated as
                symmetric (peer-mapped) memory and the kernel stores every updated parameter vector into
                all peers' replicas over NVLink as it produces it; a one-element all-reduce afterwards
                orders the peers' reads.  NCCL / CUDA ranks on one node only.
    fused_reduce_scatter
                fold the reduce-scatter into the step kernel: the flat gradient buffers are symmetric
                memory too, and the kernel reads its slice of every rank's gradients over NVLink and
                averages them (fp32 sum in rank order starting with its own, one rounding to the
                gradient dtype) as it goes; a one-element all-reduce before the launch makes sure that
                every rank's gradients are complete.  Same restrictions.
    use_switch  route the fused collectives through the NVLink switch (the symmetric allocations' multicast
                mappings): parameters leave as one multicast store instead of one store per peer, 16-bit
                gradients arrive as one multicast load-reduce instead of one load per peer, so each
                direction of the links carries about one replica's volume whatever the rank count (a gain
                from four ranks on; with two ranks the switch only adds traffic).  Off by default because
                the switch's bf16 / fp16 addition is not IEEE round-to-nearest (measured: one in five
                two-rank sums differs from the correctly rounded one in the last place), so results are
                no longer bit-identical to the reference arithmetic unless all ranks hold equal gradients.
    max_grad_norm
                clip the (averaged) gradients at this global norm, as optax.clip_by_global_norm in front
                of the optimizer does (examples/train_gpt2_pretrain.py:56-70): every rank sums the squares
                of its reduce-scattered slice on the device, the sums are all-reduced, and the step kernel
                rescales the gradients as it loads them.  Together with fused_reduce_scatter the sweep that
                sums the squares is also the reduce-scatter: it reads the peers' slices over NVLink, leaves the
                averaged slice in local memory for the step and its squares in the sum (fo_mean_sq_norm), so
                the gradients still cross the links once.
    """

    def __init__(self, optimizer: str, params: Any, *, group=None, step_fn: Optional[StepFn] = None,
                 n_slices: Optional[int] = None, fused_allgather: bool = False, fused_reduce_scatter: bool = False,
                 max_grad_norm: Optional[float] = None, use_switch: bool = False, **hparams):
        self.kind = optimizer
        if optimizer not in ("adamw", "adam", "lion", "sgd", "sgdw"):
            raise ValueError(f"unknown optimizer {optimizer!r}")
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized()
        self.world_size = dist.get_world_size(group) if self.distributed else 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        self._step_fn = step_fn or eng.launch
        self.param_groups = hparams.pop("param_groups", None)
        self.defaults = self._defaults(optimizer, hparams)
        self.name = "flash_" + optimizer
        self.opt_code = {"adamw": _lib.FO_OPT_ADAM, "adam": _lib.FO_OPT_ADAM, "lion": _lib.FO_OPT_LION,
                         "sgd": _lib.FO_OPT_SGD, "sgdw": _lib.FO_OPT_SGD}[optimizer]
        self.decoupled = optimizer in ("adamw", "sgdw", "lion")
        self.count = 0

        utils._validate_master_weight_bits(self.defaults["master_weight_bits"])
        utils._validate_fused_group_size(self.defaults["group_size"], quantize=self.defaults["quantize"],
                                         fused=self.defaults["fused"])
        utils._validate_param_dtypes(params, self.defaults, self.param_groups, self.name)
        utils._validate_meaningful_master_weight_bits(params, self.defaults, self.param_groups, self.name)
        path_leaves, self.treedef = utils._tree_leaves_with_paths(params)
        self.paths = [p for p, _ in path_leaves]
        leaves = [as_tensor(leaf) for _, leaf in path_leaves]
        self.shapes = [tuple(t.shape) for t in leaves]
        self.configs = [utils._group_config_for_path(p, t, self.defaults, self.param_groups) for p, t in zip(self.paths, leaves)]
        # leaves of one param group share one config object, so per-step scalars are derived once per group
        interned: Dict[Any, Dict[str, Any]] = {}
        self.configs = [interned.setdefault(tuple(sorted(c.items(), key=lambda kv: kv[0])), c) for c in self.configs]
        self._group_configs: List[Dict[str, Any]] = []
        for c in self.configs:
            if not any(c is g for g in self._group_configs):
                self._group_configs.append(c)
        self._group_id = [next(i for i, g in enumerate(self._group_configs) if g is c) for c in self.configs]
        for c in self.configs:
            if c["quantize"] and c["group_size"] != 32:
                raise ValueError("Zero1Optimizer shards on 32-element group boundaries: group_size must be 32")

        device = leaves[0].device if leaves else torch.device("cpu")
        self.device = device
        self.fused_allgather = bool(fused_allgather) and self.world_size > 1
        self.fused_reduce_scatter = bool(fused_reduce_scatter) and self.world_size > 1
        if self.fused_allgather or self.fused_reduce_scatter:
            if device.type != "cuda" or dist.get_backend(group) != "nccl":
                raise ValueError("fused collectives need CUDA tensors and an NCCL process group")
            if self.world_size - 1 > _lib.FO_MAX_PEERS:
                raise ValueError(f"fused collectives support at most {_lib.FO_MAX_PEERS + 1} ranks")
            if n_slices not in (None, 1):
                raise ValueError("fused collectives work on whole buckets: n_slices must be 1")
            n_slices = 1
        self.max_grad_norm = None if max_grad_norm is None else float(max_grad_norm)
        if self.max_grad_norm is not None:
            if device.type != "cuda":
                raise ValueError("max_grad_norm needs CUDA tensors")
            n_slices = 1  # the norm is known only after the last reduce-scatter: nothing to pipeline
        # Who reads the peers' gradients: the step kernel itself, or, when the step clips by the global norm (whose
        # value needs the whole averaged gradient first), the norm sweep, which leaves this rank's averaged
        # slice in grad_shards for the step.
        self._rs_in_step = self.fused_reduce_scatter and self.max_grad_norm is None
        self._rs_in_norm = self.fused_reduce_scatter and self.max_grad_norm is not None
        if self._rs_in_norm and use_switch:
            raise ValueError("max_grad_norm with fused_reduce_scatter reads the peers point to point: use_switch must be off")
        self.use_switch = use_switch
        self.peer_offsets: List[List[int]] = []
        self.peer_grad_offsets: List[List[int]] = []
        self.mc_param_offsets: List[int] = []
        self.mc_grad_offsets: List[int] = []
        self.buckets: List[BucketLayout] = []
        self.flat_params: List[torch.Tensor] = []
        self.flat_grads: List[torch.Tensor] = []
        self.grad_shards: List[torch.Tensor] = []
        by_dtype: Dict[torch.dtype, List[int]] = {}
        for i, t in enumerate(leaves):
            by_dtype.setdefault(t.dtype, []).append(i)
        param_views: List[Optional[torch.Tensor]] = [None] * len(leaves)
        grad_views: List[Optional[torch.Tensor]] = [None] * len(leaves)
        for dtype, ids in by_dtype.items():
            layout = plan_bucket(dtype, ids, [leaves[i].numel() for i in ids], self.world_size, n_slices)
            flat_p = self._alloc_flat(layout.total, dtype, self.fused_allgather, self.peer_offsets, self.mc_param_offsets)
            flat_g = self._alloc_flat(layout.total, dtype, self.fused_reduce_scatter, self.peer_grad_offsets, self.mc_grad_offsets)
            for i, start in zip(ids, layout.starts):
                n = leaves[i].numel()
                flat_p[start:start + n].copy_(leaves[i].reshape(-1))
                param_views[i] = flat_p[start:start + n].view(self.shapes[i])
                grad_views[i] = flat_g[start:start + n].view(self.shapes[i])
            self.buckets.append(layout)
            self.flat_params.append(flat_p)
            self.flat_grads.append(flat_g)
            # one rank owns everything: the "scattered" gradient is the flat buffer itself
            # (nor is there a scattered copy when the kernel reads the peers' gradients itself)
            own_shard = self.world_size > 1 and not self._rs_in_step
            self.grad_shards.append(torch.zeros(layout.shard, dtype=dtype, device=device) if own_shard else flat_g)
        self.params = self.treedef.unflatten(param_views)
        self.grads = self.treedef.unflatten(grad_views)
        if self.fused_allgather or self.fused_reduce_scatter:
            self._token = torch.zeros(1, dtype=torch.float32, device=device)
            dist.all_reduce(self._token, group=self.group)  # every rank has filled its replica before anyone writes into it
        # state of the segments this rank owns, keyed by (bucket, segment index)
        self.state: Dict[Tuple[int, int], ShardState] = {}
        for b, layout in enumerate(self.buckets):
            for s, seg in enumerate(layout.segments[self.rank]):
                self.state[(b, s)] = self._init_segment(layout.dtype, seg)

    # ---- construction helpers ---------------------------------------------------------------------

    def _alloc_flat(self, n: int, dtype: torch.dtype, symmetric: bool, offsets: List[List[int]], mc_offsets: List[int]) -> torch.Tensor:
        """Flat buffer of a bucket; when a fused collective works on it, a symmetric allocation whose peer
        mappings give the byte offsets from this rank's buffer to every other rank's (appended to `offsets`,
        peers in rank order)."""
        if not symmetric:
            mc_offsets.append(0)
            return torch.zeros(n, dtype=dtype, device=self.device)
        import torch.distributed._symmetric_memory as symm_mem

        buf = symm_mem.empty(n, dtype=dtype, device=self.device)
        buf.zero_()
        pg = self.group if self.group is not None else dist.group.WORLD
        handle = symm_mem.rendezvous(buf, pg.group_name)
        ptrs = list(handle.buffer_ptrs)
        if int(ptrs[self.rank]) != buf.data_ptr():
            raise RuntimeError("symmetric allocation: the local mapping is not the tensor's address; peer offsets would be wrong")
        offsets.append([int(ptrs[r]) - int(ptrs[self.rank]) for r in range(self.world_size) if r != self.rank])
        multicast = int(getattr(handle, "multicast_ptr", 0) or 0)
        if self.use_switch and not multicast:
            raise ValueError("use_switch=True, but the symmetric allocation has no multicast mapping on this system")
        mc_offsets.append(multicast - int(ptrs[self.rank]) if self.use_switch else 0)
        self._symm_handles = getattr(self, "_symm_handles", []) + [handle]
        return buf

    @staticmethod
    def _defaults(optimizer: str, hp: Dict[str, Any]) -> Dict[str, Any]:
        common = {"quantize": True, "master_weight_bits": 24, "group_size": 32, "fused": True}
        if optimizer in ("adamw", "adam"):
            d = {"learning_rate": 1e-3, "b1": 0.9, "b2": 0.999, "eps": 1e-8,
                 "weight_decay": 1e-2 if optimizer == "adamw" else 0.0}
        elif optimizer == "lion":
            d = {"learning_rate": 1e-4, "b1": 0.9, "b2": 0.99, "weight_decay": 0.0}
        else:
            d = {"learning_rate": 1e-3, "momentum": 0.0, "dampening": 0.0, "weight_decay": 0.0, "nesterov": False}
        d.update(common)
        unknown = set(hp) - set(d)
        if unknown:
            raise TypeError(f"unexpected hyper-parameters for {optimizer}: {sorted(unknown)}")
        d.update(hp)
        return d

    def _uses_momentum(self, config) -> bool:
        return self.opt_code != _lib.FO_OPT_SGD or config["momentum"] > 0.0

    def _init_segment(self, dtype: torch.dtype, seg: Segment) -> ShardState:
        config = self.configs[seg.leaf]
        n = seg.hi - seg.lo
        dev = self.device
        ecc = None
        if dtype in (torch.bfloat16, torch.float16) and config["master_weight_bits"] in (24, 32):
            ecc = torch.zeros(n, dtype=torch.int8 if config["master_weight_bits"] == 24 else torch.int16, device=dev)
        mu = mu_s = nu = nu_s = None
        if self._uses_momentum(config):
            groups = -(-n // 32)
            if config["quantize"]:
                mu, mu_s = torch.zeros(n, dtype=torch.int8, device=dev), torch.zeros(groups, dtype=torch.float16, device=dev)
                if self.opt_code == _lib.FO_OPT_ADAM:
                    nu, nu_s = torch.zeros(n, dtype=torch.uint8, device=dev), torch.zeros(groups, dtype=torch.float16, device=dev)
            else:
                mu = torch.zeros(n, dtype=torch.float32, device=dev)
                if self.opt_code == _lib.FO_OPT_ADAM:
                    nu = torch.zeros(n, dtype=torch.float32, device=dev)
        return ShardState(ecc, mu, mu_s, nu, nu_s)

    # ---- the step --------------------------------------------------------------------------------

    def _hyper(self, config, lr: float, count: int):
        if self.opt_code == _lib.FO_OPT_ADAM:
            return adam_hyper(config, lr, count, self.decoupled)
        if self.opt_code == _lib.FO_OPT_LION:
            return lion_hyper(config, lr)
        return sgd_hyper(config, lr, self.decoupled)

    def local_work(self) -> List[eng.LeafWork]:
        """LeafWork of every segment this rank owns, for the step about to run."""
        count_before = torch.tensor(self.count, dtype=torch.int32)
        if getattr(self, "_static_work", None) is not None:
            # buffers never move: only the hyper-parameters change from step to step
            out = []
            cache: Dict[int, Any] = {}
            for w, leaf, _, _ in self._static_work:
                config = self.configs[leaf]
                key = id(config)
                if key not in cache:
                    lr = utils._resolve_learning_rate(config["learning_rate"], count_before)
                    cache[key] = self._hyper(config, lr, self.count + 1)
                out.append(w._replace(hyper=cache[key]))
            return out
        work: List[eng.LeafWork] = []
        meta: List[Tuple[int, int, int]] = []
        dev_index = self.device.index if self.device.type == "cuda" else -1
        for b, layout in enumerate(self.buckets):
            flat_p, g_shard = self.flat_params[b], self.grad_shards[b]
            own_shard = g_shard is not self.flat_grads[b]  # else gradients are addressed like parameters
            for s, seg in enumerate(layout.segments[self.rank]):
                config = self.configs[seg.leaf]
                lr = utils._resolve_learning_rate(config["learning_rate"], count_before)
                st = self.state[(b, s)]
                n = seg.hi - seg.lo
                if st.mu is None:
                    state_kind = _lib.FO_STATE_NONE
                elif config["quantize"]:
                    state_kind = _lib.FO_STATE_QUANT
                else:
                    state_kind = _lib.FO_STATE_FULL
                ecc_bits = 0 if st.ecc is None else st.ecc.element_size() * 8
                bucket = (dev_index, DTYPE_CODE[layout.dtype], DTYPE_CODE[layout.dtype], ecc_bits, state_kind, 32)
                at = flat_position(layout, self.rank, seg.offset)
                work.append(eng.LeafWork(
                    bucket, g_shard[seg.offset:seg.offset + n] if own_shard else g_shard[at:at + n], flat_p[at:at + n],
                    st.ecc, st.mu, st.mu_scales, st.nu, st.nu_scales, self._hyper(config, lr, self.count + 1)))
                meta.append((seg.leaf, b, seg.slice))
        self._static_work = [(w, leaf, b, sl) for w, (leaf, b, sl) in zip(work, meta)]
        return work

    def _run(self, tag: Tuple[Any, ...], pick: Callable[[int, int, int], bool], peers=None, grad_peers=None,
             mc_param: int = 0, mc_grad: int = 0) -> int:
        """Step kernels for the segments `pick(leaf, bucket, slice)` selects.  With the default step function the
        descriptor tables of a selection are built once (tag names the selection) and only the hyper-parameters
        are refreshed per step; an injected step function gets the list of LeafWork as before."""
        if self._step_fn is not eng.launch:
            work = self.local_work()
            items = [w for w, (_, leaf, b, sl) in zip(work, self._static_work) if pick(leaf, b, sl)]
            if not items:
                return 0
            if peers is None and grad_peers is None and not mc_param and not mc_grad:
                return self._step_fn(self.opt_code, items)
            return self._step_fn(self.opt_code, items, peers, grad_peers, mc_param, mc_grad)
        if getattr(self, "_static_work", None) is None:
            self.local_work()
        plans = self.__dict__.setdefault("_plans", {})
        key = (tag, peers is not None, grad_peers is not None, bool(mc_param), bool(mc_grad))
        plan = plans.get(key)
        if plan is None:
            chosen = [(w, self._group_id[leaf]) for w, leaf, b, sl in self._static_work if pick(leaf, b, sl)]
            plan = plans[key] = eng.PreparedLaunch(self.opt_code, [w for w, _ in chosen], [g for _, g in chosen],
                                                   peers, grad_peers, mc_param, mc_grad) if chosen else None
        if plan is None:
            return 0
        count_before = None
        hypers = {}
        for gid, config in enumerate(self._group_configs):
            lr = config["learning_rate"]
            if callable(lr):  # a schedule sees the pre-increment count as a tensor, as in the reference
                if count_before is None:
                    count_before = torch.tensor(self.count, dtype=torch.int32)
                lr = utils._resolve_learning_rate(lr, count_before)
            else:
                lr = utils._resolve_learning_rate(lr, self.count)
            hypers[gid] = self._hyper(config, lr, self.count + 1)
        return plan.run(hypers)

    def _slices(self) -> List[Tuple[int, int]]:
        """(bucket, slice) pairs in the order the collectives are issued."""
        return [(b, sl) for b, layout in enumerate(self.buckets) for sl in range(layout.n_slices)]

    def _rs_args(self, b: int, sl: int):
        layout = self.buckets[b]
        slice_len = layout.piece * self.world_size
        return (self.grad_shards[b][sl * layout.piece:(sl + 1) * layout.piece],
                self.flat_grads[b][sl * slice_len:(sl + 1) * slice_len])

    def _ag_args(self, b: int, sl: int):
        layout = self.buckets[b]
        slice_len = layout.piece * self.world_size
        return self.flat_params[b][sl * slice_len:(sl + 1) * slice_len], layout.piece

    def reduce_scatter_grads(self) -> None:
        if self.world_size == 1:
            aliased = self.__dict__.get("_one_rank_alias")
            if aliased is None:  # one rank: the "shard" normally is the flat buffer itself
                aliased = self._one_rank_alias = all(s.data_ptr() == f.data_ptr() for s, f in zip(self.grad_shards, self.flat_grads))
            if aliased:
                return
        for b, sl in self._slices():
            out, full = self._rs_args(b, sl)
            _reduce_scatter_mean(out, full, self.group, self.world_size)

    def all_gather_params(self) -> None:
        if self.world_size == 1:
            return
        for b, sl in self._slices():
            full, piece = self._ag_args(b, sl)
            _all_gather_inplace(full, piece, self.group, self.world_size)

    def _pipelined(self) -> bool:
        return (self.world_size > 1 and dist.get_backend(self.group) == "nccl" and self.device.type == "cuda"
                and any(layout.n_slices > 1 for layout in self.buckets))

    def _step_pipelined(self) -> None:
        """Slice by slice: the kernels of slice s run while the reduce-scatter of slice s+1 is in flight, and
        each all-gather is queued as soon as its slice is updated (NCCL serialises them behind the
        reduce-scatters on its own stream).  Device-side ordering only; the host never waits."""
        order = self._slices()
        rs = []
        for b, sl in order:
            out, full = self._rs_args(b, sl)
            rs.append(dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.AVG, group=self.group, async_op=True))
        ag = []
        for handle, (b, sl) in zip(rs, order):
            handle.wait()  # the compute stream waits for this slice's gradients
            self._run(("slice", b, sl), lambda _leaf, wb, wsl, b=b, sl=sl: wb == b and wsl == sl)
            full, piece = self._ag_args(b, sl)
            mine = full[self.rank * piece:(self.rank + 1) * piece]
            ag.append(dist.all_gather_into_tensor(full, mine, group=self.group, async_op=True))
        for handle in ag:
            handle.wait()

    def step_from_host(self, host_grads: Any, n_groups: int = 8) -> Any:
        """One optimizer step on gradients that live in (pinned) host memory.  On a single rank without
        clipping the leaves are cut into `n_groups` groups of about equal size; the host-to-device copy
        of a group runs on a copy stream while the step of the group before it runs, so the step hides
        behind the transfer.  Otherwise (several ranks, clipping: the whole gradient must be there first)
        it is a copy followed by `step()`.  Same result either way.  Returns `self.params`."""
        leaves, treedef = pytree.tree_flatten(host_grads)
        if treedef != self.treedef:
            raise ValueError(f"{self.name} gradients must match parameter structure")
        mine = pytree.tree_leaves(self.grads)
        if self.world_size > 1 or self.max_grad_norm is not None or self.device.type != "cuda":
            for dst, src in zip(mine, leaves):
                dst.copy_(as_tensor(src).reshape(dst.shape), non_blocking=True)
            return self.step()
        total = sum(t.numel() * t.element_size() for t in mine)
        main = torch.cuda.current_stream(self.device)
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream(self.device)
        copier = self._copy_stream
        copier.wait_stream(main)  # the previous step has finished reading the gradient buffers
        group: List[int] = []
        acc, share = 0, total / max(1, n_groups)
        order = list(range(len(mine)))

        def flush():
            nonlocal group
            if not group:
                return
            with torch.cuda.stream(copier):
                for i in group:
                    mine[i].copy_(as_tensor(leaves[i]).reshape(mine[i].shape), non_blocking=True)
                done = torch.cuda.Event()
                done.record(copier)
            main.wait_event(done)
            chosen = frozenset(group)  # every segment of these leaves (a leaf that straddles slices has several)
            self._run(("leaves", tuple(group)), lambda leaf, _b, _sl: leaf in chosen)
            group = []

        for i in order:
            group.append(i)
            acc += mine[i].numel() * mine[i].element_size()
            if acc >= share:
                flush()
                acc = 0
        flush()
        self.count += 1
        return self.params

    ALL_PHASES = ("reduce_scatter", "step", "all_gather")

    def step(self, grads: Any = None, phases: Tuple[str, ...] = ALL_PHASES) -> Any:
        """One optimizer step.  `grads` (optional) is copied into the flat gradient buffers;
        leave it out when backward already wrote into `self.grads`.  Returns `self.params`.

        `phases` is for measurement: leaving "reduce_scatter" out steps on this rank's own gradients,
        leaving "all_gather" out keeps the updated slice local (the replicas then disagree; the state
        is of no further use).  The default runs the whole ZeRO-1 step."""
        unknown = set(phases) - set(self.ALL_PHASES)
        if unknown or "step" not in phases:
            raise ValueError(f"phases must contain 'step' and only names of {self.ALL_PHASES}, got {phases}")
        do_rs, do_ag = "reduce_scatter" in phases, "all_gather" in phases
        if grads is not None:
            leaves, treedef = pytree.tree_flatten(grads)
            if treedef != self.treedef:
                raise ValueError(f"{self.name} gradients must match parameter structure")
            for mine, theirs in zip(pytree.tree_leaves(self.grads), leaves):
                theirs = as_tensor(theirs)
                if theirs.dtype != mine.dtype and theirs.element_size() > mine.element_size():
                    # the flat gradient buffers (and the reduce-scatter) have the parameters' dtype
                    raise TypeError(f"{self.name}: a {theirs.dtype} gradient would be narrowed to the {mine.dtype} gradient "
                                    "buffer of its leaf; cast it yourself or write into `.grads` directly")
                mine.copy_(theirs.to(mine.dtype).reshape(mine.shape))
        if self._pipelined():
            if not (do_rs and do_ag):
                raise ValueError("the sliced pipeline runs whole steps only")
            self._step_pipelined()
            self.count += 1
            return self.params
        if do_rs:
            if self.fused_reduce_scatter:
                dist.all_reduce(self._token, group=self.group)  # every rank's gradients are complete before any kernel reads them
            else:
                self.reduce_scatter_grads()
        with self._clip_context():
            return self._launch_and_gather(do_rs, do_ag)

    def _clip_context(self):
        """Global-norm clipping for the launches of this step: the squares of this rank's slices (padding is
        zero), summed over the ranks."""
        if self.max_grad_norm is None:
            return contextlib.nullcontext()
        if self._rs_in_norm:
            sq = torch.zeros(1, dtype=torch.float64, device=self.device)
            for b, layout in enumerate(self.buckets):
                mine = self.flat_grads[b][self.rank * layout.shard:(self.rank + 1) * layout.shard]
                eng.mean_sq_norm(mine, self.grad_shards[b], self.peer_grad_offsets[b], sq, accumulate=b > 0)
        else:
            sq = eng.sq_norm_of(list(self.grad_shards))
        if self.world_size > 1:
            dist.all_reduce(sq, group=self.group)
        return eng.grad_clip(sq, self.max_grad_norm)

    def _launch_and_gather(self, do_rs: bool = True, do_ag: bool = True) -> Any:
        if self.fused_allgather or self.fused_reduce_scatter:
            for b in range(len(self.buckets)):
                self._run(("bucket", b), lambda _leaf, wb, _sl, b=b: wb == b,
                          self.peer_offsets[b] if (self.fused_allgather and do_ag) else None,
                          self.peer_grad_offsets[b] if (self._rs_in_step and do_rs) else None,
                          self.mc_param_offsets[b] if do_ag else 0, self.mc_grad_offsets[b] if do_rs else 0)
            self.count += 1
            if self.fused_allgather:
                # all ranks' kernels are complete: their stores into this replica, their reads of these gradients
                dist.all_reduce(self._token, group=self.group)
            elif do_ag:
                self.all_gather_params()  # a collective, hence also the barrier that protects the gradients
            elif self._rs_in_step and do_rs:
                dist.all_reduce(self._token, group=self.group)
            return self.params
        self._run(("all",), lambda _leaf, _b, _sl: True)
        self.count += 1
        if do_ag:
            self.all_gather_params()
        return self.params

    # ---- checkpoint / export -------------------------------------------------------------------------

    def local_state_dict(self) -> Dict[str, Any]:
        """This rank's shard: segment table plus tensors (save one per rank, reload with load_local_state_dict)."""
        out = {"count": self.count, "world_size": self.world_size, "rank": self.rank, "segments": {}}
        for (b, s), st in self.state.items():
            seg = self.buckets[b].segments[self.rank][s]
            out["segments"][(b, s)] = {"leaf": seg.leaf, "lo": seg.lo, "hi": seg.hi,
                                       **{k: v for k, v in st._asdict().items() if v is not None}}
        return out

    def load_local_state_dict(self, sd: Dict[str, Any]) -> None:
        if sd["world_size"] != self.world_size or sd["rank"] != self.rank:
            raise ValueError("shard was saved for a different world size or rank")
        self.count = int(sd["count"])
        for key, entry in sd["segments"].items():
            seg = self.buckets[key[0]].segments[self.rank][key[1]]
            if (entry["leaf"], entry["lo"], entry["hi"]) != (seg.leaf, seg.lo, seg.hi):
                raise ValueError(f"segment {key} does not match this layout")
            st = self.state[key]
            for name, mine in st._asdict().items():
                if mine is not None:
                    mine.copy_(entry[name])

    # -- unsharded state in the reference's layout, assembled on the device ----------------------------------

    _STREAMS = ("ecc", "mu", "mu_scales", "nu", "nu_scales")

    def _gather_stream(self, b: int, name: str) -> Optional[torch.Tensor]:
        """The flat buffer of one state stream of bucket b, assembled from all ranks' slices with one
        all-gather per slice, on the device the state lives on (no host copy).  Element i of the result belongs
        to position i of the bucket's flat parameter buffer (i // 32 for the group scales).  None when no leaf
        of the bucket has the stream; mixed dtypes inside a bucket (param groups that differ in
        master_weight_bits) are not handled here."""
        layout = self.buckets[b]
        mine = [(seg, getattr(self.state[(b, s)], name)) for s, seg in enumerate(layout.segments[self.rank])]
        # every rank must agree on dtype and presence without talking: derive both from the configs
        kinds = set()
        for leaf in layout.leaves:
            c = self.configs[leaf]
            has_ecc = layout.dtype in (torch.bfloat16, torch.float16) and c["master_weight_bits"] in (24, 32)
            quant, mom = c["quantize"], self._uses_momentum(c)
            if name == "ecc":
                kinds.add((torch.int8 if c["master_weight_bits"] == 24 else torch.int16) if has_ecc else None)
            elif name in ("mu", "nu"):
                present = mom and (name == "mu" or self.opt_code == _lib.FO_OPT_ADAM)
                kinds.add(None if not present else ((torch.int8 if name == "mu" else torch.uint8) if quant else torch.float32))
            else:
                present = mom and quant and (name == "mu_scales" or self.opt_code == _lib.FO_OPT_ADAM)
                kinds.add(torch.float16 if present else None)
        if kinds == {None}:
            return None
        if len(kinds) != 1:
            raise NotImplementedError("state_dict(): leaves of one dtype bucket differ in how they store " + name)
        dtype = kinds.pop()
        per = 32 if name.endswith("scales") else 1
        piece, world = layout.piece // per, self.world_size
        full = torch.zeros(layout.n_slices * world * piece, dtype=dtype, device=self.device)
        for seg, t in mine:
            at = flat_position(layout, self.rank, seg.offset) // per
            full[at:at + t.numel()].copy_(t)
        raw = full.view(torch.uint8)  # bytes travel: every backend carries uint8, not every one int16 / fp16
        width = full.element_size()
        for sl in range(layout.n_slices):
            _all_gather_inplace(raw[sl * world * piece * width:(sl + 1) * world * piece * width], piece * width, self.group, world)
        return full

    def state_dict(self) -> Dict[str, Any]:
        """The optimizer state in the reference's checkpoint form (flashoptim_jax/adamw.py:639-644, lion.py:234-239,
        sgd.py:314-319 over utils.py:377-407): {"count", "mu", ["nu",] "ecc"}, each tree serialised leaf by leaf as
        {"kind": "quantized", "values", "scales"} or {"kind": "array", "value"}.  Collective: every rank calls it and
        every rank gets the whole state; the slices travel device to device (one all-gather per state stream)."""
        from .quantization import QuantizedArray

        n_leaves = len(self.shapes)
        ecc: List[Any] = [None] * n_leaves
        mu: List[Any] = [None] * n_leaves
        nu: List[Any] = [None] * n_leaves
        for b, layout in enumerate(self.buckets):
            flat = {name: self._gather_stream(b, name) for name in self._STREAMS}
            for leaf, start, n in zip(layout.leaves, layout.starts, layout.sizes):
                shape, groups = self.shapes[leaf], -(-n // 32)
                take = lambda name: None if flat[name] is None else (  # noqa: E731
                    flat[name][start // 32:start // 32 + groups] if name.endswith("scales") else flat[name][start:start + n].view(shape)).clone()
                sentinel = lambda: torch.zeros((), dtype=torch.int32, device=self.device)  # noqa: E731
                ecc[leaf] = take("ecc") if flat["ecc"] is not None else sentinel()
                for vals, scales, out in (("mu", "mu_scales", mu), ("nu", "nu_scales", nu)):
                    if flat[vals] is None:
                        out[leaf] = sentinel()
                    elif flat[scales] is not None:
                        out[leaf] = QuantizedArray(values=take(vals), scales=take(scales))
                    else:
                        out[leaf] = take(vals)
        sd = {"count": torch.tensor(self.count, dtype=torch.int32), "mu": utils._tree_state_dict(self.treedef.unflatten(mu)),
              "ecc": utils._tree_state_dict(self.treedef.unflatten(ecc))}
        if self.opt_code == _lib.FO_OPT_ADAM:
            sd["nu"] = utils._tree_state_dict(self.treedef.unflatten(nu))
        return sd

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        """Inverse of state_dict(), for any world size: every rank copies the slices it owns out of the
        unsharded trees (which may live on the host or on any device)."""
        from .quantization import QuantizedArray

        trees = {name: pytree.tree_leaves(utils._tree_from_state_dict(sd[name]), is_leaf=lambda x: isinstance(x, QuantizedArray))
                 for name in ("mu", "nu", "ecc") if name in sd}
        for name, leaves in trees.items():
            if len(leaves) != len(self.shapes):
                raise ValueError(f"{self.name} state trees must match parameter structure")
        self.count = int(sd["count"])
        for (b, s), st in self.state.items():
            seg = self.buckets[b].segments[self.rank][s]
            glo, ghi = seg.lo // 32, -(-seg.hi // 32)

            def put(dst, src, lo, hi):
                if dst is None:
                    return
                src = as_tensor(src).reshape(-1)
                if src.dtype != dst.dtype or src.numel() < hi:
                    raise ValueError(f"{self.name} state of leaf {seg.leaf} does not fit this optimizer's layout")
                dst.copy_(src[lo:hi])

            if st.ecc is not None:
                put(st.ecc, trees["ecc"][seg.leaf], seg.lo, seg.hi)
            for vals, scales, key in ((st.mu, st.mu_scales, "mu"), (st.nu, st.nu_scales, "nu")):
                if vals is None:
                    continue
                leaf = trees[key][seg.leaf]
                if isinstance(leaf, QuantizedArray):
                    put(vals, leaf.values, seg.lo, seg.hi)
                    put(scales, leaf.scales, glo, ghi)
                else:
                    put(vals, leaf, seg.lo, seg.hi)

    def master_weights(self) -> Any:
        """reconstruct_weights for the sharded optimizer (flashoptim_jax/compression.py:124-126, README "export"):
        the fp32 master weights as a tree like `params`.  Collective: the ECC slices are all-gathered on the
        device, then every rank reconstructs (the reconstruction kernel, one pass over parameter + ECC)."""
        from .compression import reconstruct_leaf

        out: List[Any] = [None] * len(self.shapes)
        param_leaves = pytree.tree_leaves(self.params)
        for b, layout in enumerate(self.buckets):
            ecc = self._gather_stream(b, "ecc")
            for leaf, start, n in zip(layout.leaves, layout.starts, layout.sizes):
                p = param_leaves[leaf]
                out[leaf] = p.to(torch.float32) if ecc is None else reconstruct_leaf(p, ecc[start:start + n].view(self.shapes[leaf]))
        return self.treedef.unflatten(out)

    def set_master_weights(self, fp32_params: Any) -> Any:
        """set_fp32_params for the sharded optimizer (flashoptim_jax/compression.py:129-146, README "import"):
        every rank splits the slices it owns into stored parameter + ECC (the split kernel), then the updated
        parameters are all-gathered.  The moments are left as they are.  Returns `self.params`."""
        from .compression import split_leaf

        leaves, treedef = pytree.tree_flatten(fp32_params)
        if treedef != self.treedef:
            raise ValueError("fp32_params and param_template must have matching tree structure")
        for (b, s), st in self.state.items():
            layout = self.buckets[b]
            seg = layout.segments[self.rank][s]
            at = flat_position(layout, self.rank, seg.offset)
            src = as_tensor(leaves[seg.leaf]).reshape(-1)[seg.lo:seg.hi].to(device=self.device, dtype=torch.float32)
            mwb = self.configs[seg.leaf]["master_weight_bits"] if st.ecc is not None else None
            lp, ecc = split_leaf(src, narrow_dtype=layout.dtype, master_weight_bits=mwb)
            self.flat_params[b][at:at + (seg.hi - seg.lo)].copy_(lp)
            if st.ecc is not None:
                st.ecc.copy_(ecc)
        self.all_gather_params()
        return self.params

    # -- per-rank files -----------------------------------------------------------------------------------------

    SHARD_FORMAT = 1

    def save_shards(self, directory: str) -> str:
        """Writes this rank's slice of the state to `directory` (every rank calls it; no communication):
        `shard_<rank>_of_<world>.pt` holds a header (format number, optimizer, step count, the table of
        segments with their leaf paths and element ranges) and the slice's tensors on the host.  Reload
        with load_shards on the same world size, or convert with state_dict() / load_state_dict() to move to
        another."""
        import os as _os

        _os.makedirs(directory, exist_ok=True)
        path = _os.path.join(directory, f"shard_{self.rank:05d}_of_{self.world_size:05d}.pt")
        segments = []
        for (b, s), st in sorted(self.state.items()):
            seg = self.buckets[b].segments[self.rank][s]
            segments.append({"bucket": b, "index": s, "leaf": seg.leaf, "path": "/".join(str(x) for x in self.paths[seg.leaf]),
                             "lo": seg.lo, "hi": seg.hi, "tensors": {k: v.detach().cpu() for k, v in st._asdict().items() if v is not None}})
        torch.save({"format": self.SHARD_FORMAT, "optimizer": self.name, "count": self.count, "world_size": self.world_size,
                    "rank": self.rank, "leaf_shapes": [list(x) for x in self.shapes], "segments": segments}, path)
        return path

    def load_shards(self, directory: str) -> None:
        import os as _os

        path = _os.path.join(directory, f"shard_{self.rank:05d}_of_{self.world_size:05d}.pt")
        if not _os.path.exists(path):
            raise FileNotFoundError(f"{path}: no shard for rank {self.rank} of {self.world_size} (saved with another world size? "
                                    "use state_dict() / load_state_dict() to re-shard)")
        blob = torch.load(path, map_location="cpu", weights_only=False)
        if blob.get("format") != self.SHARD_FORMAT or blob["optimizer"] != self.name:
            raise ValueError(f"{path} is not a format-{self.SHARD_FORMAT} shard of {self.name}")
        if [list(x) for x in self.shapes] != blob["leaf_shapes"]:
            raise ValueError(f"{path} was saved for a different parameter tree")
        for entry in blob["segments"]:
            key = (entry["bucket"], entry["index"])
            seg = self.buckets[key[0]].segments[self.rank][key[1]]
            if (entry["leaf"], entry["lo"], entry["hi"]) != (seg.leaf, seg.lo, seg.hi):
                raise ValueError(f"segment {key} of {path} does not match this layout")
            for name, mine in self.state[key]._asdict().items():
                if mine is not None:
                    mine.copy_(entry["tensors"][name])
        self.count = int(blob["count"])

    def gather_state(self, dst: int = 0) -> Optional[Dict[str, Any]]:
        """Assemble the reference's unsharded state on rank `dst`: {"count", "mu", "nu", "ecc"} trees with
        the layout tx.init() gives (QuantizedArray leaves, 0-d int32 sentinels)."""
        from .quantization import QuantizedArray

        pieces = {name: [None] * len(self.shapes) for name in ("ecc", "mu", "mu_scales", "nu", "nu_scales")}
        gathered: List[Any] = [None] * self.world_size
        mine = [(self.buckets[b].segments[self.rank][s], {k: v.cpu() for k, v in st._asdict().items() if v is not None})
                for (b, s), st in self.state.items()]
        if self.world_size > 1:
            dist.gather_object(mine, gathered if self.rank == dst else None, dst=dst, group=self.group)
        else:
            gathered = [mine]
        if self.rank != dst:
            return None
        full: Dict[str, List[Any]] = {k: [None] * len(self.shapes) for k in pieces}
        for rank_items in gathered:
            for seg, tensors in rank_items:
                n = 1
                for d in self.shapes[seg.leaf]:
                    n *= d
                for name, t in tensors.items():
                    if full[name][seg.leaf] is None:
                        length = -(-n // 32) if name.endswith("scales") else n
                        full[name][seg.leaf] = torch.zeros(length, dtype=t.dtype)
                    if name.endswith("scales"):
                        full[name][seg.leaf][seg.lo // 32: seg.lo // 32 + t.numel()] = t
                    else:
                        full[name][seg.leaf][seg.lo:seg.hi] = t
        ecc, mu, nu = [], [], []
        for i, shape in enumerate(self.shapes):
            ecc.append(full["ecc"][i].view(shape) if full["ecc"][i] is not None else torch.zeros((), dtype=torch.int32))
            for vals, scales, out in (("mu", "mu_scales", mu), ("nu", "nu_scales", nu)):
                v, s = full[vals][i], full[scales][i]
                if v is None:
                    out.append(torch.zeros((), dtype=torch.int32))
                elif s is not None:
                    out.append(QuantizedArray(values=v.view(shape), scales=s))
                else:
                    out.append(v.view(shape))
        state = {"count": torch.tensor(self.count, dtype=torch.int32), "mu": self.treedef.unflatten(mu),
                 "ecc": self.treedef.unflatten(ecc)}
        if self.opt_code == _lib.FO_OPT_ADAM:
            state["nu"] = self.treedef.unflatten(nu)
        return state
