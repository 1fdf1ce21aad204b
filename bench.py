"""Optimizer-step benchmark: Llama-3-8B-shaped pytree, flash AdamW with 32-bit master weights.

    python bench.py --gpus N --steps K --warmup W            (this library)
    python bench.py --impl reference ...                     (the reference's CPU path, restated)

One step = one pass of the fused update over the whole pytree.  With N > 1 the step is
ZeRO-1 (launch with torchrun, one rank per GPU): reduce-scatter(mean) of the bf16 gradients,
the fused kernel on the rank's slice, all-gather of the updated parameters - both collectives
inside the kernel over NVLink peer pointers by default, through NCCL with --nccl-reduce-scatter /
--nccl-allgather.
Inputs are synthetic (seeded normal draws with the configured shapes and scales).  Rank 0
prints ONE JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "optimizer-step params/sec"
UNIT = "params/s"

# algorithmic bytes per parameter of one in-place step (bf16 grads, group size 32):
# read grad 2 + param 2 + ecc 2 + mu 1 + nu 1 + two fp16 scales per 32 elements; write the same minus the grad
BYTES_PER_PARAM_BF16_ECC16 = (2 + 2 + 2 + 1 + 1 + 0.125) + (2 + 2 + 1 + 1 + 0.125)  # 14.25
BYTES_PER_PARAM_F32 = (4 + 4 + 1 + 1 + 0.125) + (4 + 1 + 1 + 0.125)                   # 16.25
# DRAM bytes per parameter seen by one ncu capture of the bf16 kernel (profiles/), scaled to a launch by its parameter count
NCU_DRAM_BYTES_PER_PARAM = 13.47  # profiles/step_kernel_adam_bf16_ecc16_quant__one_64M_leaf.md: 904.3 MB per 67,108,864 params; traffic is proportional to the parameter count


def llama3_8b_shapes():
    """Leaf shapes of the Llama-3-8B pytree: 291 leaves, 8,030,261,248 parameters."""
    shapes = {"tok_embeddings": ((128256, 4096), "bf16"), "lm_head": ((128256, 4096), "bf16"), "norm": ((4096,), "f32")}
    for i in range(32):
        p = f"layers.{i:02d}."
        shapes[p + "wq"] = ((4096, 4096), "bf16")
        shapes[p + "wk"] = ((4096, 1024), "bf16")
        shapes[p + "wv"] = ((4096, 1024), "bf16")
        shapes[p + "wo"] = ((4096, 4096), "bf16")
        shapes[p + "w1"] = ((4096, 14336), "bf16")
        shapes[p + "w3"] = ((4096, 14336), "bf16")
        shapes[p + "w2"] = ((14336, 4096), "bf16")
        shapes[p + "attention_norm"] = ((4096,), "f32")
        shapes[p + "ffn_norm"] = ((4096,), "f32")
    return shapes


def small_shapes():
    """A 1/64-scale pytree with the same leaf mix, for quick checks (not the benchmark workload)."""
    shapes = {"tok_embeddings": ((8192, 1024), "bf16"), "lm_head": ((8192, 1024), "bf16"), "norm": ((1024,), "f32")}
    for i in range(8):
        p = f"layers.{i:02d}."
        for name, shp in (("wq", (1024, 1024)), ("wk", (1024, 256)), ("wv", (1024, 256)), ("wo", (1024, 1024)),
                          ("w1", (1024, 3584)), ("w3", (1024, 3584)), ("w2", (3584, 1024))):
            shapes[p + name] = (shp, "bf16")
        shapes[p + "attention_norm"] = ((1024,), "f32")
        shapes[p + "ffn_norm"] = ((1024,), "f32")
    return shapes


def one_leaf_shapes():
    """One 2^26-element bf16 leaf (0.96 GB touched per step): the small case ncu captures are taken on."""
    return {"w": ((8192, 8192), "bf16")}


WORKLOADS = {"llama3_8b": llama3_8b_shapes, "llama3_8b_div64": small_shapes, "adamw_leaf_64m": one_leaf_shapes}
HPARAMS = dict(learning_rate=3e-4, b1=0.9, b2=0.999, eps=1e-8, weight_decay=0.1, master_weight_bits=32)


def numel(shape):
    n = 1
    for d in shape:
        n *= d
    return n


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU, sampled every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(n_params: int, steps: int, threads: int = 0):
    """The reference's CPU path (restated in C, OpenMP) on a bounded sample: AdamW on n_params bf16 parameters."""
    import numpy as np

    from oracle import c_oracle as C
    from oracle import flashoptim_oracle as O
    from tests import helpers as H

    C.build()
    cores = C.set_threads(threads)
    rng = np.random.default_rng(0)
    pnp = rng.standard_normal(n_params, dtype=np.float32) * np.float32(0.02)
    leaf = H.fresh_leaf(pnp.astype(H.BF16), C.ADAM, C.STATE_QUANT, 16)
    g = (rng.standard_normal(n_params, dtype=np.float32) * np.float32(1e-4)).astype(H.BF16)
    times = []
    for t in range(1, steps + 2):
        hp = H.hyper_tuple(C.ADAM, O.UNFUSED, t, lr=HPARAMS["learning_rate"], wd=HPARAMS["weight_decay"])
        t0 = time.perf_counter()
        H.oracle_step(C.ADAM, g, leaf, C.STATE_QUANT, 32, hp)
        times.append(time.perf_counter() - t0)
    times = times[1:]  # first call pages memory in
    per_step = sum(times) / len(times)
    return {"value": n_params / per_step, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"AdamW (32-bit master) on one {n_params}-element bf16 leaf, {len(times)} steps, C restatement of the reference's CPU path with OpenMP"}, per_step


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = 1 << 26
    base, per_step = cpu_baseline(n, max(1, args.steps))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": args.workload, "optimizer": "flash_adamw", **{k: v for k, v in HPARAMS.items()},
                                                        "note": "JAX is not installed, so the reference's CPU (unfused) path runs as its C restatement on a bounded sample"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


_REAL_STDOUT = None


def quiet_stdout():
    """Point file descriptor 1 at stderr for the duration of the run: libraries that write to stdout on their own
    (NCCL prints its version there at NCCL_DEBUG=VERSION) must not add lines to the one JSON line of the result."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    """The one JSON line, on the real stdout."""
    text = json.dumps(line) + "\n"
    sys.stdout.flush()
    if _REAL_STDOUT is None:
        sys.stdout.write(text)
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, text.encode())


def run_ours(args):
    quiet_stdout()
    import torch
    import torch.distributed as dist

    from flashoptim_jax_b200 import _engine as eng
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    shapes = WORKLOADS[args.workload]()
    total_params = sum(numel(s) for s, _ in shapes.values())
    gen = torch.Generator(device=device)
    gen.manual_seed(1234)  # same draws on every rank: parameters are replicated
    params = {}
    for name, (shape, kind) in shapes.items():
        if kind == "bf16":
            params[name] = (torch.randn(shape, device=device, generator=gen) * 0.02).to(torch.bfloat16)
        else:
            params[name] = torch.ones(shape, device=device, dtype=torch.float32)

    kernel_ms = {}  # per (param dtype code) -> list of launch durations
    pending = []

    def timed_launch(opt, work, peers=None, grad_peers=None, mc_param=0, mc_grad=0):
        by_bucket = {}
        for w in work:
            by_bucket.setdefault(w.bucket, []).append(w)
        calls = 0
        for bucket, items in by_bucket.items():
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            calls += eng.launch(opt, items, peers, grad_peers, mc_param, mc_grad)
            e1.record()
            pending.append((bucket[1], sum(w.param.numel() for w in items), e0, e1))
        return calls

    launches = [0]

    def counting_launch(opt, work, peers=None, grad_peers=None, mc_param=0, mc_grad=0):
        n = timed_launch(opt, work, peers, grad_peers, mc_param, mc_grad)
        launches[0] += n
        return n

    fused = {"fused_allgather": world > 1 and not args.nccl_allgather,
             "fused_reduce_scatter": world > 1 and not args.nccl_reduce_scatter and args.clip is None}
    try:
        zero = Zero1Optimizer("adamw", params, step_fn=counting_launch, max_grad_norm=args.clip, n_slices=args.slices,
                              use_switch=args.switch, **fused, **HPARAMS)
    except Exception as e:  # no peer-mapped (symmetric) memory on this system: every rank fails alike
        if not any(fused.values()):
            raise
        print(f"fused collectives unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
        args.nccl_allgather = args.nccl_reduce_scatter = True
        args.switch = False
        zero = Zero1Optimizer("adamw", params, step_fn=counting_launch, max_grad_norm=args.clip, n_slices=args.slices, **HPARAMS)
    del params
    torch.cuda.empty_cache()
    ggen = torch.Generator(device=device)
    # The same draw on every rank: the averaged gradient of the N-rank job then equals the
    # gradient of the 1-rank job (strong scaling of one problem).  Different fixed draws per rank
    # would average to exact zeros at about 7e-4 of the positions, the same ones every step, which
    # no training run with fresh gradients per step has.
    ggen.manual_seed(99)
    from flashoptim_jax_b200 import tree as pytree

    for g in pytree.tree_leaves(zero.grads):
        g.copy_((torch.randn(g.shape, device=device, generator=ggen) * 1e-4).to(g.dtype))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        zero.step()
    barrier()
    pending.clear()
    launches[0] = 0
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        zero.step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    elapsed_ms = e0.elapsed_time(e1)
    n_launch = launches[0]
    if args.clip is not None:
        n_launch += 2 * len(zero.buckets) * args.steps  # fo_sq_norm: partial sums and their fixed-order total, per dtype
    for code, n_par, a, b in pending:
        kernel_ms.setdefault(code, []).append((n_par, a.elapsed_time(b)))
    if world > 1:
        t = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t)
    ms_per_step = elapsed_ms / args.steps
    value = total_params / (ms_per_step * 1e-3)

    # roofline of the dominant kernel (the bf16 / int16-ECC AdamW launch), from its own CUDA-event durations
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    else:
        peak, peak_src = 6650.0, "fallback"
    bf16_launches = kernel_ms.get(1, [])
    n_par = bf16_launches[0][0] if bf16_launches else 0
    avg_ms = sum(ms for _, ms in bf16_launches) / max(1, len(bf16_launches))
    achieved = n_par * BYTES_PER_PARAM_BF16_ECC16 / (avg_ms * 1e-3) / 1e9 if avg_ms else 0.0
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None if NCU_DRAM_BYTES_PER_PARAM is None else NCU_DRAM_BYTES_PER_PARAM * n_par,
                "kernel": "step_kernel<adam, bf16, ecc16, quant>", "params_per_launch": n_par, "avg_launch_ms": avg_ms,
                "algorithmic_bytes_per_param": BYTES_PER_PARAM_BF16_ECC16, "peak_source": peak_src}

    e2e = None
    if not args.no_e2e:
        e2e = measure_e2e(args, zero, device, ggen, world, barrier, total_params)
    link_bytes = (sum(g.numel() * g.element_size() for g in pytree.tree_leaves(zero.grads))
                  + sum(q.numel() * q.element_size() for q in pytree.tree_leaves(zero.params)))
    zero_info = {"mc": list(zero.mc_param_offsets) + list(zero.mc_grad_offsets)}
    finish(args, world, rank, shapes, total_params, value, ms_per_step, roofline, e2e, n_launch, clocks, link_bytes, zero_info)


def measure_e2e(args, zero, device, ggen, world, barrier, total_params):
    """End to end through the public API with gradients arriving from pinned host memory every step."""
    import torch
    import torch.distributed as dist

    from flashoptim_jax_b200 import tree as pytree

    e2e_steps = max(1, min(args.steps, 2))
    grad_leaves = pytree.tree_leaves(zero.grads)
    # pinned host gradients: every leaf is a window of one staging buffer (the values repeat; 16 GB of
    # pinned memory per rank would be needed otherwise), fp32 norm leaves of a small one
    stage_elems = max(1 << 28, max(g.numel() for g in grad_leaves))
    stage = torch.empty(stage_elems, dtype=torch.bfloat16, pin_memory=True)
    fill = 1 << 26
    for lo in range(0, stage_elems, fill):
        m = min(fill, stage_elems - lo)
        stage[lo:lo + m].copy_((torch.randn(m, device=device, generator=ggen) * 1e-4).to(torch.bfloat16).cpu())
    stage32 = torch.full((max(g.numel() for g in grad_leaves if g.dtype == torch.float32),), 1e-4, dtype=torch.float32).pin_memory()
    host_leaves, off = [], 0
    for g in grad_leaves:
        n = g.numel()
        if g.dtype == torch.float32:
            host_leaves.append(stage32[:n].view(g.shape))
            continue
        if off + n > stage_elems:
            off = 0
        host_leaves.append(stage[off:off + n].view(g.shape))
        off += n
    host_grads = pytree.tree_unflatten(pytree.tree_structure(zero.grads), host_leaves)
    h2d = sum(g.numel() * g.element_size() for g in grad_leaves)
    probe = torch.empty(1, dtype=torch.float32).pin_memory()
    first_param = pytree.tree_leaves(zero.params)[0].view(-1)

    def e2e_step():
        zero.step_from_host(host_grads)  # host -> device copies of this step's gradients, overlapped with the step on one rank
        probe.copy_(first_param[:1].float(), non_blocking=True)  # device -> host read of a result
        torch.cuda.current_stream().synchronize()

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t)
    return {"value": total_params / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
            "ms_per_step": e2e_s * 1e3, "steps": e2e_steps}


def finish(args, world, rank, shapes, total_params, value, ms_per_step, roofline, e2e, n_launch, clocks, link_bytes, zero_info):
    import torch.distributed as dist

    if rank == 0:
        base = None
        if world == 1 and not args.no_cpu_baseline:
            base, _ = cpu_baseline(1 << 26, 3)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": args.workload, "leaves": len(shapes), "params": total_params, "optimizer": "flash_adamw",
                       **HPARAMS, "grad_dtype": "bf16", "parallelism": "single" if world == 1 else f"zero1x{world}",
                       "reduce_scatter": None if world == 1 else ("nccl" if (args.nccl_reduce_scatter or args.clip is not None) else "fused into the step kernel (peer loads)"),
                       "clip_global_norm": args.clip, "slices": args.slices,
                       "switch": None if world == 1 else bool(any(zero_info["mc"])),
                       "allgather": None if world == 1 else ("nccl" if args.nccl_allgather else "fused into the step kernel (peer stores)"),
                       "l2": "working set per step (>= 14 B/param) exceeds the 126 MB L2, no flush needed"},
            "roofline": roofline, "cpu_baseline": base, "e2e": e2e, "gpu_launches": n_launch, "clocks": clocks,
            "hbm_gbs_whole_step": total_params * BYTES_PER_PARAM_BF16_ECC16 / (ms_per_step * 1e-3) / 1e9,
        }
        if world > 1:
            # What must cross NVLink per GPU and direction in one ZeRO-1 step: (N-1)/N of the gradients in
            # (reduce-scatter) and of the parameters out (all-gather), and the same amounts the other way
            # for the peers.  770 GB/s: peer copy per direction measured on this pool.
            per_direction = link_bytes * (world - 1) / world
            if any(zero_info["mc"]):
                # through the switch: every gradient leaves once (the switch adds), the reduced slice comes in;
                # the parameter slice leaves once (the switch replicates), every replica's full copy comes in
                per_direction = (link_bytes / 2) * (1 + 1 / world)
            achieved = per_direction / (ms_per_step * 1e-3) / 1e9
            line["nvlink"] = {"bytes_per_direction_per_gpu": per_direction, "achieved": achieved, "peak": 770.0, "unit": "GB/s",
                              "frac": achieved / 770.0, "floor_ms": per_direction / 770e9 * 1e3}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="llama3_8b")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (used for ncu captures)")
    ap.add_argument("--nccl-allgather", action="store_true", help="N > 1: NCCL all-gather after the step instead of peer stores inside it")
    ap.add_argument("--switch", action="store_true",
                    help="N > 1: fused collectives through the NVLink switch (multicast store, multicast load-reduce); "
                         "off by default: the switch's bf16 addition is not round-to-nearest, so parity with the reference is lost")
    ap.add_argument("--slices", type=int, default=None,
                    help="N > 1 with both NCCL collectives: slices per bucket whose reduce-scatter / step / all-gather overlap")
    ap.add_argument("--clip", type=float, default=None,
                    help="clip the gradients at this global norm inside the step (adds the sum-of-squares sweep; off by default)")
    ap.add_argument("--nccl-reduce-scatter", action="store_true", help="N > 1: NCCL reduce-scatter before the step instead of peer loads inside it")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
