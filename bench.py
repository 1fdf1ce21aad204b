"""Optimizer-step benchmark.  Default workload: Llama-3-8B-shaped pytree, flash AdamW with 32-bit
master weights.

    python bench.py --gpus N --steps K --warmup W            (this library)
    python bench.py --impl reference ...                     (the reference's CPU path, restated)

One step = one pass of the fused update over the whole pytree.  With N > 1 the step is
ZeRO-1 (launch with torchrun, one rank per GPU): reduce-scatter(mean) of the bf16 gradients,
the fused kernel on the rank's slice, all-gather of the updated parameters - both collectives
inside the kernel over NVLink by default, through NCCL with --nccl-reduce-scatter /
--nccl-allgather.
Inputs are synthetic (seeded normal draws with the configured shapes and scales).  The timed region
of K steps is repeated (--repeats, default 5) and the median repeat is reported; after it one more
step is checked against the CPU oracle on a sample of leaves.  Rank 0 prints ONE JSON line.

Other workloads (--workload): the ResNet-50 pytree under flash_sgdw and the GPT-2-small pytree under
flash_adamw / flash_lion (many small leaves; also timed through the public tx.step), a 1/64-scale
Llama pytree and one 2^26-element leaf (the small case profiler captures are taken on).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import random
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "optimizer-step params/sec"
UNIT = "params/s"

# DRAM bytes per parameter (dram__bytes_read.sum + dram__bytes_write.sum) of one profiler capture of each
# kernel on a 2^26-element bf16 leaf with bf16 gradients, keyed by (optimizer, ECC bits); traffic is
# proportional to the parameter count.  AdamW / int16 ECC: 917.4 MB per 67,108,864 parameters.
NCU_DRAM_BYTES_PER_PARAM = {("adamw", 16): 13.67, ("adamw", 8): 11.62, ("lion", 8): 9.56, ("sgdw", 8): 9.54}


def bytes_per_param(optimizer: str, param_bytes: int, ecc_bits: int, grad_bytes: int) -> float:
    """Algorithmic bytes of one in-place step per parameter (quantized moments, group size 32): the
    gradient is read; parameter, ECC, codes and fp16 group scales are read and written."""
    moments = 2 if optimizer in ("adamw", "adam") else 1
    state = param_bytes + ecc_bits / 8 + moments * (1 + 2 / 32)
    return grad_bytes + 2 * state


# ---- workloads ------------------------------------------------------------------------------------------
# a leaf: (shape, kind); kinds: "bf16" N(0, 0.02), "bf16_he" He-normal, "bf16_zeros", "f32_ones", "f32_zeros"


def llama3_8b_shapes():
    """Leaf shapes of the Llama-3-8B pytree: 291 leaves, 8,030,261,248 parameters."""
    shapes = {"tok_embeddings": ((128256, 4096), "bf16"), "lm_head": ((128256, 4096), "bf16"), "norm": ((4096,), "f32_ones")}
    for i in range(32):
        shapes.update(llama3_layer_shapes(i))
    return shapes


def llama3_layer_shapes(i: int):
    p = f"layers.{i:02d}."
    return {p + "wq": ((4096, 4096), "bf16"), p + "wk": ((4096, 1024), "bf16"), p + "wv": ((4096, 1024), "bf16"),
            p + "wo": ((4096, 4096), "bf16"), p + "w1": ((4096, 14336), "bf16"), p + "w3": ((4096, 14336), "bf16"),
            p + "w2": ((14336, 4096), "bf16"), p + "attention_norm": ((4096,), "f32_ones"), p + "ffn_norm": ((4096,), "f32_ones")}


def small_shapes():
    """A 1/64-scale pytree with the same leaf mix, for quick checks (not the benchmark workload)."""
    shapes = {"tok_embeddings": ((8192, 1024), "bf16"), "lm_head": ((8192, 1024), "bf16"), "norm": ((1024,), "f32_ones")}
    for i in range(8):
        p = f"layers.{i:02d}."
        for name, shp in (("wq", (1024, 1024)), ("wk", (1024, 256)), ("wv", (1024, 256)), ("wo", (1024, 1024)),
                          ("w1", (1024, 3584)), ("w3", (1024, 3584)), ("w2", (3584, 1024))):
            shapes[p + name] = (shp, "bf16")
        shapes[p + "attention_norm"] = ((1024,), "f32_ones")
        shapes[p + "ffn_norm"] = ((1024,), "f32_ones")
    return shapes


def one_leaf_shapes():
    """One 2^26-element bf16 leaf (0.96 GB touched per step): the small case profiler captures are taken on."""
    return {"w": ((8192, 8192), "bf16")}


def resnet50_shapes():
    """The 161 leaves of the reference's flax ResNet-50 (examples/train_imagenet.py:149-309): 53 HWIO
    convolution kernels (bf16, He-normal), 53 BatchNorm scale / bias pairs (fp32 vectors of 64..2048), the
    2048x1000 classifier (bf16) and its 1000-element fp32 bias; 25,557,032 parameters."""
    shapes = {"stem_conv/kernel": ((7, 7, 3, 64), "bf16_he"), "stem_bn/scale": ((64,), "f32_ones"), "stem_bn/bias": ((64,), "f32_zeros")}
    cin = 64
    for stage, (f, blocks) in enumerate(zip((64, 128, 256, 512), (3, 4, 6, 3)), start=1):
        for blk in range(blocks):
            p = f"layer{stage}_block{blk}/"
            for name, shp, width in (("conv1", (1, 1, cin, f), f), ("conv2", (3, 3, f, f), f), ("conv3", (1, 1, f, 4 * f), 4 * f)):
                shapes[p + name + "/kernel"] = (shp, "bf16_he")
                bn = "bn" + name[-1]
                shapes[p + bn + "/scale"] = ((width,), "f32_zeros" if bn == "bn3" else "f32_ones")  # zero_init_residual
                shapes[p + bn + "/bias"] = ((width,), "f32_zeros")
            if blk == 0:
                shapes[p + "proj_conv/kernel"] = ((1, 1, cin, 4 * f), "bf16_he")
                shapes[p + "proj_bn/scale"] = ((4 * f,), "f32_ones")
                shapes[p + "proj_bn/bias"] = ((4 * f,), "f32_zeros")
            cin = 4 * f
    shapes["fc/kernel"] = ((2048, 1000), "bf16_he")
    shapes["fc/bias"] = ((1000,), "f32_zeros")
    return shapes


def gpt2_small_shapes():
    """The 148 leaves of GPT-2 small in the un-stacked form: wte, wpe, 12 x (ln_1, c_attn, attn c_proj, ln_2,
    c_fc, mlp c_proj, each with its bias), ln_f; matrices bf16 N(0, 0.02), biases bf16 zeros, layer norms fp32;
    124,439,808 parameters."""
    shapes = {"wte": ((50257, 768), "bf16"), "wpe": ((1024, 768), "bf16")}
    for i in range(12):
        p = f"h.{i:02d}."
        shapes[p + "ln_1.scale"] = ((768,), "f32_ones")
        shapes[p + "ln_1.bias"] = ((768,), "f32_zeros")
        shapes[p + "attn.c_attn.w"] = ((768, 2304), "bf16")
        shapes[p + "attn.c_attn.b"] = ((2304,), "bf16_zeros")
        shapes[p + "attn.c_proj.w"] = ((768, 768), "bf16")
        shapes[p + "attn.c_proj.b"] = ((768,), "bf16_zeros")
        shapes[p + "ln_2.scale"] = ((768,), "f32_ones")
        shapes[p + "ln_2.bias"] = ((768,), "f32_zeros")
        shapes[p + "mlp.c_fc.w"] = ((768, 3072), "bf16")
        shapes[p + "mlp.c_fc.b"] = ((3072,), "bf16_zeros")
        shapes[p + "mlp.c_proj.w"] = ((3072, 768), "bf16")
        shapes[p + "mlp.c_proj.b"] = ((768,), "bf16_zeros")
    shapes["ln_f.scale"] = ((768,), "f32_ones")
    shapes["ln_f.bias"] = ((768,), "f32_zeros")
    return shapes


def _no_decay(path, _leaf) -> bool:
    """The reference's ImageNet recipe: no weight decay on biases and BatchNorm leaves
    (examples/train_imagenet.py make_weight_decay_matcher)."""
    last = str(path[-1])
    return last.endswith("bias") or "bn" in last


LLAMA_HP = dict(learning_rate=3e-4, b1=0.9, b2=0.999, eps=1e-8, weight_decay=0.1, master_weight_bits=32)
WORKLOADS = {
    # name: (shapes, optimizer, hyper-parameters, gradient sigma, outlier fraction)
    "llama3_8b": (llama3_8b_shapes, "adamw", LLAMA_HP, 1e-4, 0.0),
    "llama3_8b_div64": (small_shapes, "adamw", LLAMA_HP, 1e-4, 0.0),
    "adamw_leaf_64m": (one_leaf_shapes, "adamw", LLAMA_HP, 1e-4, 0.0),
    # the same single leaf under the other kernels (24-bit master weights), for their profiles
    "adamw24_leaf_64m": (one_leaf_shapes, "adamw", dict(LLAMA_HP, master_weight_bits=24), 1e-4, 0.0),
    "lion_leaf_64m": (one_leaf_shapes, "lion", dict(learning_rate=1e-4, b1=0.9, b2=0.99, weight_decay=1e-2, master_weight_bits=24), 1e-4, 0.0),
    "sgdw_leaf_64m": (one_leaf_shapes, "sgdw", dict(learning_rate=1e-2, momentum=0.9, weight_decay=1e-2, master_weight_bits=24), 1e-4, 0.0),
    # fp32 parameters and gradients (no ECC): the third kind of leaf the kernels take
    "adamw_f32_leaf_64m": (lambda: {"w": ((8192, 8192), "f32")}, "adamw", dict(LLAMA_HP, master_weight_bits=None), 1e-4, 0.0),
    "resnet50": (resnet50_shapes, "sgdw", dict(learning_rate=0.1, momentum=0.9, weight_decay=1e-4, master_weight_bits=24,
                                               param_groups=[{"params": _no_decay, "weight_decay": 0.0}]), 1e-3, 0.0),
    "gpt2_small": (gpt2_small_shapes, "adamw", dict(learning_rate=1e-3, b1=0.9, b2=0.999, eps=1e-8, weight_decay=1e-2,
                                                    master_weight_bits=24), 1e-3, 1e-4),
    "gpt2_small_lion": (gpt2_small_shapes, "lion", dict(learning_rate=1e-4, b1=0.9, b2=0.99, weight_decay=1e-2,
                                                        master_weight_bits=24), 1e-3, 1e-4),
}


def numel(shape):
    n = 1
    for d in shape:
        n *= d
    return n


def make_param(shape, kind, device, gen):
    import torch

    if kind == "bf16":
        return (torch.randn(shape, device=device, generator=gen) * 0.02).to(torch.bfloat16)
    if kind == "bf16_he":
        fan_in = numel(shape[:-1])
        return (torch.randn(shape, device=device, generator=gen) * math.sqrt(2.0 / fan_in)).to(torch.bfloat16)
    if kind == "bf16_zeros":
        return torch.zeros(shape, device=device, dtype=torch.bfloat16)
    if kind == "f32":
        return torch.randn(shape, device=device, generator=gen) * 0.02
    if kind == "f32_ones":
        return torch.ones(shape, device=device, dtype=torch.float32)
    if kind == "f32_zeros":
        return torch.zeros(shape, device=device, dtype=torch.float32)
    raise ValueError(kind)


def fill_grad(g, sigma, outliers, gen):
    """g <- N(0, sigma) in g's dtype, a fraction `outliers` of the entries scaled by 100."""
    import torch

    x = torch.randn(g.shape, device=g.device, generator=gen) * sigma
    if outliers > 0:
        x = torch.where(torch.rand(g.shape, device=g.device, generator=gen) < outliers, x * 100.0, x)
    g.copy_(x.to(g.dtype))


def json_hparams(hp):
    return {k: (v if not callable(v) and k != "param_groups" else "see bench.py") for k, v in hp.items()}


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
        sm, mx, power, reasons = [], [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(power) if power else None}


# ---- CPU legs (the only places that execute oracle/) -----------------------------------------------------


def cpu_baseline(steps: int):
    """The reference's CPU (unfused) path, restated in C with OpenMP on every host core, on a bounded sample
    of the Llama workload: the nine leaves of one transformer layer (218,120,192 of the 8,030,261,248
    parameters: seven bf16 matrices with int16 ECC, two fp32 norm vectors)."""
    import numpy as np

    from oracle import c_oracle as C
    from oracle import driver as D
    from oracle import flashoptim_oracle as O

    C.build()
    cores = C.set_threads(os.cpu_count() or 1)  # explicitly: torchrun exports OMP_NUM_THREADS=1
    rng = np.random.default_rng(0)
    leaves = []
    for _, (shape, kind) in llama3_layer_shapes(0).items():
        n = numel(shape)
        if kind == "bf16":
            p = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)).astype(D.BF16)
            g = (rng.standard_normal(n, dtype=np.float32) * np.float32(1e-4)).astype(D.BF16)
            leaves.append((D.fresh_leaf(p, C.ADAM, C.STATE_QUANT, 16), g))
        else:
            p = np.ones(n, dtype=np.float32)
            g = rng.standard_normal(n, dtype=np.float32) * np.float32(1e-4)
            leaves.append((D.fresh_leaf(p, C.ADAM, C.STATE_QUANT, 0), g))
    n_params = sum(g.size for _, g in leaves)
    times = []
    for t in range(1, steps + 2):
        hp = D.hyper_tuple(C.ADAM, O.UNFUSED, t, lr=LLAMA_HP["learning_rate"], wd=LLAMA_HP["weight_decay"])
        t0 = time.perf_counter()
        for leaf, g in leaves:
            D.oracle_step(C.ADAM, g, leaf, C.STATE_QUANT, 32, hp)
        times.append(time.perf_counter() - t0)
    times = times[1:]  # the first pass pages memory in
    per_step = sorted(times)[len(times) // 2]
    return {"value": n_params / per_step, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"one of the 32 transformer layers of the Llama-3-8B pytree (9 leaves, {n_params} parameters), "
                      f"{len(times)} steps, C restatement of the reference's CPU path with OpenMP"}, per_step


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    shapes_fn, _, hp, _, _ = WORKLOADS["llama3_8b"]
    shapes = shapes_fn()
    base, per_step = cpu_baseline(max(1, args.steps))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "llama3_8b", "leaves": len(shapes), "params": sum(numel(s) for s, _ in shapes.values()),
                   "optimizer": "flash_adamw", **json_hparams(hp), "grad_dtype": "bf16"},
        "reference_is": "the reference's CPU (fused=False) path as its C / OpenMP restatement (oracle/, pinned bit for bit on the "
                        "reference's own source text run over a NumPy stand-in for jax); JAX itself is not installable here, so "
                        "no number of the live JAX CPU path exists",
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---- checker: one more step on the device against the CPU oracle, on a sample of leaves ------------------


def parity_check(zero, device):
    """Runs one more optimizer step and recomputes it with the C oracle for a sample of this rank's
    segments (the first, the last and the largest of every dtype bucket; for long ones a window at either
    end): every stored array must match bit for bit.  The gradients of the benchmark are the same on every
    rank, so their mean is each rank's own gradient, whatever the route and order of the reduction."""
    import numpy as np
    import torch

    from oracle import c_oracle as C
    from oracle import driver as D
    from oracle import flashoptim_oracle as O

    from flashoptim_jax_b200 import _lib, utils
    from flashoptim_jax_b200.zero1 import flat_position

    C.build()
    C.set_threads(os.cpu_count() or 1)
    window = 1 << 20
    samples = []
    for b, layout in enumerate(zero.buckets):
        segs = layout.segments[zero.rank]
        if not segs:
            continue
        pick = {0, len(segs) - 1, max(range(len(segs)), key=lambda s: segs[s].hi - segs[s].lo)}
        shapes_seen = set()
        for s, seg in enumerate(segs):  # one segment per distinct leaf shape as well
            shp = zero.shapes[seg.leaf]
            if shp not in shapes_seen:
                shapes_seen.add(shp)
                pick.add(s)
        for s in sorted(pick):
            n = segs[s].hi - segs[s].lo
            spans = [(0, n)] if n <= 2 * window else [(0, window), ((n - window) // 32 * 32, n)]
            for lo, hi in spans:
                samples.append((b, s, lo, hi))

    def snap(b, s, lo, hi):
        layout = zero.buckets[b]
        seg = layout.segments[zero.rank][s]
        st = zero.state[(b, s)]
        at = flat_position(layout, zero.rank, seg.offset)
        glo, ghi = lo // 32, -(-hi // 32)
        arr = lambda t, a, z: None if t is None else D.to_numpy(t[a:z])
        return D.LeafArrays(arr(zero.flat_params[b], at + lo, at + hi), arr(st.ecc, lo, hi), arr(st.mu, lo, hi), arr(st.mu_scales, glo, ghi),
                            arr(st.nu, lo, hi), arr(st.nu_scales, glo, ghi)), D.to_numpy(zero.flat_grads[b][at + lo:at + hi])

    def mean_as_the_kernel_forms_it(g):
        """Equal gradients on all ranks: the fused reduce-scatter adds them in fp32 (own value first, then the
        peers), divides by the rank count and rounds once to the gradient dtype.  k * g is exact for 16-bit
        gradients (k <= 8), so the mean is g itself; an fp32 sum of fp32 values rounds at every addition from
        the third on, and the last place of the mean can differ from g's."""
        if zero.world_size <= 2 or g.dtype != np.float32:
            return g
        acc = g.copy()
        for _ in range(zero.world_size - 1):
            acc = (acc + g).astype(np.float32)
        return (acc / np.float32(zero.world_size)).astype(np.float32)

    if zero.world_size > 2 and not zero.fused_reduce_scatter:
        # NCCL's order of additions is its own: fp32 buckets cannot be predicted to the bit
        samples = [x for x in samples if zero.buckets[x[0]].dtype != torch.float32]
    before = [snap(*x) for x in samples]
    count = zero.count + 1
    zero.step()
    torch.cuda.synchronize(device)
    mismatches, elements, detail = 0, 0, []
    for (b, s, lo, hi), (leaf, grad) in zip(samples, before):
        seg = zero.buckets[b].segments[zero.rank][s]
        config = zero.configs[seg.leaf]
        lr = utils._resolve_learning_rate(config["learning_rate"], torch.tensor(count - 1, dtype=torch.int32))
        hp = zero._hyper(config, lr, count)
        st = zero.state[(b, s)]
        state = C.STATE_NONE if st.mu is None else (C.STATE_QUANT if config["quantize"] else C.STATE_FULL)
        opt = {_lib.FO_OPT_ADAM: C.ADAM, _lib.FO_OPT_LION: C.LION, _lib.FO_OPT_SGD: C.SGD}[zero.opt_code]
        D.oracle_step(opt, mean_as_the_kernel_forms_it(grad), leaf, state, 32, hp)
        got, _ = snap(b, s, lo, hi)
        elements += hi - lo
        for f in leaf.fields():
            a, w = getattr(got, f), getattr(leaf, f)
            if a is None:
                continue
            bad = int(np.count_nonzero(D.bits(a).ravel() != D.bits(w).ravel()))
            if bad:
                mismatches += bad
                detail.append(f"leaf {seg.leaf} [{seg.lo + lo}:{seg.lo + hi}) {f}: {bad}")
    out = {"leaves": len({(b, s) for b, s, _, _ in samples}), "windows": len(samples), "elements": elements, "mismatches": mismatches,
           "against": "C oracle (reference's fused-kernel text), bit for bit, one step after the timed region"}
    if detail:
        out["detail"] = detail[:8]
    return out


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


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def run_ours(args):
    quiet_stdout()
    import torch
    import torch.distributed as dist

    from flashoptim_jax_b200 import _engine as eng
    from flashoptim_jax_b200 import tree as pytree
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

    shapes_fn, optimizer, hparams, sigma, outliers = WORKLOADS[args.workload]
    shapes = shapes_fn()
    total_params = sum(numel(s) for s, _ in shapes.values())
    gen = torch.Generator(device=device)
    gen.manual_seed(1234)  # same draws on every rank: parameters are replicated
    params = {name: make_param(shape, kind, device, gen) for name, (shape, kind) in shapes.items()}

    pending = []   # (bucket key, params in the launch, event, event): one entry per fo_step call
    launches = [0]

    class TimedLaunch:
        def __init__(self, key, n_params):
            self.key, self.n = key, n_params

        def __enter__(self):
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.e0.record()

        def __exit__(self, *exc):
            self.e1.record()
            pending.append((self.key, self.n, self.e0, self.e1))
            launches[0] += 1
            return False

    eng.set_launch_observer(TimedLaunch)

    # N >= 4: both collectives through the NVLink switch unless asked otherwise (see --no-switch)
    use_switch = world >= 4 and not args.no_switch and not args.nccl_allgather and not args.nccl_reduce_scatter and args.clip is None
    fused = {"fused_allgather": world > 1 and not args.nccl_allgather,
             "fused_reduce_scatter": world > 1 and not args.nccl_reduce_scatter and args.clip is None}
    try:
        zero = Zero1Optimizer(optimizer, params, max_grad_norm=args.clip, n_slices=args.slices,
                              use_switch=use_switch, **fused, **hparams)
    except Exception as e:  # no peer-mapped (symmetric) memory or no multicast mapping on this system: every rank fails alike
        if not any(fused.values()):
            raise
        print(f"fused collectives unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
        args.nccl_allgather = args.nccl_reduce_scatter = True
        use_switch = False
        fused = {"fused_allgather": False, "fused_reduce_scatter": False}
        zero = Zero1Optimizer(optimizer, params, max_grad_norm=args.clip, n_slices=args.slices, **hparams)
    public_params = params if (args.public_api and world == 1) else None
    del params
    torch.cuda.empty_cache()
    ggen = torch.Generator(device=device)
    # The same draw on every rank: the averaged gradient of the N-rank job then equals the
    # gradient of the 1-rank job (strong scaling of one problem).  Different fixed draws per rank
    # would average to exact zeros at about 7e-4 of the positions, the same ones every step, which
    # no training run with fresh gradients per step has.
    ggen.manual_seed(99)
    for g in pytree.tree_leaves(zero.grads):
        fill_grad(g, sigma, outliers, ggen)
    if args.zero_rows > 0 and "tok_embeddings" in shapes:
        # untouched embedding rows: a fixed fraction of the rows of tok_embeddings never sees a gradient
        g = zero.grads["tok_embeddings"]
        rows = torch.rand(g.shape[0], device=device, generator=ggen) < args.zero_rows
        g[rows] = 0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, repeats):
        """`repeats` regions of `steps` calls, each bracketed by a barrier and a synchronize; per-region ms per
        step, max over ranks."""
        out = []
        for _ in range(repeats):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1) / steps
            if world > 1:
                t = torch.tensor([ms], device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t)
            out.append(ms)
        return out

    for _ in range(args.warmup):
        zero.step()
    barrier()
    pending.clear()
    launches[0] = 0
    sampler = ClockSampler(local_rank)
    sampler.start()
    region_ms = timed(zero.step, args.steps, args.repeats)
    clocks = sampler.stop()
    n_launch = launches[0] // args.repeats
    if args.clip is not None:
        n_launch += 2 * len(zero.buckets) * args.steps  # fo_sq_norm: partial sums and their fixed-order total, per dtype
    ms_per_step = median(region_ms)
    value = total_params / (ms_per_step * 1e-3)
    kernel_ms = {}
    for bucket, n_par, a, b in pending:
        kernel_ms.setdefault(bucket, []).append((n_par, a.elapsed_time(b)))

    # N > 1: the three legs of the step, each timed on its own
    legs = None
    if world > 1 and not args.no_legs:
        legs = {}
        pending.clear()
        k_ms = median(timed(lambda: zero.step(phases=("step",)), args.steps, 3))
        for bucket, n_par, a, b in pending:
            kernel_ms.setdefault(("local",) + bucket, []).append((n_par, a.elapsed_time(b)))
        legs["step_kernel_only"] = {"ms_per_step": k_ms, "value": total_params / (k_ms * 1e-3), "unit": UNIT,
                                    "note": "each rank's kernel on its own slice with its own gradients, no collective; aggregate over ranks"}
        ag_ms = median(timed(lambda: zero.step(phases=("step", "all_gather")), args.steps, 3))
        legs["step_and_allgather"] = {"ms_per_step": ag_ms, "value": total_params / (ag_ms * 1e-3), "unit": UNIT}
        rs_ms = median(timed(lambda: zero.step(phases=("reduce_scatter", "step")), args.steps, 3))
        legs["reducescatter_and_step"] = {"ms_per_step": rs_ms, "value": total_params / (rs_ms * 1e-3), "unit": UNIT,
                                          "note": "replicas are left stale by this leg and gathered again after it"}
        legs["full_step"] = {"ms_per_step": ms_per_step, "value": value, "unit": UNIT}
        zero.all_gather_params()  # the replicas agree again
        barrier()

    # roofline of the dominant kernel (the launch with the most parameters), from its own CUDA-event durations:
    # at N > 1 that of the kernel alone on the local slice (the fused step is bound by the links, see "nvlink")
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    else:
        peak, peak_src = 6650.0, "fallback"
    pool = {k: v for k, v in kernel_ms.items() if (k[0] == "local") == (world > 1 and legs is not None)}
    top = max(pool, key=lambda k: pool[k][0][0]) if pool else None
    roofline = None
    if top is not None:
        bucket = top[1:] if top[0] == "local" else top
        n_par = pool[top][0][0]
        avg_ms = sum(ms for _, ms in pool[top]) / len(pool[top])
        psize = 4 if bucket[1] == 0 else 2
        bpp = bytes_per_param(optimizer, psize, bucket[3], 4 if bucket[2] == 0 else 2)
        achieved = n_par * bpp / (avg_ms * 1e-3) / 1e9
        captured = NCU_DRAM_BYTES_PER_PARAM.get((optimizer, bucket[3])) if bucket[1] == 1 and bucket[2] == 1 else None
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": captured * n_par if captured is not None else None,
                    "kernel": f"step_kernel<{optimizer}, {'f32' if bucket[1] == 0 else ('bf16' if bucket[1] == 1 else 'f16')}, ecc{bucket[3]}, quant>",
                    "params_per_launch": n_par, "avg_launch_ms": avg_ms, "launches_timed": len(pool[top]),
                    "algorithmic_bytes_per_param": bpp, "peak_source": peak_src}
        if world > 1:
            roofline["note"] = "the step kernel alone on this rank's slice (leg step_kernel_only); the whole ZeRO-1 step is link-bound, see nvlink"

    parity = None
    if not args.no_parity:
        parity = parity_check(zero, device)
        if parity.get("detail"):
            print(f"rank {rank}: parity mismatches: {parity['detail']}", file=sys.stderr)
        if world > 1:
            t = torch.tensor([parity["mismatches"], parity["elements"], parity["leaves"]], device=device, dtype=torch.int64)
            dist.all_reduce(t)
            parity.update(mismatches=int(t[0]), elements=int(t[1]), leaves=int(t[2]), ranks_checked=world)

    e2e = None
    if not args.no_e2e:
        e2e = measure_e2e(args, zero, device, ggen, world, barrier, total_params, sigma)
    public = None
    if public_params is not None:
        public = measure_public_api(optimizer, hparams, public_params, zero, args, sigma, outliers)
    link_bytes = (sum(g.numel() * g.element_size() for g in pytree.tree_leaves(zero.grads))
                  + sum(q.numel() * q.element_size() for q in pytree.tree_leaves(zero.params)))
    zero_info = {"mc": list(zero.mc_param_offsets) + list(zero.mc_grad_offsets)}

    if rank == 0:
        base = None
        if world == 1 and not args.no_cpu_baseline:
            base, _ = cpu_baseline(3)
        sm_mhz = clocks.get("sm_mhz")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": args.workload, "leaves": len(shapes), "params": total_params, "optimizer": "flash_" + optimizer,
                       **json_hparams(hparams), "grad_dtype": "bf16 (fp32 for fp32 leaves)", "grad_sigma": sigma, "grad_outliers": outliers,
                       "zero_rows": args.zero_rows or None,
                       "parallelism": "single" if world == 1 else f"zero1x{world}",
                       "reduce_scatter": None if world == 1 else ("nccl" if not fused["fused_reduce_scatter"] else "fused into the step kernel"),
                       "allgather": None if world == 1 else ("nccl" if not fused["fused_allgather"] else "fused into the step kernel"),
                       "route": None if world == 1 else ("NVLink switch (multimem.st / multimem.ld_reduce)" if any(zero_info["mc"]) else "point to point (peer loads / stores)"),
                       "clip_global_norm": args.clip, "slices": args.slices,
                       "l2": "working set per step (>= 10 B/param) exceeds the 126 MB L2, no flush needed"},
            "repeats": {"regions": len(region_ms), "ms_per_step": region_ms, "median": ms_per_step, "max": max(region_ms), "min": min(region_ms)},
            "cycles_per_element": None if not sm_mhz else ms_per_step * 1e-3 * sm_mhz * 1e6 / (total_params / world),
            "roofline": roofline, "cpu_baseline": base, "e2e": e2e, "gpu_launches": n_launch, "clocks": clocks,
            "parity_check": parity,
        }
        if legs is not None:
            line["legs"] = legs
        if public is not None:
            line["public_api"] = public
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


SQUARE_SIZES = (256, 512, 1024, 2048, 4096, 8192, 16384)
SQUARE_HP = {"adamw": dict(learning_rate=1e-3, b1=0.9, b2=0.999, eps=1e-8, weight_decay=1e-2),
             "lion": dict(learning_rate=1e-4, b1=0.9, b2=0.99, weight_decay=1e-2),
             "sgdw": dict(learning_rate=1e-2, momentum=0.9, weight_decay=1e-2)}


def percentile(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(math.ceil(q * len(xs))) - 1)]


def square_graph_samples(optimizer, hparams, n, k, n_samples, device, gen, rng):
    """The same case through the functional surface with the step's scalars formed on the device
    (capturable=True): k calls of tx.step captured in one CUDA graph, one replay per sample."""
    import torch

    import flashoptim_jax_b200 as fo

    factory = {"adamw": fo.flash_adamw, "lion": fo.flash_lion, "sgdw": fo.flash_sgdw}[optimizer]
    lr = torch.tensor(float(hparams["learning_rate"]), dtype=torch.float32, device=device)
    tx = factory(**dict(hparams, learning_rate=lr), donate=True, capturable=True)
    params = {"w": make_param((n, n), "bf16", device, gen)}
    grads = {"w": torch.empty_like(params["w"])}
    fill_grad(grads["w"], 1e-3, 1e-4, gen)
    state = tx.init(params)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # eager once: moves the counter to the device, loads the kernels
        for _ in range(5):
            params, state = tx.step(params, state, grads)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(k):
            params, state = tx.step(params, state, grads)
    samples = []
    for it in range(-1, n_samples):
        fill_grad(grads["w"], 10.0 ** rng.uniform(-4.0, -1.0), 1e-4, gen)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        if it >= 0:
            samples.append(e0.elapsed_time(e1) / k)
    del graph
    return samples


def run_square_sweep(args):
    """The square-matrix sweep of the reference's step benchmark (examples/benchmark_square_step_all.sh:7-12,
    examples/benchmark_step.py:144-157): one bf16 N x N parameter, N = 256 .. 16384, under flash_adamw / flash_lion /
    flash_sgdw with 24- and 32-bit master weights; bf16 gradients N(0, sigma) with sigma log-uniform in
    [1e-4, 1e-1] redrawn for every sample and 0.01 % of the entries scaled by 100.  Protocol as the reference's:
    5 warm-up steps, then samples of k back-to-back steps between synchronisations, CUDA events around the k
    steps, median and 95th percentile over the samples; 100 timed steps per case.  One JSON line: the headline
    value is the largest AdamW case with 32-bit master weights, every case is listed under "sweep"."""
    quiet_stdout()
    import torch

    from flashoptim_jax_b200 import tree as pytree
    from flashoptim_jax_b200.zero1 import Zero1Optimizer

    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise SystemExit("the square sweep is a single-GPU workload")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    else:
        peak, peak_src = 6650.0, "fallback"
    k, n_samples = 10, 10
    rng = random.Random(7)
    sampler = ClockSampler(0)
    sampler.start()
    sweep, launches = [], 0
    primer = Zero1Optimizer("adamw", {"w": make_param((4096, 4096), "bf16", device, torch.Generator(device=device))}, **SQUARE_HP["adamw"])
    for _ in range(500):  # first use of the library in this process: module loading, allocator, and the clocks leave idle
        primer.step()
    torch.cuda.synchronize()
    del primer
    for optimizer in ("adamw", "lion", "sgdw"):
        for mwb in (24, 32):
            for n in SQUARE_SIZES:
                gen = torch.Generator(device=device)
                gen.manual_seed(n + mwb)
                hparams = dict(SQUARE_HP[optimizer], master_weight_bits=mwb)
                zero = Zero1Optimizer(optimizer, {"w": make_param((n, n), "bf16", device, gen)}, **hparams)
                g = zero.grads["w"]
                samples = []
                for it in range(-1, n_samples):  # sample -1: the warm-up steps
                    fill_grad(g, 10.0 ** rng.uniform(-4.0, -1.0), 1e-4, gen)
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(5 if it < 0 else k):
                        zero.step()
                    e1.record()
                    torch.cuda.synchronize()
                    if it >= 0:
                        samples.append(e0.elapsed_time(e1) / k)
                        launches += k
                bpp = bytes_per_param(optimizer, 2, 8 if mwb == 24 else 16, 2)
                ms = median(samples)
                case = {"optimizer": "flash_" + optimizer, "n": n, "master_weight_bits": mwb, "params": n * n,
                        "ms_per_step": ms, "ms_per_step_p95": percentile(samples, 0.95), "params_per_s": n * n / (ms * 1e-3),
                        "gb_per_s": n * n * bpp / (ms * 1e-3) / 1e9, "frac_of_peak": n * n * bpp / (ms * 1e-3) / 1e9 / peak,
                        "l2_resident": n * n * bpp < 126e6}
                if not args.no_parity:
                    chk = parity_check(zero, device)
                    case["parity_mismatches"] = chk["mismatches"]
                    if chk.get("detail"):
                        print(f"{optimizer} {n} mwb {mwb}: parity mismatches: {chk['detail']}", file=sys.stderr)
                del zero, g
                torch.cuda.empty_cache()
                graph_samples = square_graph_samples(optimizer, hparams, n, k, n_samples, device, gen, rng)
                launches += k * n_samples
                case["cuda_graph"] = {"ms_per_step": median(graph_samples), "ms_per_step_p95": percentile(graph_samples, 0.95),
                                      "params_per_s": n * n / (median(graph_samples) * 1e-3)}
                sweep.append(case)
                torch.cuda.empty_cache()
    clocks = sampler.stop()
    head = next(c for c in sweep if c["optimizer"] == "flash_adamw" and c["master_weight_bits"] == 32 and c["n"] == SQUARE_SIZES[-1])
    emit({
        "metric": METRIC, "value": head["params_per_s"], "unit": UNIT, "n_gpus": 1, "steps": k * n_samples, "warmup": 5,
        "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "square_sweep", "headline": "flash_adamw, 16384 x 16384 bf16, 32-bit master weights",
                   "sizes": list(SQUARE_SIZES), "optimizers": ["flash_adamw", "flash_lion", "flash_sgdw"], "master_weight_bits": [24, 32],
                   "hparams": SQUARE_HP, "grad_dtype": "bf16", "grad_sigma": "log-uniform in [1e-4, 1e-1] per sample", "grad_outliers": 1e-4,
                   "protocol": f"5 warm-up steps, {n_samples} samples of {k} back-to-back steps, median and p95 over the samples; "
                               "cuda_graph: the same k steps as one captured graph of tx.step calls (scalars formed on the device)",
                   "l2": "cases marked l2_resident touch less than the 126 MB L2 per step and run from it (no flush): their GB/s is "
                         "not an HBM figure; the others exceed L2"},
        "roofline": {"bound": "hbm", "achieved": head["gb_per_s"], "peak": peak, "unit": "GB/s", "frac": head["frac_of_peak"],
                     "traffic": NCU_DRAM_BYTES_PER_PARAM[("adamw", 16)] * head["params"], "kernel": "step_kernel<adamw, bf16, ecc16, quant>",
                     "params_per_launch": head["params"], "avg_launch_ms": head["ms_per_step"], "peak_source": peak_src,
                     "algorithmic_bytes_per_param": bytes_per_param("adamw", 2, 16, 2)},
        "cpu_baseline": None, "e2e": None, "gpu_launches": launches, "clocks": clocks,
        "parity_check": None if args.no_parity else {"cases": len(sweep), "mismatches": sum(c["parity_mismatches"] for c in sweep),
                                                     "against": "C oracle (reference's fused-kernel text), bit for bit, one step after each case's timed steps"},
        "sweep": sweep,
    })



def measure_public_api(optimizer, hparams, params, zero, args, sigma, outliers):
    """The same step through the public surface, tx.init / tx.step with donated buffers (what a user of the
    reference's API calls), host cost of flattening and table building included."""
    import torch

    import flashoptim_jax_b200 as fo
    from flashoptim_jax_b200 import tree as pytree

    factory = {"adamw": fo.flash_adamw, "adam": fo.flash_adam, "lion": fo.flash_lion, "sgd": fo.flash_sgd, "sgdw": fo.flash_sgdw}[optimizer]
    tx = factory(**hparams, donate=True)
    state = tx.init(params)
    grads = pytree.tree_map(lambda g: g.clone(), zero.grads)
    for _ in range(3):
        params, state = tx.step(params, state, grads)
    torch.cuda.synchronize()
    samples = []
    for _ in range(args.repeats):
        t0 = time.perf_counter()
        for _ in range(args.steps):
            params, state = tx.step(params, state, grads)
        torch.cuda.synchronize()
        samples.append((time.perf_counter() - t0) / args.steps * 1e3)
    out = {"ms_per_step": median(samples), "all": samples, "note": "tx.step(params, state, grads) with donate=True, wall clock including the host side"}
    # the same steps with the scalars formed on the device, captured once as a CUDA graph and replayed
    lr = torch.tensor(float(hparams["learning_rate"]), dtype=torch.float32, device=grads[next(iter(grads))].device)
    tx = factory(**dict(hparams, learning_rate=lr), donate=True, capturable=True)
    state = tx.init(params)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            params, state = tx.step(params, state, grads)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(args.steps):
            params, state = tx.step(params, state, grads)
    graph.replay()
    torch.cuda.synchronize()
    replays = []
    for _ in range(args.repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        replays.append(e0.elapsed_time(e1) / args.steps)
    out["cuda_graph"] = {"ms_per_step": median(replays), "all": replays,
                         "note": f"{args.steps} calls of tx.step(capturable=True) captured in one CUDA graph, one replay per sample, CUDA events"}
    return out


def measure_e2e(args, zero, device, ggen, world, barrier, total_params, sigma):
    """End to end through the public API with gradients arriving from pinned host memory every step."""
    import torch
    import torch.distributed as dist

    from flashoptim_jax_b200 import tree as pytree

    e2e_steps = max(1, min(args.steps, 2))
    grad_leaves = pytree.tree_leaves(zero.grads)
    # pinned host gradients: every leaf is a window of one staging buffer (the values repeat; 16 GB of
    # pinned memory per rank would be needed otherwise), fp32 leaves of a small one
    big16 = [g.numel() for g in grad_leaves if g.dtype != torch.float32]
    big32 = [g.numel() for g in grad_leaves if g.dtype == torch.float32]
    stage_elems = max([1 << 22] + big16) if total_params < (1 << 28) else max([1 << 28] + big16)
    stage = torch.empty(stage_elems, dtype=torch.bfloat16, pin_memory=True)
    fill = 1 << 26
    for lo in range(0, stage_elems, fill):
        m = min(fill, stage_elems - lo)
        stage[lo:lo + m].copy_((torch.randn(m, device=device, generator=ggen) * sigma).to(torch.bfloat16).cpu())
    stage32 = torch.full((max([1] + big32),), sigma, dtype=torch.float32).pin_memory()
    host_leaves, off = [], 0
    for g in grad_leaves:
        n = g.numel()
        if g.dtype == torch.float32:
            host_leaves.append(stage32[:n].view(g.shape))
            continue
        if off + n > stage_elems:
            off = 0
        host_leaves.append(stage[off:off + n].view(g.dtype).view(g.shape))
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
            "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
            "note": "gradients come from pinned host memory every step; the updated parameters and the optimizer state stay on the "
                    "device by design (their consumer is the next forward pass), so only a 4-byte probe of the result is read back"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the median region is reported")
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["square_sweep"], default="llama3_8b")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (used for profiler captures)")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of one more step after the timed region")
    ap.add_argument("--no-legs", action="store_true", help="N > 1: skip the separate timings of kernel only / kernel + all-gather")
    ap.add_argument("--public-api", action="store_true", help="N = 1: also time the step through tx.init / tx.step")
    ap.add_argument("--zero-rows", type=float, default=0.0,
                    help="fraction of the rows of tok_embeddings whose gradient is exactly zero on every step (untouched embedding rows)")
    ap.add_argument("--nccl-allgather", action="store_true", help="N > 1: NCCL all-gather after the step instead of stores inside it")
    ap.add_argument("--nccl-reduce-scatter", action="store_true", help="N > 1: NCCL reduce-scatter before the step instead of loads inside it")
    ap.add_argument("--no-switch", action="store_true",
                    help="N >= 4: keep the fused collectives on point-to-point peer loads / stores instead of the NVLink switch")
    ap.add_argument("--slices", type=int, default=None,
                    help="N > 1 with both NCCL collectives: slices per bucket whose reduce-scatter / step / all-gather overlap")
    ap.add_argument("--clip", type=float, default=None,
                    help="clip the gradients at this global norm inside the step (adds the sum-of-squares sweep; off by default)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    args.repeats = max(1, args.repeats)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "square_sweep":
        run_square_sweep(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
