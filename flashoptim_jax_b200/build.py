"""Builds libflashoptim_b200.so in-tree with nvcc for sm_100a.

The step-kernel family is split into ten instantiation slices (optimizer x state kind)
compiled from one source with different -D switches, so the build runs in parallel.
Objects go to csrc/build/, the library to lib/.  Nothing is compiled at import time:
call build_native() (or `python -m flashoptim_jax_b200.build`).
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from typing import List, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libflashoptim_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",  # a*b+c never contracts; the explicit __fmaf_rn calls stay FMAs
    "--ftz=false", "--prec-div=true", "--prec-sqrt=true",
    "-Xcompiler", "-fPIC,-ffp-contract=off,-O2",
]

# (object name, source, extra defines)
_OPTS = (("adam", "FO_OPT_ADAM"), ("lion", "FO_OPT_LION"), ("sgd", "FO_OPT_SGD"))
_KINDS = (("quant", 0), ("full", 1), ("generic", 3))


# block shape of a slice: (threads per block, resident blocks per SM).  Measured on B200: the plain
# Adam kernels run best as one 512-thread block per SM (all warps of an SM share one instruction
# stream and one set of tables); the kernels that also read peers' gradients keep 256-thread blocks,
# whose smaller stages leave room for a deeper copy pipeline.  Lion gains 2 % from one 768-thread block
# over three of 256; SGD measures the same either way and keeps the default (256 x 3).
_SHAPES = {("adam", 0): (512, 1), ("lion", 0): (768, 1)}


def _units(shapes=None, ffi_dir: str | None = None) -> List[Tuple[str, str, List[str]]]:
    shapes = _SHAPES if shapes is None else shapes
    units = [(name, name + ".cu", []) for name in ("fo_api", "fo_codec", "fo_selftest", "fo_norm")]
    if ffi_dir is not None:
        units.append(("fo_ffi", "fo_ffi.cc", ["-x", "cu", f"-I{ffi_dir}"]))

    def step_unit(oname: str, omacro: str, kname: str, kind: int, aux: int | None):
        suffix = "" if aux is None else ("_aux" if aux else "_plain")
        flags = [f"-DFO_INST_OPT={omacro}", f"-DFO_INST_KIND={kind}", f"-DFO_INST_AUX={aux or 0}",
                 f"-DFO_INST_NAME=lookup_{oname}_{kname}{suffix}"]
        shape = shapes.get((oname, aux))
        if shape is not None and kind != 3:
            flags += [f"-DFO_THREADS={shape[0]}", f"-DFO_MIN_BLOCKS_ADAM={shape[1]}", f"-DFO_MIN_BLOCKS_MOMENTUM={shape[1]}"]
            if len(shape) > 2:
                flags.append(f"-DFO_PLAIN_STAGES={shape[2]}")
        units.append((f"fo_step_{oname}_{kname}{suffix}", "fo_step_inst.cu", flags))

    for oname, omacro in _OPTS:
        for kname, kind in _KINDS:
            if kind == 3:
                step_unit(oname, omacro, kname, kind, None)
            else:
                for aux in (0, 1):
                    step_unit(oname, omacro, kname, kind, aux)
    for aux in (0, 1):
        step_unit("sgd", "FO_OPT_SGD", "none", 2, aux)
    return units


def ffi_include_dir() -> str | None:
    """Directory of jaxlib's XLA FFI headers (xla/ffi/api/ffi.h), or None when jax is not installed.
    The jax.ffi shim (csrc/fo_ffi.cc) is compiled into the library only when this resolves."""
    try:
        import jax.ffi  # noqa: PLC0415

        path = jax.ffi.include_dir()
    except Exception:  # jax absent, or too old to have jax.ffi
        return None
    return path if os.path.exists(os.path.join(path, "xla", "ffi", "api", "ffi.h")) else None


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libflashoptim_b200.so")
    return nvcc


def _sources_digest(extra: List[str], units=None) -> str:
    h = hashlib.sha256()
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for name in sorted(os.listdir(root)):
            if name.endswith((".cu", ".cuh", ".h", ".cc")):
                with open(os.path.join(root, name), "rb") as f:
                    h.update(name.encode())
                    h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + extra).encode())
    h.update(repr(units if units is not None else _units()).encode())
    return h.hexdigest()


def build_native(force: bool = False, jobs: int | None = None, extra_flags: List[str] | None = None,
                 lib_path: str = LIB_PATH, verbose: bool = False, shapes=None) -> str:
    """Compile every CUDA source for sm_100a and link the shared object; returns its path.
    `shapes` overrides the block shapes of the step slices ({(optimizer, aux): (threads, blocks per SM)})."""
    extra = list(extra_flags or [])
    units = _units(shapes, ffi_include_dir())
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(os.path.dirname(lib_path), exist_ok=True)
    stamp = lib_path + ".digest"
    digest = _sources_digest(extra, units)
    if not force and os.path.exists(lib_path) and os.path.exists(stamp) and open(stamp).read() == digest:
        return lib_path
    nvcc = _nvcc()
    tag = hashlib.sha256((" ".join(extra) + repr(shapes)).encode()).hexdigest()[:8] if (extra or shapes is not None) else "std"

    def compile_one(unit):
        name, src, defs = unit
        obj = os.path.join(OBJ_DIR, f"{name}.{tag}.o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, *defs, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {name}:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        if verbose and (r.stdout or r.stderr):
            print(f"[{name}]\n{r.stdout}{r.stderr}")
        return obj

    jobs = jobs or max(1, min(len(units), os.cpu_count() or 1))
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs) as pool:
        objs = list(pool.map(compile_one, units))
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib_path, *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(digest)
    return lib_path


if __name__ == "__main__":
    path = build_native(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
