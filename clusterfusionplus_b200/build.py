"""Build libclusterfusion_b200.so in-tree with nvcc for sm_100a.

    python clusterfusionplus_b200/build.py [--force] [--verbose]

Four translation units, compiled separately (objects cached under lib/obj/) and linked into one
shared library: the decode kernel with the C ABI, the batched Llama decode blocks (hand-written
tcgen05 skinny GEMMs + paged attention), the elementwise kernels of the prompt pass, and the tensor-core prefill
GEMM, which is built from the CUTLASS / CuTe headers found in the Python environment (the `flashinfer` wheel
vendors them; set CUTLASS_INCLUDE to use another copy).  The library has no torch dependency;
it links the CUDA runtime statically and finds the driver's tensor-map encoder at run time.
"""
from __future__ import annotations

import importlib.util
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
HEADER = os.path.join(os.path.dirname(HERE), "include", "clusterfusion_b200.h")
OUT = os.path.join(HERE, "lib", "libclusterfusion_b200.so")
OBJ = os.path.join(HERE, "lib", "obj")

# source -> (dependencies besides itself, needs the CUTLASS headers)
UNITS = {
    "capi.cu": (["decode_kernel.cuh", "pipeline.cuh", "dsm.cuh", "prefill_gemm.h", "host_common.h", HEADER], False),
    "llama_batch.cu": (["llama_batch_kernel.cuh", "pipeline.cuh", "host_common.h", HEADER], False),
    "prefill_gemm.cu": (["prefill_gemm.h"], True),
    "prefill_ops.cu": (["host_common.h", HEADER], False),
}
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def cutlass_includes() -> list:
    """Include directories of a CUTLASS tree that has the sm_100 collectives."""
    roots = []
    if os.environ.get("CUTLASS_INCLUDE"):
        roots.append(os.path.dirname(os.environ["CUTLASS_INCLUDE"].rstrip("/")))
    spec = importlib.util.find_spec("flashinfer")
    if spec and spec.submodule_search_locations:
        roots.append(os.path.join(list(spec.submodule_search_locations)[0], "data", "cutlass"))
    for root in roots:
        inc = os.path.join(root, "include")
        if os.path.exists(os.path.join(inc, "cutlass", "gemm", "collective", "collective_builder.hpp")):
            dirs = [inc]
            util = os.path.join(root, "tools", "util", "include")
            if os.path.isdir(util):
                dirs.append(util)
            return dirs
    raise RuntimeError("CUTLASS headers not found: set CUTLASS_INCLUDE to <cutlass>/include")


def _deps(src: str) -> list:
    extra, _ = UNITS[src]
    return [os.path.join(CSRC, src)] + [d if os.path.isabs(d) else os.path.join(CSRC, d) for d in extra]


def _stale(target: str, deps: list) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    cmd = [nvcc_path(), *ARCH, "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-c", "-o", obj,
           os.path.join(CSRC, src)]
    if UNITS[src][1]:
        cmd += ["--expt-relaxed-constexpr"] + [f"-I{d}" for d in cutlass_includes()]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}")
    return obj


def up_to_date() -> bool:
    return not _stale(OUT, [d for s in UNITS for d in _deps(s)])


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return OUT
    os.makedirs(OBJ, exist_ok=True)
    todo = [s for s in UNITS if force or _stale(os.path.join(OBJ, s.replace(".cu", ".o")), _deps(s))]
    with ThreadPoolExecutor(max_workers=len(UNITS)) as ex:
        list(ex.map(lambda s: _compile(s, verbose), todo))
    objs = [os.path.join(OBJ, s.replace(".cu", ".o")) for s in UNITS]
    r = subprocess.run([nvcc_path(), *ARCH, "-shared", "-o", OUT, *objs], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("linking libclusterfusion_b200.so failed")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
