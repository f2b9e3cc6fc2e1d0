"""In-tree build of libhtree_b200.so with nvcc for sm_100a (cross-compiles without a GPU).

    python -m htree_b200.build [--force] [--verbose]

The library is written next to this file so that it travels with the source tree; nothing is installed.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libhtree_b200.so")
PROBES_LIB = os.path.join(HERE, "libhtree_b200_probes.so")    # measurement aids of the benchmark (csrc/bench/), not the operator
OBJ_DIR = os.path.join(HERE, "build")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put the CUDA toolkit on PATH")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, defines=(), out: str = LIB, obj_dir: str = OBJ_DIR) -> str:
    """Compile every .cu under csrc/ and link the shared library.  Returns its path.
    `defines` (e.g. ["HTREE_FWD_MIN_BLOCKS=3"]) with a separate `out`/`obj_dir` builds a tuning variant of the same ABI."""
    nvcc = _nvcc()
    LIB_, OBJ_DIR_ = out, obj_dir
    os.makedirs(OBJ_DIR_, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "htree_b200.h"))
    srcs = sources()
    objs = [os.path.join(OBJ_DIR_, os.path.basename(s)[:-3] + ".o") for s in srcs]
    dflags = [f"-D{d}" for d in defines]

    def compile_one(pair):
        src, obj = pair
        if not (force or _stale(obj, [src] + headers)):
            return ""
        r = subprocess.run([nvcc, *ARCH, *FLAGS, *dflags, "-c", src, "-o", obj], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        logs = list(ex.map(compile_one, zip(srcs, objs)))
    if verbose:
        for log in logs:
            if log:
                print(log)
    if force or _stale(LIB_, objs):
        r = subprocess.run([nvcc, *ARCH, "-shared", "-o", LIB_, *objs, "-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if out == LIB:
        build_probes(force)
    return LIB_


def build_probes(force: bool = False) -> str:
    """The benchmark's ceiling probes (csrc/bench/probes.cu) as a shared library of their own."""
    src = os.path.join(CSRC, "bench", "probes.cu")
    deps = [src, os.path.join(CSRC, "mma_common.cuh"), os.path.join(CSRC, "common.cuh")]
    if force or _stale(PROBES_LIB, deps):
        r = subprocess.run([_nvcc(), *ARCH, *FLAGS, "-shared", "-o", PROBES_LIB, src, "-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return PROBES_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
