"""Builds libspingalett.so in-tree: C23 host sources with gcc, sm_100a kernels
with nvcc, one shared object (CUDA runtime linked statically).

    python -m spingalett_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "lib", "libspingalett.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
GCC = "gcc"

# extra -D switches for experiments (e.g. SPG_NVCC_DEFS="-DSPG_DBG_X"); never set in a normal build
NVCC_FLAGS = os.environ.get("SPG_NVCC_DEFS", "").split() + [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I" + os.path.join(ROOT, "include"),
    "-I" + os.path.join(CSRC, "cuda"),
]
GCC_FLAGS = [
    "-std=c2x", "-O2", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra", "-D_GNU_SOURCE",
    "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(CSRC, "host"),
]


def _sources():
    cu = sorted(os.path.join(CSRC, "cuda", f) for f in os.listdir(os.path.join(CSRC, "cuda")) if f.endswith(".cu"))
    c = sorted(os.path.join(CSRC, "host", f) for f in os.listdir(os.path.join(CSRC, "host")) if f.endswith(".c"))
    return cu, c


def _headers():
    out = []
    for d in (os.path.join(CSRC, "cuda"), os.path.join(CSRC, "host"), os.path.join(ROOT, "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                out.append(os.path.join(d, f))
    return out


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)


def build(force=False, verbose=False, ptxas_v=False):
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    cu, c = _sources()
    hdr_time = max(os.path.getmtime(h) for h in _headers())
    objs = []
    dirty = False
    for src in cu + c:
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time)
        if not stale:
            continue
        dirty = True
        if src.endswith(".cu"):
            _run([NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_v else []) + ["-c", src, "-o", obj], verbose or ptxas_v)
        else:
            _run([GCC] + GCC_FLAGS + ["-c", src, "-o", obj], verbose)
    if dirty or not os.path.exists(LIB):
        _run([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs +
             ["-Xlinker", "-Bsymbolic", "-lpthread", "-ldl", "-lm"], verbose)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_v="--ptxas" in sys.argv))
