"""Compile the CUDA sources of this package for sm_100a into powerinfer_b200/libpowerinfer_b200.so.

nvcc cross-compiles without a GPU.  The library is built in-tree so that it travels with the source
tree; it links the CUDA runtime statically and depends on nothing else.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libpowerinfer_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "powerinfer_b200.h"))
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    for s in sources():
        src, obj = os.path.join(CSRC, s), os.path.join(objdir, s[:-3] + ".o")
        if force or _stale(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        r = subprocess.run([NVCC] + FLAGS + ["-c", src, "-o", obj], capture_output=True, text=True)
        with open(obj[:-2] + ".ptxas.log", "w") as f:
            f.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return src

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        for done in ex.map(compile_one, jobs):
            if verbose:
                print("compiled", os.path.basename(done))
    objs = [os.path.join(objdir, s[:-3] + ".o") for s in sources()]
    if force or jobs or _stale(LIB, objs):
        r = subprocess.run([NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return LIB


GGML_LIB = os.path.join(HERE, "libggml_cuda_b200.so")


def reference_dir():
    """The reference checkout whose ggml.h the drop-in back end is compiled against: $POWERINFER_REF, else a sibling
    directory `reference` next to this repository; None when neither exists."""
    for cand in (os.environ.get("POWERINFER_REF"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.exists(os.path.join(cand, "ggml-cuda.h")):
            return os.path.abspath(cand)
    return None


def build_ggml_backend(force: bool = False) -> str | None:
    """powerinfer_b200/libggml_cuda_b200.so: the ggml-cuda.h symbol set over libpowerinfer_b200.so.  It reads struct
    ggml_tensor, so it needs the reference's headers at compile time; where they are absent the prebuilt file is kept."""
    ref = reference_dir()
    src = os.path.join(HERE, "ggml_backend", "ggml_cuda_b200.cu")
    if ref is None:
        return GGML_LIB if os.path.exists(GGML_LIB) else None
    if force or _stale(GGML_LIB, [src, LIB, os.path.join(os.path.dirname(HERE), "include", "powerinfer_b200.h")]):
        r = subprocess.run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
                            "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", ref, "-I", os.path.join(os.path.dirname(HERE), "include"),
                            "-o", GGML_LIB, src, "-L", HERE, "-lpowerinfer_b200", "-Xlinker", "-rpath=$ORIGIN"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("ggml back end failed to build:\n" + r.stdout + r.stderr)
    return GGML_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
    print(build_ggml_backend(force="--force" in sys.argv))
