"""Ahead-of-time build of the native library (no JIT at run time).

``python -m fleet_chiplet_megakernel_b200._build`` or ``build()`` compiles the
CUDA sources for sm_100a into ``libb200mk.so`` next to this file.  The built
library is what the package loads; there is no fallback when it is missing.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200mk.so")
# mk_kernel_tp.cu, mk_kernel_hier.cu and mk_kernel_moe.cu include mk_kernel.cu with other build switches (see its header)
SOURCES = ["mk_kernel.cu", "mk_kernel_tp.cu", "mk_kernel_hier.cu", "mk_kernel_moe.cu", "mk_runtime.cpp", "mk_noalloc.cu"]
HEADERS = ["mk_types.h", os.path.join("..", "..", "include", "b200mk.h")]


def _nvcc():
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found: the native library cannot be built")


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
    if verbose:
        flags = ["-Xptxas", "-v"] + flags
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    # one nvcc per source, side by side (the three builds of the kernel dominate), then one link
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        cmd = [_nvcc()] + flags + ["-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            print(" ".join(cmd))
        procs.append((cmd, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for cmd, obj, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stdout.write(out)
        if pr.returncode != 0:
            raise subprocess.CalledProcessError(pr.returncode, cmd)
        objs.append(obj)
    subprocess.check_call([_nvcc(), "-shared", "-o", LIB] + objs)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print(LIB)
