"""In-tree build of the two shared libraries of this package.

``libgsb200.so``      CUDA kernels + the C ABI of ``include/gsb200.h`` (nvcc, sm_100a only,
                      no framework dependency).
``libgs_b200_torch.so`` the host layer: ``torch.classes.gs_classes.Graph`` and
                      ``torch.ops.gs_ops.*`` registered from C++ (g++), calling the C ABI.

Both are written next to this file so that they travel with the source tree.
nvcc cross-compiles without a GPU, so the build also works on a CPU-only box.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_CUDA = os.path.join(HERE, "libgsb200.so")
LIB_TORCH = os.path.join(HERE, "libgs_b200_torch.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    cus = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = cus + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not force and _newer(LIB_CUDA, deps):
        return LIB_CUDA
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    objs = []
    for cu in cus:
        obj = os.path.join(objdir, os.path.basename(cu)[:-3] + ".o")
        objs.append(obj)
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", cu, "-o", obj]
        procs.append((cu, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    for cu, pr in procs:
        out, _ = pr.communicate()
        log.append(out)
        if pr.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {cu}")
    with open(os.path.join(objdir, "ptxas.log"), "w") as f:
        f.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    subprocess.check_call([_nvcc(), "-shared", "-o", LIB_CUDA, *objs, "-lcudart"])
    return LIB_CUDA


def build_torch(force: bool = False) -> str:
    import torch

    srcs = sorted(glob.glob(os.path.join(HERE, "host", "*.cc")))
    deps = srcs + glob.glob(os.path.join(HERE, "host", "*.h")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not force and _newer(LIB_TORCH, deps + [LIB_CUDA]):
        return LIB_TORCH
    tp = os.path.dirname(torch.__file__)
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    common = [
        cxx, "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        f"-I{tp}/include", f"-I{tp}/include/torch/csrc/api/include", f"-I{cuda_home}/include",
        f"-I{os.path.join(ROOT, 'include')}",
    ]
    procs, objs = [], []
    for s in srcs:
        obj = os.path.join(objdir, os.path.basename(s)[:-3] + ".host.o")
        objs.append(obj)
        procs.append((s, subprocess.Popen([*common, "-c", s, "-o", obj], stdout=subprocess.PIPE,
                                          stderr=subprocess.STDOUT, text=True)))
    for s, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"g++ failed on {s}")
    subprocess.check_call([
        cxx, "-shared", "-o", LIB_TORCH, *objs, f"-L{HERE}", "-lgsb200", f"-L{tp}/lib", "-ltorch",
        "-ltorch_cpu", "-lc10", "-lc10_cuda", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tp}/lib",
    ])
    return LIB_TORCH


def build_all(force: bool = False, verbose: bool = False):
    return build_cuda(force, verbose), build_torch(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", LIB_CUDA, LIB_TORCH)
