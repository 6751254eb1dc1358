"""Builds oracle/_ref/gs_ref.so: the reference's own CUDA implementation files for the hot path,
compiled UNMODIFIED from where they lie in the reference tree, plus the small binding in
ref_binding.cc.  Test infrastructure only (tier-2 oracle for the GPU tests and the
"reference on the same GPU" timing).

    python oracle/build_ref.py [--reference /path/to/gSampler] [--jobs N]

Needs nvcc, the torch headers and the reference tree; where the tree is absent (e.g. on a GPU box
that only received the prebuilt file) it does nothing.  The reference includes <glog/logging.h>,
which is not installed here; oracle/ref_shim/ provides a stand-in whose failed checks throw.
About 5 minutes of nvcc per file; objects are cached in oracle/_ref/.
"""
import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SOURCES = [
    "src/cuda/slicing.cu", "src/cuda/sampling.cu", "src/cuda/unique_reindex.cu",
    "src/cuda/fusion/slice_sampling.cu", "src/cuda/batch/slicing.cu",
    "src/cuda/batch/batch_relabel.cu", "src/cuda/fusion/random_walk.cu",
    "src/cuda/fusion/node2vec.cu", "src/cuda/fusion/column_row_slicing.cu",
    "src/cuda/sampling_probs.cu", "src/cuda/list_sampling.cu", "src/cuda/list_sampling_probs.cu",
    "src/cuda/batch/list_sampling_probs.cu", "src/cuda/spmm.cu", "src/cuda/sddmm.cu", "src/bcast.cc",
    "src/cuda/sort_indices.cu", "src/cuda/fusion/fused_coo_u_op_v.cu", "src/cuda/fusion/fused_csc_u_op_v.cu",
    "src/cuda/fusion/fused_coo_e_square_sum.cu", "src/cuda/fusion/fused_csc_e_square_sum.cu",
    "src/cuda/fusion/fused_coo_e_div_u_sum.cu", "src/cuda/fusion/fused_csc_e_div_u_sum.cu",
]


def reference_dir():
    """The gSampler source tree: $GSAMPLER_REFERENCE, else a checkout named ``reference`` beside
    this repository; None when neither exists."""
    cand = os.environ.get("GSAMPLER_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src", "cuda")) else None


def python_dir():
    """Where stage_python() puts the reference's Python package."""
    return os.path.join(OUT, "python")


def stage_python(reference=None):
    """Copies the reference's own Python layer (python/gs: Matrix, BatchMatrix, gs.jit.compile with
    its fx tracer and passes, gs.ops) UNMODIFIED into oracle/_ref/python/gs, next to gs_ref.so and
    with the same standing: made by this recipe, git-ignored, test infrastructure only.  The tests
    import it over this repository's libraries to check that it runs on them as it stands."""
    reference = reference or reference_dir()
    src = os.path.join(reference or "", "python", "gs")
    if not os.path.isdir(src):
        return None
    dst = os.path.join(python_dir(), "gs")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.so"))
    return dst


def lib_path():
    return os.path.join(OUT, "gs_ref.so")


def build(reference=None, jobs=None, verbose=True):
    reference = reference or reference_dir()
    if not reference or not os.path.isdir(os.path.join(reference, "src", "cuda")):
        return None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return None
    import torch

    tp = os.path.dirname(torch.__file__)
    os.makedirs(OUT, exist_ok=True)
    inc = ["-I" + os.path.join(reference, "src"), "-I" + os.path.join(reference, "src", "cuda"),
           "-I" + os.path.join(HERE, "ref_shim"), "-I" + os.path.join(tp, "include"),
           "-I" + os.path.join(tp, "include", "torch", "csrc", "api", "include"),
           "-I" + sysconfig.get_paths()["include"]]
    common = ["-std=c++17", "-O2", "-D_GLIBCXX_USE_CXX11_ABI=1", "-DTORCH_EXTENSION_NAME=gs_ref",
              "-Xcompiler", "-fPIC", "-w"]
    cuda = ["--extended-lambda", "--expt-relaxed-constexpr", "-gencode", "arch=compute_100a,code=sm_100a"]
    binding = os.path.join(HERE, "ref_binding.cc")
    units = [(os.path.join(reference, s), os.path.join(OUT, os.path.basename(os.path.dirname(s)) + "_" +
              os.path.splitext(os.path.basename(s))[0] + ".o")) for s in SOURCES]
    units.append((binding, os.path.join(OUT, "ref_binding.o")))

    def compile_one(unit):
        src, obj = unit
        if os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(src):
            return 0
        cmd = [nvcc, *common, *cuda, *inc, "-x", "cu", "-c", src, "-o", obj]
        if verbose:
            print("nvcc", os.path.relpath(src, reference) if src.startswith(reference) else src, flush=True)
        return subprocess.call(cmd)

    with ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
        rcs = list(ex.map(compile_one, units))
    if any(rcs):
        raise RuntimeError("reference build failed (%s)" % rcs)
    objs = [o for _, o in units]
    out = lib_path()
    if not os.path.exists(out) or any(os.path.getmtime(o) > os.path.getmtime(out) for o in objs):
        libdir = os.path.join(tp, "lib")
        subprocess.check_call([nvcc, "-shared", "-o", out, *objs, "-L" + libdir, "-lc10", "-lc10_cuda",
                               "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
                               "-Xlinker", "-rpath," + libdir])
    return out


def load():
    """Imports the built module (after torch), or returns None when it has not been built."""
    path = lib_path()
    if not os.path.exists(path):
        return None
    import importlib.util

    import torch  # noqa: F401  (its libraries must be loaded first)

    spec = importlib.util.spec_from_file_location("gs_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--jobs", type=int, default=None)
    a = ap.parse_args()
    print(stage_python(a.reference))
    print(build(a.reference, a.jobs))
