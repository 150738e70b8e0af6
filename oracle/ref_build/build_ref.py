"""Compile the reference's own CUDA path into oracle/_ref/libtsnecuda_ref.so (test infrastructure).

The reference's sources are compiled where they lie (nothing is copied into this repository):
every .cu under <reference>/src/{kernels,util,ext} and src/fit_tsne.cu, except
src/util/distance_utils.cu, which needs FAISS (an external dependency that is not installed).
That file's two functions come from knn_shim.cu; include-only stand-ins for the nine <faiss/...>
headers the reference's headers pull in are generated into oracle/_ref/stub/.  ref_harness.cu adds
stage-level entry points.  The reference's own build system is not run.

Needs nvcc and the reference tree; the result travels to the GPU box as a prebuilt file.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.normpath(os.path.join(HERE, "..", "_ref"))
LIB = os.path.join(OUT, "libtsnecuda_ref.so")


def find_reference_root():
    """Where the reference tree lies: TSNE_REFERENCE_ROOT, else a directory named `reference` beside this
    repository.  Nothing else is searched."""
    env = os.environ.get("TSNE_REFERENCE_ROOT")
    if env:
        return env
    repo = os.path.normpath(os.path.join(HERE, "..", ".."))
    return os.path.join(os.path.dirname(repo), "reference")


FAISS_HEADERS = ["IndexFlat.h", "IndexIVFFlat.h", "IndexIVFPQ.h", "gpu/GpuIndexFlat.h", "gpu/GpuIndexIVFFlat.h",
                 "gpu/GpuIndexIVFPQ.h", "gpu/StandardGpuResources.h", "gpu/GpuCloner.h"]
METRIC_STUB = """#pragma once
// include-only stand-in: just the enum the reference's Options struct stores
namespace faiss { enum MetricType { METRIC_INNER_PRODUCT = 0, METRIC_L2 = 1, METRIC_L1, METRIC_Linf, METRIC_Lp,
                                    METRIC_Canberra = 20, METRIC_BrayCurtis, METRIC_JensenShannon }; }
"""


def stage_python_wrapper(ref):
    """Put the reference's own Python package (src/python/tsnecuda: __init__.py, TSNE.py) under
    oracle/_ref/python/, unmodified, so that the drop-in test can import it next to this repository's
    libtsnecuda.so on a machine that has no reference tree.  Build output like the .so: never committed."""
    import shutil
    pkg = os.path.join(ref, "src", "python", "tsnecuda")
    if not os.path.isdir(pkg):
        return None
    dst = os.path.join(OUT, "python", "tsnecuda")
    os.makedirs(dst, exist_ok=True)
    for name in ("__init__.py", "TSNE.py"):
        shutil.copyfile(os.path.join(pkg, name), os.path.join(dst, name))
    return dst


def build(force=False, reference_root=None):
    ref = reference_root or find_reference_root()
    src = os.path.join(ref, "src")
    if not os.path.isdir(src):
        return LIB if os.path.exists(LIB) else None
    stage_python_wrapper(ref)
    own = [os.path.join(HERE, "knn_shim.cu"), os.path.join(HERE, "ref_harness.cu")]
    theirs = sorted(glob.glob(os.path.join(src, "kernels", "*.cu")) + glob.glob(os.path.join(src, "util", "*.cu")) +
                    glob.glob(os.path.join(src, "ext", "*.cu")) + [os.path.join(src, "fit_tsne.cu")])
    theirs = [f for f in theirs if os.path.basename(f) != "distance_utils.cu"]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(f) < os.path.getmtime(LIB) for f in own + theirs):
        return LIB
    stub = os.path.join(OUT, "stub", "faiss")
    os.makedirs(os.path.join(stub, "gpu"), exist_ok=True)
    with open(os.path.join(stub, "MetricType.h"), "w") as f:
        f.write(METRIC_STUB)
    for h in FAISS_HEADERS:
        with open(os.path.join(stub, h), "w") as f:
            f.write("#pragma once\n")
    objdir = os.path.join(OUT, "obj")
    os.makedirs(objdir, exist_ok=True)
    flags = ["-std=c++17", "-O3", "-DNO_ZMQ", "-gencode=arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC", "-w",
             "-I", ref, "-I", src, "-I", os.path.join(src, "include"), "-I", os.path.join(OUT, "stub")]

    def cc(f):
        o = os.path.join(objdir, os.path.basename(f).replace(".cu", ".o"))
        subprocess.check_call(["nvcc", "-c", f, "-o", o] + flags)
        return o

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(cc, theirs + own))
    subprocess.check_call(["nvcc", "-shared", "-o", LIB] + objs + ["-lcufft", "-lcublas", "-lcusparse", "-Xlinker", "-Bsymbolic"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
