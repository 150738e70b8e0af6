"""Build recipe for libtsnecuda.so (hand-written sm_100a CUDA + C++ host orchestration).

  python -m tsne_cuda_b200.build [--force]

Compiles every .cu under csrc/ with nvcc for sm_100a only and links them into
tsne_cuda_b200/libtsnecuda.so, next to the Python wrapper that loads it.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libtsnecuda.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers():
    return (glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) +
            glob.glob(os.path.join(HERE, "..", "include", "*.h")) +
            glob.glob(os.path.join(HERE, "..", "include", "tsnecuda", "*.h")))


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    hdr_time = max(os.path.getmtime(h) for h in _headers())

    def cc(src):
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if (not force and os.path.exists(obj) and os.path.getmtime(obj) > os.path.getmtime(src)
                and os.path.getmtime(obj) > hdr_time):
            return obj, False
        cmd = ["nvcc", "-c", src, "-o", obj] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
        subprocess.check_call(cmd)
        return obj, True

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        res = list(ex.map(cc, sources()))
    objs = [o for o, _ in res]
    if force or any(ch for _, ch in res) or not os.path.exists(LIB):
        subprocess.check_call(["nvcc", "-shared", "-o", LIB] + objs +
                              ["-gencode", "arch=compute_100a,code=sm_100a", "-ldl", "-Xlinker", "-Bsymbolic"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
