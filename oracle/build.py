"""Build recipe for the CPU oracle (test infrastructure; never imported by the product).

  python oracle/build.py          -> oracle/_build/liboracle.so   (gcc, OpenMP)
  python oracle/build.py --ref    -> also oracle/_ref/libtsnecuda_ref.so, the reference's own CUDA
                                     sources compiled where they lie (needs the reference tree)
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")
LIB = os.path.join(OUT, "liboracle.so")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "tsne_oracle.c")
    os.makedirs(OUT, exist_ok=True)
    if force or _stale(LIB, [src]):
        cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
               "-o", LIB, src, "-lm"]
        subprocess.check_call(cmd)
    return LIB


def build_reference(force=False, reference_root=None):
    """Compile the reference's CUDA path (see oracle/ref_build/build_ref.py). Returns the .so path or None."""
    sys.path.insert(0, os.path.join(HERE, "ref_build"))
    import build_ref  # noqa: E402
    return build_ref.build(force=force, reference_root=reference_root)


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_reference(force="--force" in sys.argv))
