"""Builds ``libiree_uk_b200.so`` in-tree with nvcc for sm_100a.

``python -m iree_b200.build`` (or ``build()``) compiles every ``csrc/*.cu|*.cc`` file whose
object is older than its sources and links them into ``iree_b200/libiree_uk_b200.so``. nvcc
cross-compiles without a GPU.
"""
import glob
import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
OBJ_DIR = os.path.join(_HERE, "build")
LIB_PATH = os.path.join(_HERE, "libiree_uk_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-Xcompiler", "-Wall",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, ptxas_info=False):
    """Compile and link the library; returns its path. With IREE_UK_B200_EXPERIMENTS set in the
    environment the tuning overrides (environment variables read at run time, used for
    parameter sweeps) are compiled in; the ordinary build has none."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    experiments = bool(os.environ.get("IREE_UK_B200_EXPERIMENTS"))
    stamp = os.path.join(OBJ_DIR, "experiments" if experiments else "product")
    other = os.path.join(OBJ_DIR, "product" if experiments else "experiments")
    if os.path.exists(other) or not os.path.exists(stamp):  # flavour changed: rebuild everything
        for f in glob.glob(os.path.join(OBJ_DIR, "*.o")) + [other]:
            if os.path.exists(f):
                os.remove(f)
        open(stamp, "w").close()
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        [os.path.join(_HERE, "..", "include", "iree_uk_b200.h")]
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cc")))
    objs = []
    for src in sources:
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
        objs.append(obj)
        if _newer(obj, [src] + headers):
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + \
                (["-DIREE_UK_B200_EXPERIMENTS"] if experiments else []) + \
                ["-x", "cu", "-c", src, "-o", obj]
            if verbose:
                print(" ".join(cmd), flush=True)
            subprocess.check_call(cmd)
    if _newer(LIB_PATH, objs):
        cmd = [_nvcc(), "-shared", "-cudart", "static", "-o", LIB_PATH] + objs
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return LIB_PATH


if __name__ == "__main__":
    build(verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(LIB_PATH)
