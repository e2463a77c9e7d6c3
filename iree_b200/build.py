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


PLUGIN_PATH = os.path.join(_HERE, "libiree_uk_b200_plugin.so")
PLUGIN_SRC = os.path.join(_HERE, "..", "plugin", "iree_uk_b200_plugin.c")


def reference_include_dir():
    """``runtime/src`` of an IREE checkout (for the standalone executable-plugin header): the
    IREE_REFERENCE_SRC environment variable, or a checkout named ``reference`` beside this
    repository; None when neither exists."""
    cands = [os.environ.get("IREE_REFERENCE_SRC"),
             os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference", "runtime", "src")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "iree", "hal", "local", "executable_plugin.h")):
            return c
    return None


def build_plugin(verbose=False):
    """Compiles the IREE executable plugin (plugin/iree_uk_b200_plugin.c) against the plugin
    header of an IREE checkout and links it to the library beside it. Returns its path, or None
    when no checkout is available (an already built plugin is then left as it is)."""
    inc = reference_include_dir()
    if inc is None:
        return PLUGIN_PATH if os.path.exists(PLUGIN_PATH) else None
    deps = [PLUGIN_SRC, LIB_PATH] + glob.glob(os.path.join(_HERE, "..", "include", "*.h"))
    if _newer(PLUGIN_PATH, deps):
        cmd = ["gcc", "-std=c11", "-O2", "-Wall", "-Wextra", "-fPIC", "-shared",
               "-fvisibility=hidden", "-I" + inc, "-I" + os.path.join(_HERE, "..", "include"),
               PLUGIN_SRC, "-o", PLUGIN_PATH, "-L" + _HERE, "-liree_uk_b200",
               "-Wl,-rpath,$ORIGIN"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return PLUGIN_PATH


if __name__ == "__main__":
    build(verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(LIB_PATH)
    print(build_plugin(verbose=True))
