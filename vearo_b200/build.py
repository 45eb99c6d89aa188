"""Builds libvearo_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libvearo_b200.so")
LIB_BC = os.path.join(HERE, "libvearo_b200_bc.so")          # the bounds-check build (python build.py --bounds-check)
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "host", "*.cpp")))


def _deps(src):
    d = [src] + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "host", "*.h")) + \
        glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h"))
    return d


def _compile(src, verbose, ptxas_v, bounds_check=False):
    obj = os.path.join(OBJ, ("bc_" if bounds_check else "") + os.path.relpath(src, CSRC).replace(os.sep, "_") + ".o")
    if os.path.exists(obj) and all(os.path.getmtime(d) <= os.path.getmtime(obj) for d in _deps(src)):
        return obj
    cmd = [NVCC] + FLAGS + (["-DVB200_BOUNDS_CHECK"] if bounds_check else []) + (["-Xptxas", "-v"] if ptxas_v else []) + ["-x", "cu", "-c", src, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s" % (src, r.stderr))
    if verbose or ptxas_v:
        sys.stderr.write(r.stderr)
    return obj


def build(verbose=False, ptxas_v=False, bounds_check=False):
    """The library; with bounds_check=True the variant whose kernels verify every computed gather / scatter index
    (libvearo_b200_bc.so; select it with VB200_LIB=<path> before importing vearo_b200)."""
    os.makedirs(OBJ, exist_ok=True)
    srcs = sources()
    lib = LIB_BC if bounds_check else LIB
    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, ptxas_v, bounds_check), srcs))
    if not os.path.exists(lib) or any(os.path.getmtime(o) > os.path.getmtime(lib) for o in objs):
        cmd = [NVCC, "-Wno-deprecated-gpu-targets", "-shared", "-o", lib] + objs + ["-ldl"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return lib


if __name__ == "__main__":
    build(verbose="--quiet" not in sys.argv, ptxas_v="--ptxas" in sys.argv, bounds_check="--bounds-check" in sys.argv)
