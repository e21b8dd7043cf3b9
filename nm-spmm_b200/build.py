"""In-tree build of libnmspmm_b200.so with nvcc for sm_100a (no GPU needed)."""
from __future__ import annotations

import concurrent.futures
import glob
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.environ.get("NMSPMM_BUILD_DIR") or os.path.join(CSRC, "build")
LIB = os.environ.get("NMSPMM_BUILD_LIB") or os.path.join(HERE, "libnmspmm_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC] + os.environ.get("NMSPMM_NVCC_EXTRA", "").split()


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _headers():
    return (glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
            + glob.glob(os.path.join(ROOT, "include", "*.h")))


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, os.path.basename(src) + ".o")
    if _stale(obj, [src] + _headers()):
        cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        out = subprocess.run(cmd, capture_output=True, text=True)
        if out.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s%s" % (src, out.stdout, out.stderr))
        if verbose:
            keep = [l for l in out.stderr.splitlines() if "registers" in l or "spill" in l or "Compiling" in l]
            with open(obj + ".ptxas.txt", "w") as f:
                f.write("\n".join(keep) + "\n")
    return obj


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile every source under csrc/ and link the shared library.  Returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    if force:
        for f in glob.glob(os.path.join(OBJ, "*.o")):
            os.remove(f)
    srcs = _sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), srcs))
    if _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        out = subprocess.run(cmd, capture_output=True, text=True)
        if out.returncode != 0:
            raise RuntimeError("link failed:\n" + out.stdout + out.stderr)
    if verbose:
        print("built", LIB)
    return LIB


if __name__ == "__main__":
    build(verbose=True)
