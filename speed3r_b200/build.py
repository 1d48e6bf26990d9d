"""Build recipe for the C-ABI library: every ``csrc/*.cu`` is compiled for sm_100a with nvcc and
linked into ``speed3r_b200/libspeed3r_b200.so`` (kept in-tree, next to the package).  The tests-only
companion ``libspeed3r_b200_check.so`` (``csrc/check/*.cu`` plus the shared host plumbing) is built
beside it; the package never loads it.

    python -m speed3r_b200.build [-v] [--force]
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "csrc", "build")
LIB = os.path.join(PKG, "libspeed3r_b200.so")
CHECK_LIB = os.path.join(PKG, "libspeed3r_b200_check.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return cand


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(PKG, "..", "include", "*.h"))
    os.makedirs(OBJ, exist_ok=True)
    if _stale(obj, [src] + headers):
        cmd = [_nvcc()] + NVCC_FLAGS + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = os.path.join(OBJ, os.path.basename(src)[:-3] + ".ptxas.log")
        with open(log, "w") as f:
            f.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
    return obj


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    if force:
        for f in glob.glob(os.path.join(OBJ, "*.o")):
            os.remove(f)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    check_srcs = sorted(glob.glob(os.path.join(CSRC, "check", "*.cu")))
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs) + len(check_srcs))) as ex:
        all_objs = list(ex.map(lambda s: _compile(s, verbose), srcs + check_srcs))
    objs, check_objs = all_objs[:len(srcs)], all_objs[len(srcs):]
    api_obj = [o for o in objs if os.path.basename(o) == "api.o"]
    for lib, members in ((LIB, objs), (CHECK_LIB, check_objs + api_obj)):
        if _stale(lib, members):
            cmd = [_nvcc(), "-shared", "-o", lib] + members + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv))
