"""Builds libsynapse_b200.so in-tree with nvcc for sm_100a (no other architecture is compiled)."""
from __future__ import annotations

import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libsynapse_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"] + os.environ.get("SYN_NVCC_FLAGS", "").split()


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    stamp = os.path.getmtime(target)
    return any(os.path.getmtime(d) > stamp for d in deps)


def _compile(source, verbose):
    obj = os.path.join(OBJ, os.path.basename(source)[:-3] + ".o")
    if not _stale(obj, [source] + _headers()):
        return obj, ""
    cmd = [NVCC, *FLAGS, "-c", source, "-o", obj] + (["-Xptxas", "-v"] if verbose else [])
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed for {source}:\n{result.stdout}\n{result.stderr}")
    return obj, result.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every .cu under csrc/ and links the shared library. Returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    if force:
        for name in glob.glob(os.path.join(OBJ, "*.o")):
            os.remove(name)
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as pool:
        results = list(pool.map(lambda s: _compile(s, verbose), _sources()))
    objects = [obj for obj, _ in results]
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    if force or _stale(LIB, objects):
        cmd = [NVCC, "-shared", "-o", LIB, *objects, "-gencode", "arch=compute_100a,code=sm_100a"]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
