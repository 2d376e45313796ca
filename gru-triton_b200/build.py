"""Build the CUDA library in-tree: ``gru-triton_b200/lib/libb200gru.so``.

Plain nvcc, sm_100a only, no framework headers.  ``python gru-triton_b200/build.py``
or ``build()`` from Python.  Objects are rebuilt when a source or header is newer.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_DIR = os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(LIB_DIR, os.environ.get("B200GRU_LIB_NAME", "libb200gru.so"))

SOURCES = ["api.cu", "diag_scan.cu", "block_scan.cu", "block_gemm.cu", "butterfly_scan.cu", "butterfly_scan2.cu",
           "tc_gemm.cu", "tc_step.cu", "tc_scan.cu", "weight_prep.cu", "tc_api.cu", "calib_scan.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",                 # elementwise gate math rounds like the eager reference; dots use fmaf()
    "-Xcompiler", "-fPIC",
    "-I", INCLUDE,
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set $NVCC)")


def _newest_dep() -> float:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "b200gru.h"), __file__]
    return max(os.path.getmtime(p) for p in deps)


def _compile(nvcc: str, src: str, obj: str, verbose: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("B200GRU_EXTRA_NVCC_FLAGS", "").split(), "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile (if stale) and return the path of the shared library."""
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    newest = _newest_dep()
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= newest:
        return LIB_PATH
    nvcc = _nvcc()
    jobs = []
    objs = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        for s in SOURCES:
            src = os.path.join(CSRC, s)
            obj = os.path.join(OBJ_DIR, s.replace(".cu", ".o"))
            objs.append(obj)
            if force or not os.path.exists(obj) or os.path.getmtime(obj) < newest:
                jobs.append(ex.submit(_compile, nvcc, src, obj, verbose))
        for j in jobs:
            out = j.result()
            if verbose and out:
                print(out, file=sys.stderr)
    tmp = LIB_PATH + ".tmp"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-cudart", "static"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
