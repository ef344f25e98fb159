"""Builds build/lib/libc_runtime_api.so (sm_100a) from tinyflow_b200/csrc/*.cu with nvcc.

The output path mirrors the reference's loader, which opens
``<repo>/build/lib/libc_runtime_api.so`` (pycode/tinyflow/_base.py:10-20).
Run ``python -m tinyflow_b200.build`` or call :func:`build`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "tinyflow_b200", "csrc")
OBJ_DIR = os.path.join(ROOT, "build", "obj")
LIB_PATH = os.path.join(ROOT, "build", "lib", "libc_runtime_api.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; cannot build libc_runtime_api.so")


def _newer(src: str, dst: str, deps) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(p) > t for p in [src, *deps])


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> str:
    """Compile every .cu under csrc/ (in parallel) and link the shared library. Returns its path."""
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(os.path.dirname(LIB_PATH), exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(ROOT, "include", "c_runtime_api.h"))
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    objs, jobs = [], []
    for f in sources:
        src, obj = os.path.join(CSRC, f), os.path.join(OBJ_DIR, f[:-3] + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0 or ptxas_info:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for " + cmd[-3])

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB_PATH):
        run([nvcc, "-shared", "-o", LIB_PATH, *objs, "-ldl"])
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv))
