"""Builds libhtgs_b200.so (the sm_100a rasterizer core) in-tree with nvcc.

No torch headers are involved: the core is a plain C-ABI shared library.
Run `python -m htgs_b200.build` (add `-v` for ptxas resource usage).
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libhtgs_b200.so")
SOURCES = ["api.cu", "preprocess.cu", "binning.cu", "binning_unordered.cu", "blend.cu", "blend_fast.cu", "train.cu", "noalloc.cu", "filter3d.cu", "weights.cu", "activation.cu", "exchange.cu"]
HEADERS = ["common.cuh", "kernels.h", os.path.join("..", "..", "include", "htgs_b200.h")]

# IEEE division / sqrt and no fast-math: the per-fragment arithmetic has to round exactly like
# the reference's base build (its setup.py adds no fast-math flag to the main extension).
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-O2",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC")
    return cand


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = _nvcc()
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    headers = [os.path.normpath(os.path.join(CSRC, h)) for h in HEADERS]
    objs, jobs = [], []
    for src in sources:
        src_path = os.path.join(CSRC, src)
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [src_path] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src_path, "-o", obj]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        return src, res.returncode, res.stdout

    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            for src, rc, out in pool.map(run, jobs):
                if verbose or rc != 0:
                    sys.stdout.write(f"--- {src} ---\n{out}\n")
                if rc != 0:
                    raise RuntimeError(f"nvcc failed on {src}")
    if jobs or force or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH] + objs + ["-lcudart"]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:
            sys.stdout.write(res.stdout)
            raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="-f" in sys.argv, verbose="-v" in sys.argv))
