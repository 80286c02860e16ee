"""Builds libhtgs_b200.so (the sm_100a rasterizer core) in-tree with nvcc, and the two torch extension modules over it.

No torch headers are involved in the core: it is a plain C-ABI shared library.  The torch / pybind layer is one host-only
source (csrc/bindings.cpp) compiled twice with the host compiler into htgs_b200/pybind/_C.*.so and _C_benchmarking.*.so.
Run `python -m htgs_b200.build` (add `-v` for ptxas resource usage, `--no-bindings` to skip the torch modules).
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


PYBIND_DIR = os.path.join(HERE, "pybind")
BINDINGS_SRC = os.path.join(CSRC, "bindings.cpp")


def binding_paths():
    import sysconfig
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    return os.path.join(PYBIND_DIR, "_C" + suffix), os.path.join(PYBIND_DIR, "_C_benchmarking" + suffix)


def build_bindings(force: bool = False) -> tuple:
    """Compiles csrc/bindings.cpp into the extension modules `_C` and `_C_benchmarking` (same names and signatures as the
    reference's pybind modules) and links them against libhtgs_b200.so.  Host compiler only; takes a minute or two."""
    import shutil as _shutil
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    lib = build()
    # The system compiler, not $CXX: this image exports CXX as a wrapper script around g++ meant for nvcc's -ccbin, and a
    # module built through it crashed as soon as a C++ exception left libc10 (every failing TORCH_CHECK).  HTGS_B200_CXX overrides.
    cxx = os.environ.get("HTGS_B200_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else None) or _shutil.which("g++") or _shutil.which("c++")
    if not cxx:
        raise RuntimeError("no C++ compiler found; set HTGS_B200_CXX")
    try:
        includes, libdirs = ce.include_paths("cuda"), ce.library_paths("cuda")
    except TypeError:      # older signature
        includes, libdirs = ce.include_paths(cuda=True), ce.library_paths(cuda=True)
    includes = list(includes) + [sysconfig.get_paths()["include"]]
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-Wno-unused-variable", "-Wno-unused-function", "-DTORCH_API_INCLUDE_EXTENSION_H",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for pname in ("COMPILER_TYPE", "STDLIB", "BUILD_ABI"):      # keeps pybind11's internals compatible with torch's own build
        pval = getattr(torch._C, f"_PYBIND11_{pname}", None)
        if pval is not None:
            flags.append(f'-DPYBIND11_{pname}="{pval}"')
    link = [f"-L{d}" for d in libdirs] + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
                                          f"-L{HERE}", "-lhtgs_b200", "-Wl,-rpath,$ORIGIN/.."] + [f"-Wl,-rpath,{d}" for d in libdirs]
    targets = binding_paths()
    jobs = []
    for target, name, extra in ((targets[0], "_C", []), (targets[1], "_C_benchmarking", ["-DHTGS_BINDINGS_BENCHMARKING"])):
        if force or _stale(target, [BINDINGS_SRC, lib, os.path.normpath(os.path.join(CSRC, "..", "..", "include", "htgs_b200.h"))]):
            jobs.append((name, [cxx] + flags + extra + [f"-DTORCH_EXTENSION_NAME={name}"] + [f"-I{d}" for d in includes] + [BINDINGS_SRC, "-o", target] + link))
    if jobs:
        os.makedirs(PYBIND_DIR, exist_ok=True)
        init = os.path.join(PYBIND_DIR, "__init__.py")
        if not os.path.exists(init):
            raise RuntimeError(f"{init} is missing")

        def run(job):
            name, cmd = job
            res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            return name, res.returncode, res.stdout

        with concurrent.futures.ThreadPoolExecutor(max_workers=2) as pool:
            for name, rc, out in pool.map(run, jobs):
                if rc != 0:
                    sys.stdout.write(f"--- bindings {name} ---\n{out}\n")
                    raise RuntimeError(f"compiling the torch extension module {name} failed")
        # self-test in a child process: a failing check inside the module must surface as a Python exception, with or without a GPU
        probe = ("import torch\nfrom htgs_b200.pybind import _C\n"
                 "try:\n    _C.context_handle(100000)\nexcept RuntimeError:\n    print('exceptions-ok')\n")
        res = subprocess.run([sys.executable, "-c", probe], cwd=os.path.dirname(HERE), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if "exceptions-ok" not in res.stdout:
            for target in targets:
                if os.path.exists(target):
                    os.remove(target)
            raise RuntimeError("the torch extension modules were built but do not survive a C++ exception (removed them again):\n" + res.stdout[-2000:])
    return targets


if __name__ == "__main__":
    print(build(force="-f" in sys.argv, verbose="-v" in sys.argv))
    if "--no-bindings" not in sys.argv:
        print(*build_bindings(force="-f" in sys.argv), sep="\n")
