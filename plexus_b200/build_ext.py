"""Build the CUDA extension in-tree for sm_100a.

``python -m plexus_b200.build_ext`` compiles every ``.cu`` under ``csrc`` with
``nvcc -gencode arch=compute_100a,code=sm_100a`` (the kernels include no torch
headers, so this takes seconds per file), compiles the pybind11/torch wrapper
``bindings.cpp`` with the host compiler, and links ``plexus_b200/_C.so`` next
to the package sources.  nvcc cross-compiles: no GPU is needed to build.
"""

from __future__ import annotations

import glob
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
BUILD = os.path.join(PKG, "build")
NAME = "_C"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "--use_fast_math", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def cuda_sources():
    return sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))


def headers():
    return sorted(glob.glob(os.path.join(CSRC, "include", "*")))


def so_path() -> str:
    return os.path.join(PKG, NAME + ".so")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def is_fresh() -> bool:
    return not _stale(so_path(), cuda_sources() + headers() + [os.path.join(CSRC, "bindings.cpp")])


def _run(cmd, log):
    res = subprocess.run(cmd, capture_output=True, text=True)
    log.append((" ".join(cmd), res.stdout + res.stderr))
    if res.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and is_fresh():
        return so_path()
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(BUILD, exist_ok=True)
    nvcc = os.path.join(ce.CUDA_HOME or "/usr/local/cuda", "bin", "nvcc")
    cuda_inc = os.path.join(ce.CUDA_HOME or "/usr/local/cuda", "include")
    log = []
    jobs = []
    objs = []
    extra = os.environ.get("PLEXUS_EXTRA_DEFINES", "").split()  # e.g. -DPLX_GEMM_PROF for timing probes
    for src in cuda_sources():
        obj = os.path.join(BUILD, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers()):
            jobs.append([nvcc, *NVCC_FLAGS, *extra, "-c", src, "-o", obj])
    bsrc = os.path.join(CSRC, "bindings.cpp")
    bobj = os.path.join(BUILD, "bindings.o")
    objs.append(bobj)
    if force or _stale(bobj, [bsrc] + headers()):
        inc = [f"-I{p}" for p in ce.include_paths(device_type="cuda")] + [
            f"-I{sysconfig.get_paths()['include']}", f"-I{cuda_inc}",
        ]
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        jobs.append([
            os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-c", bsrc, "-o", bobj,
            f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *extra, *inc,
        ])
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(lambda c: _run(c, log), jobs))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_lib = os.path.join(ce.CUDA_HOME or "/usr/local/cuda", "lib64")
    _run([
        os.environ.get("CXX", "g++"), "-shared", *objs, "-o", so_path(),
        f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
        f"-L{cuda_lib}", "-lcudart", f"-Wl,-rpath,{torch_lib}",
    ], log)
    if verbose:
        for cmd, out in log:
            print("$", cmd)
            print(out)
    with open(os.path.join(BUILD, "build.log"), "w") as f:
        for cmd, out in log:
            f.write("$ " + cmd + "\n" + out + "\n")
    return so_path()


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
