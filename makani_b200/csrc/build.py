"""In-tree build of the sm_100a extension `makani_b200/csrc/_C.so`.

Kernels (`*.cu`) are compiled by nvcc for `sm_100a` only and know nothing about torch; `bindings.cpp` is the
only translation unit that includes torch headers.  Objects are rebuilt when their sources (or headers)
are newer.  Works without a GPU (nvcc cross-compiles).

    python -m makani_b200.csrc.build [--force] [--verbose]
"""

from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "build")
TARGET = os.path.join(HERE, "_C.so")

CU_SOURCES = ["gemm_tcgen05.cu", "fused_ops.cu", "peer.cu", "spectral_modes.cu", "no_alloc.cu"]
CPP_SOURCES = ["bindings.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _cuda_home() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return cand
    raise RuntimeError("nvcc not found; set CUDA_HOME")


def _newer(src_list, out) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in src_list)


def _run(cmd, verbose, log_path=None):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path:
        with open(log_path, "w") as f:
            f.write(" ".join(cmd) + "\n" + res.stdout)
    if verbose or res.returncode != 0:
        print(" ".join(cmd))
        print(res.stdout)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd[:3])} ...")


def build(force: bool = False, verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension

    os.makedirs(BUILD, exist_ok=True)
    cuda = _cuda_home()
    nvcc = os.path.join(cuda, "bin", "nvcc")
    headers = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))]
    cu_sources = [s for s in CU_SOURCES if os.path.exists(os.path.join(HERE, s))]

    jobs = []
    objs = []
    for src in cu_sources:
        obj = os.path.join(BUILD, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _newer([os.path.join(HERE, src)] + headers, obj):
            jobs.append(([nvcc] + NVCC_FLAGS + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj],
                         os.path.join(BUILD, src + ".log")))

    inc = []
    for p in cpp_extension.include_paths(device_type="cuda") if "device_type" in cpp_extension.include_paths.__code__.co_varnames \
            else cpp_extension.include_paths(cuda=True):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"], "-isystem", os.path.join(cuda, "include")]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for src in CPP_SOURCES:
        obj = os.path.join(BUILD, src.replace(".cpp", ".o"))
        objs.append(obj)
        if force or _newer([os.path.join(HERE, src)] + headers, obj):
            jobs.append((["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                          "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                          "-I", HERE] + inc + ["-c", os.path.join(HERE, src), "-o", obj], None))

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _run(j[0], verbose, j[1]), jobs))

    if jobs or force or _newer(objs, TARGET):
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cmd = ["g++", "-shared", "-o", TARGET] + objs + [
            f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-ltorch_python", f"-L{os.path.join(cuda, 'lib64')}", f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}", "-lcudart",
        ]
        _run(cmd, verbose)
    return TARGET


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print("built", path)
