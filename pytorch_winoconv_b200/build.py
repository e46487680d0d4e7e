"""In-tree build of the native code.

* ``libwinoconv_b200.so``  -- the C-ABI library (CUDA kernels for sm_100a + host driver),
  compiled by nvcc from ``csrc/*.cu``; no torch headers, so it builds in about a minute.
* ``MakePytorchBackend*.so`` -- the pybind11 / torch extension that exports the reference's
  operator names (``DWM``, ``WinoSplit``, ``WinoConcat``, ``AddGPU``, ``Foo``; reference:
  ``pybind/bind.cpp:11-24``) on top of the C ABI; host C++ only (g++).

Both land next to this file so a repository snapshot carries them.  ``python -m
pytorch_winoconv_b200.build`` builds both; objects are cached under ``build/`` by source mtime.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(ROOT, "include")
BUILD_DIR = os.path.join(ROOT, "build", "winoconv")
CAPI_LIB = os.path.join(PKG_DIR, "libwinoconv_b200.so")

CUDA_SOURCES = ["wino_transforms.cu", "wino_gemm_simt.cu", "wino_gemm_tcgen05.cu", "wino_fused23.cu", "wino_rowfused.cu", "wino_probe.cu", "wino_capi.cu"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".hpp"))]
    hs.append(os.path.join(INCLUDE, "winoconv_b200.h"))
    return hs


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    return res


def build_capi(verbose: bool = False) -> str:
    """Compile csrc/*.cu for sm_100a and link libwinoconv_b200.so.  Returns its path."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    headers = _headers()
    jobs, objs = [], []
    for src in CUDA_SOURCES:
        sp = os.path.join(CSRC, src)
        obj = os.path.join(BUILD_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        if not _newer(obj, [sp] + headers):
            jobs.append([_nvcc(), *NVCC_FLAGS, "-DWINOCONV_BUILDING", "-I", INCLUDE, "-I", CSRC, "-c", sp, "-o", obj])
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            for res in ex.map(_run, jobs):
                if verbose and res.stderr:
                    print(res.stderr, file=sys.stderr)
    if not _newer(CAPI_LIB, objs):
        _run([_nvcc(), "-shared", "-o", CAPI_LIB, *objs, "-cudart", "shared"])
    return CAPI_LIB


def backend_path() -> str:
    return os.path.join(PKG_DIR, "MakePytorchBackend" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_backend(verbose: bool = False) -> str:
    """Build the torch extension module MakePytorchBackend next to this file."""
    import torch
    from torch.utils import cpp_extension

    build_capi(verbose)
    out = backend_path()
    srcs = [os.path.join(CSRC, "backend_ops.cpp"), os.path.join(CSRC, "backend_bind.cpp")]
    if _newer(out, srcs + _headers() + [CAPI_LIB]):
        return out
    os.makedirs(BUILD_DIR, exist_ok=True)
    inc = cpp_extension.include_paths("cuda") if hasattr(cpp_extension, "include_paths") else []
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    flags = ["-std=c++17", "-O2", "-fPIC", "-DTORCH_EXTENSION_NAME=MakePytorchBackend",
             "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    includes = ["-I", INCLUDE, "-I", CSRC, "-I", sysconfig.get_paths()["include"], "-I", os.path.join(cuda_home, "include")]
    for p in inc:
        includes += ["-isystem", p]
    objs = []
    jobs = []
    for sp in srcs:
        obj = os.path.join(BUILD_DIR, os.path.basename(sp).replace(".cpp", ".o"))
        objs.append(obj)
        if not _newer(obj, [sp] + _headers()):
            jobs.append(["g++", *flags, *includes, "-c", sp, "-o", obj])
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            list(ex.map(_run, jobs))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    link = ["g++", "-shared", "-o", out, *objs, "-L", PKG_DIR, "-l:libwinoconv_b200.so", "-L", torch_lib,
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-L", os.path.join(cuda_home, "lib64"), "-lcudart",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(link)
    return out


def build_all(verbose: bool = False):
    return build_capi(verbose), build_backend(verbose)


if __name__ == "__main__":
    for path in build_all(verbose=True):
        print(path)
