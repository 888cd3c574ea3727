"""In-tree build of the two native artefacts of mor_b200.

``libmor_b200.so``  the CUDA kernels behind the C ABI of ``include/mor_b200.h``
                    (nvcc, sm_100a only, no torch headers; a few seconds).
``_C.*.so``         the PyTorch shim that registers ``torch.ops.mor.*`` and forwards
                    to the C ABI (g++ against the torch headers; about a minute).

Both land next to this file so that they travel with the source tree; nothing is
installed into site-packages.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libmor_b200.so")
CU_SOURCES = ["fq_elementwise.cu", "fq_reduce.cu", "fq_scaling.cu", "fq_block.cu", "fq_group.cu", "fq_resident.cu", "p2p.cu", "api.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(os.path.dirname(HERE), "include", "mor_b200.h"))
    return hs


def shim_path() -> str:
    return os.path.join(HERE, "_C" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    hdrs = _headers()
    objs = []

    def compile_one(src):
        s = os.path.join(CSRC, src)
        o = os.path.join(BUILD, src.replace(".cu", ".o"))
        if force or not _newer(o, [s] + hdrs):
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
            if verbose:
                sys.stderr.write(r.stderr)
        return o

    with ThreadPoolExecutor(max_workers=len(CU_SOURCES)) as ex:
        objs = list(ex.map(compile_one, CU_SOURCES))
    if force or not _newer(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link of libmor_b200.so failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def build_extension(force: bool = False) -> str:
    """Compile csrc/torch_shim.cpp into mor_b200/_C.<abi>.so, linked against libmor_b200.so."""
    import torch
    from torch.utils import cpp_extension

    build_library(force=False)
    out = shim_path()
    src = os.path.join(CSRC, "torch_shim.cpp")
    if not force and _newer(out, [src, LIB] + _headers()):
        return out
    tdir = os.path.dirname(torch.__file__)
    inc = [f"-I{p}" for p in cpp_extension.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *inc, src, "-o", out,
           f"-L{HERE}", "-lmor_b200", "-Wl,-rpath,$ORIGIN",
           f"-L{os.path.join(tdir, 'lib')}", f"-Wl,-rpath,{os.path.join(tdir, 'lib')}",
           "-lc10", "-lc10_cuda", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-ltorch_python",
           "-L/usr/local/cuda/lib64", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed on torch_shim.cpp:\n{r.stdout}\n{r.stderr}")
    return out


def build_all(force: bool = False) -> None:
    build_library(force=force)
    build_extension(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print(LIB)
    print(shim_path())
