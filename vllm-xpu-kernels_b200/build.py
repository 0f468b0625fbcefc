"""In-tree build of the two shared objects of this package (no cmake, no setuptools).

  vllm_xpu_kernels/libkvcache_b200.so   CUDA kernels + C ABI   (nvcc, sm_100a only)
  vllm_xpu_kernels/_C.abi3.so           torch op registration  (g++, links the above)

Run ``python build.py`` (add ``--force`` to rebuild, ``--verbose`` for ptxas register
and spill figures).  Both objects are rebuilt only when a source is newer.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig

ROOT = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(ROOT)
CSRC = os.path.join(ROOT, "csrc")
PKG = os.path.join(ROOT, "vllm_xpu_kernels")
INCLUDE = os.path.join(REPO, "include")

CUDA_LIB = os.path.join(PKG, "libkvcache_b200.so")
TORCH_EXT = os.path.join(PKG, "_C.abi3.so")

CUDA_SOURCES = [os.path.join(CSRC, "kvcache_kernels.cu"), os.path.join(CSRC, "fp8_quant_kernels.cu"),
                os.path.join(CSRC, "rope_kernels.cu"), os.path.join(CSRC, "paged_attention_kernels.cu")]
EXT_SOURCES = [os.path.join(CSRC, "cache.cpp"), os.path.join(CSRC, "fp8_quant.cpp"),
               os.path.join(CSRC, "pos_encoding.cpp"), os.path.join(CSRC, "flash_api.cpp"),
               os.path.join(CSRC, "torch_bindings.cpp")]
HEADERS = [
    os.path.join(INCLUDE, "kvcache_b200.h"),
    os.path.join(CSRC, "ops.h"),
    os.path.join(CSRC, "dispatch_utils.h"),
    os.path.join(CSRC, "core", "registration.h"),
]
CUDA_HEADERS = [HEADERS[0]] + [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cuh")]


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} (exit {r.returncode})")
    if verbose:
        sys.stderr.write(r.stderr)


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def build_cuda_lib(force: bool = False, verbose: bool = False) -> str:
    if force or _stale(CUDA_LIB, CUDA_SOURCES + CUDA_HEADERS):
        cmd = [
            _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
            "--threads", str(len(CUDA_SOURCES)), "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", INCLUDE, "-I", CSRC, "-o", CUDA_LIB,
        ]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        _run(cmd + CUDA_SOURCES, verbose)
    return CUDA_LIB


def build_torch_ext(force: bool = False, verbose: bool = False) -> str:
    build_cuda_lib(force, verbose)
    if force or _stale(TORCH_EXT, EXT_SOURCES + HEADERS + [CUDA_LIB]):
        import torch
        from torch.utils import cpp_extension

        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        cxx = "g++"  # the system compiler; a CXX override in the environment may lack its runtime files
        cmd = [
            cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall",
            "-DTORCH_EXTENSION_NAME=_C", "-DPy_LIMITED_API=0x03090000",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
            "-I", INCLUDE, "-I", CSRC, "-I", sysconfig.get_paths()["include"],
            "-I", os.path.join(cuda_home, "include"),
        ]
        for inc in cpp_extension.include_paths():
            cmd += ["-isystem", inc]
        cmd += EXT_SOURCES
        cmd += [
            "-o", TORCH_EXT, "-L", PKG, "-l:libkvcache_b200.so", "-L", torch_lib, "-lc10", "-lc10_cuda",
            "-ltorch_cpu", "-ltorch", "-Wl,-rpath,$ORIGIN", "-Wl,--no-as-needed",
        ]
        _run(cmd, verbose)
    return TORCH_EXT


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_torch_ext(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ns = ap.parse_args()
    build_all(ns.force, ns.verbose)
    print(CUDA_LIB)
    print(TORCH_EXT)
