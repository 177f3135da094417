"""In-tree build of the native pieces (no JIT cache, nothing installed outside the package):

  libomni_attn_sm100.so            CUDA kernels + C ABI        (nvcc, sm_100a only)
  omni_attn.cpython-*.so           pybind module with the reference's five entry points
                                   (g++ against the torch headers, links the library above)

``python -m omni_attention_b200.build`` builds both; cross-compilation needs no GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_NAME = "libomni_attn_sm100.so"
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)
PYBIND_PATH = os.path.join(PKG_DIR, "omni_attn" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
CUDA_SOURCES = ["omni_abi.cu", "omni_fwd_simple.cu", "omni_fwd_ws.cu", "omni_mask_build.cu", "omni_bwd.cu"]
CUDA_HEADERS = ["ptx_sm100.cuh", "omni_common.cuh", "omni_launch.h", os.path.join("..", "..", "include", "omni_attn_sm100.h")]


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps if os.path.exists(d))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def build_library(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in CUDA_HEADERS]
    if not force and _newer(LIB_PATH, deps):
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "-shared", "-o", LIB_PATH, *srcs]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True, cwd=CSRC)
    return LIB_PATH


def build_pybind(force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension

    src = os.path.join(CSRC, "omni_attn_pybind.cc")
    if not force and _newer(PYBIND_PATH, [src, LIB_PATH, os.path.join(PKG_DIR, "..", "include", "omni_attn_sm100.h")]):
        return PYBIND_PATH
    inc = []
    for p in cpp_extension.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]:
        inc += ["-isystem", p]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [
        "g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
        "-DTORCH_EXTENSION_NAME=omni_attn", "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, src, "-o", PYBIND_PATH,
        f"-L{PKG_DIR}", "-l:" + LIB_NAME, f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda", "-ltorch_python",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}",
    ]
    subprocess.run(cmd, check=True, cwd=CSRC)
    return PYBIND_PATH


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_library(force=force, verbose=verbose)
    build_pybind(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB_PATH)
    print(PYBIND_PATH)
