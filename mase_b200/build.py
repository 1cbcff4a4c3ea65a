"""Builds libmxq.so (the C-ABI library of hand-written sm_100a kernels) in-tree with nvcc.

    python -m mase_b200.build [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The library lands in `mase_b200/lib/libmxq.so`.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libmxq.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "mxq.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu under csrc/ into one shared library; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libmxq.so cannot be built")
    os.makedirs(LIB_DIR, exist_ok=True)
    objs = []
    for src in sources():
        obj = os.path.join(LIB_DIR, os.path.basename(src)[:-3] + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(
            os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC)
        ) or os.path.getmtime(obj) < os.path.getmtime(os.path.join(ROOT, "include", "mxq.h")):
            cmd = [nvcc, *NVCC_FLAGS, "-I" + os.path.join(ROOT, "include"), "-I" + CSRC, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            subprocess.run(cmd, check=True)
        objs.append(obj)
    tmp = LIB_PATH + ".tmp"  # link under another name, then swap: a reader never sees a half-written library
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", tmp, *objs, "-lcudart"]
    subprocess.run(cmd, check=True)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


EXT_NAME = "_mxq_torch"


def ext_path() -> str:
    import sysconfig

    return os.path.join(LIB_DIR, EXT_NAME + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_torch_binding(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/torch_binding.cpp (host code only, g++) into mase_b200/lib/_mxq_torch*.so, linked against
    libmxq.so and torch.  Optional: the package issues the same C calls through ctypes when it is absent."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    build()
    src = os.path.join(CSRC, "torch_binding.cpp")
    out = ext_path()
    deps = [src, os.path.join(ROOT, "include", "mxq.h")]
    if not force and os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return out
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = cpp_extension.include_paths() + [sysconfig.get_paths()["include"], os.path.join(ROOT, "include"),
                                           os.path.join(cuda_home, "include")]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=" + EXT_NAME,
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *["-I" + i for i in inc], src, "-o", out + ".tmp",
           "-L" + torch_lib, "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10", "-lc10_cuda", "-ltorch_cuda",
           "-L" + LIB_DIR, "-l:libmxq.so", "-Wl,-rpath," + torch_lib, "-Wl,-rpath,$ORIGIN"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    os.replace(out + ".tmp", out)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_torch_binding(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
