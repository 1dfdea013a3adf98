"""Builds libcswap_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcswap_b200.so")
SOURCES = ["zfp_kernels.cu", "sparse_kernels.cu", "cswap_abi.cu", "swap_manager.cu", "cost_model.cu",
           "sparse_static.cu"]
HEADERS = ["zfp_core.cuh", "zfp_field.cuh", "zfp_kernels.h", "sparse_kernels.h", "internal.h",
           os.path.join("..", "..", "include", "cswap_b200.h"), os.path.join("..", "..", "include", "cswap_compat.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for s in SOURCES:
        o = os.path.join(objdir, s.replace(".cu", ".o"))
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
              ["-c", os.path.join(CSRC, s), "-o", o]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(o)
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}")
    cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-Xcompiler", "-fPIC"]
    subprocess.check_call(cmd)
    return LIB


CPP_DRIVERS = ("execution_driver", "vgg16_step", "bert_step")


def build_cpp_driver(force: bool = False, name: str = "execution_driver") -> str:
    """Compile tests/cpp/<name>.cpp (drivers written against the C++ Execution
    class over stock libtorch, include/cswap_execution.hpp) against the in-tree
    library with g++."""
    import torch
    root = os.path.dirname(HERE)
    src = os.path.join(root, "tests", "cpp", name + ".cpp")
    hdrs = [os.path.join(root, "include", h) for h in ("cswap_execution.hpp", "cswap_b200.h")]
    exe = os.path.join(root, "tests", "cpp", name)
    if not force and os.path.exists(exe) and all(os.path.getmtime(exe) >= os.path.getmtime(f) for f in [src] + hdrs):
        return exe
    build()
    t = os.path.dirname(torch.__file__)
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    # the CUDA runtime libtorch itself is linked against (its wheel ships one), else the toolkit's
    import glob
    rt = sorted(glob.glob(os.path.join(os.path.dirname(t), "nvidia", "cuda_runtime", "lib", "libcudart.so.*")))
    rt = rt[0] if rt else os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64", "libcudart.so")
    cmd = ["g++", "-std=c++17", "-O1", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I", os.path.join(root, "include"), "-I", os.path.join(t, "include"),
           "-I", os.path.join(t, "include", "torch", "csrc", "api", "include"), "-I", cuda_inc, src, "-o", exe,
           "-L", os.path.join(t, "lib"), "-L", HERE, f"-Wl,-rpath,{os.path.join(t, 'lib')}",
           "-Wl,-rpath,$ORIGIN/../../cswap_b200", "-Wl,--no-as-needed",
           "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-lcswap_b200", rt,
           f"-Wl,-rpath,{os.path.dirname(rt)}", "-Wno-interference-size"]
    subprocess.check_call(cmd)
    return exe


def build_cpp_drivers(force: bool = False):
    return [build_cpp_driver(force, n) for n in CPP_DRIVERS]


if __name__ == "__main__":
    if "--cpp" in sys.argv:
        print(build_cpp_drivers(force="--force" in sys.argv))
        sys.exit(0)
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
