"""Build the sm_100a extension in-tree: nvcc for the ``.cu`` files (no torch headers in them, so they compile
in seconds), g++ for the torch binding layer, one shared object ``forge_train_harness_b200/_C.so``.

``python -m forge_train_harness_b200.csrc.build`` rebuilds what changed (mtime based).  nvcc cross-compiles
without a GPU, so this runs on a CPU-only box.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OBJ = os.path.join(HERE, "build")
SO = os.path.join(PKG, "_C.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
CU_SOURCES = ["elementwise.cu", "gemm_sm100.cu", "attention_sm100.cu", "comm_sm100.cu", "comm_gemm_sm100.cu", "mxfp8_sm100.cu"]
HEADERS = ["common.cuh", "sm100_ptx.cuh", "gemm_pipe.cuh", "api.h", "noalloc.h"]


def _newer(src_list, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list if os.path.exists(s))


def _run(cmd, log):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.append(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("build failed: " + " ".join(cmd))


def build(verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OBJ, exist_ok=True)
    cuda_home = ce.CUDA_HOME or "/usr/local/cuda"
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    hdrs = [os.path.join(HERE, h) for h in HEADERS]
    log, objs = [], []
    for cu in CU_SOURCES:
        src = os.path.join(HERE, cu)
        if not os.path.exists(src):
            continue
        obj = os.path.join(OBJ, cu.replace(".cu", ".o"))
        if _newer([src] + hdrs, obj):
            _run([nvcc] + NVCC_FLAGS + ["-I", HERE, "-c", src, "-o", obj], log)
        objs.append(obj)
    bsrc = os.path.join(HERE, "bindings.cpp")
    bobj = os.path.join(OBJ, "bindings.o")
    if _newer([bsrc] + hdrs, bobj):
        inc = []
        for p in ce.include_paths(device_type="cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(True):
            inc += ["-I", p]
        inc += ["-I", sysconfig.get_paths()["include"], "-I", HERE]
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-c", bsrc, "-o", bobj] + inc, log)
    objs.append(bobj)
    if _newer(objs, SO):
        libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
        tmp = SO + f".tmp{os.getpid()}"   # link beside the target, then rename: a reader never sees a half-written library
        _run(["g++", "-shared", "-o", tmp] + objs + ["-L", libdir, "-L", os.path.join(cuda_home, "lib64"),
             "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
             f"-Wl,-rpath,{libdir}"], log)
        os.replace(tmp, SO)
    with open(os.path.join(OBJ, "build.log"), "w") as f:
        f.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    return SO


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
