"""In-tree build of the native libraries (sm_100a only).

* ``libdecoding_attn_b200.so``  -- CUDA kernels + C ABI (include/decoding_attn_b200.h) + the C++
  ``decoding_attn()`` entry point (include/decoding_attn.h); built with nvcc.
* ``decoding_attn_cuda*.so``    -- the torch extension module of the same name as the reference's
  (csrc/torch/decoding_torch.cpp:82-85, setup.py:81); plain C++ linked against the library above.

Run ``python -m decoding_attention_b200.build`` (add ``--force`` to rebuild everything).
"""
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libdecoding_attn_b200.so")
EXT = os.path.join(PKG, "decoding_attn_cuda" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
NVCC_FLAGS = ["-std=c++17", "-O3", "--use_fast_math", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-ccbin", CXX]

CUDA_SOURCES = ["da_api.cu", "da_merge.cu", "da_split_d64.cu", "da_split_d96.cu", "da_split_d128.cu",
                "da_split_d256.cu", "da_split_mla_simt.cu", "da_mla_2sm_sm100.cu", "da_gqa_tc_sm100.cu", "da_gqa_quad_sm100.cu", "da_xmerge.cu", "da_noalloc.cu", "da_order.cu"]
CXX_SOURCES = ["decoding_attn.cpp"]
HEADERS = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + [
    os.path.join(ROOT, "include", "decoding_attn_b200.h"), os.path.join(ROOT, "include", "decoding_attn.h")]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), r.stdout))
    return r.stdout


def build_library(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    jobs = []
    objs = []
    for src in CUDA_SOURCES + CXX_SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + HEADERS):
            jobs.append(([NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for out in pool.map(_run, jobs):
                if verbose and out:
                    print(out)
    if jobs or force or _stale(LIB, objs):
        _run([NVCC, "-shared", "-o", LIB] + objs + ["-ccbin", CXX, "-cudart", "shared"])
    return LIB


def build_torch_extension(force=False):
    """Compile csrc/torch_binding.cpp against the installed torch (host compiler only)."""
    src = os.path.join(CSRC, "torch_binding.cpp")
    if not (force or _stale(EXT, [src, LIB] + HEADERS)):
        return EXT
    import torch
    from torch.utils import cpp_extension as ce
    inc = []
    for d in ce.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]:
        inc += ["-isystem", d]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [CXX, "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=decoding_attn_cuda",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           src, "-o", EXT] + inc + [
        "-L" + PKG, "-ldecoding_attn_b200", "-L" + tlib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
        "-ltorch", "-ltorch_python", "-L/usr/local/cuda/lib64", "-lcudart",
        "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib]
    _run(cmd)
    return EXT


def build_all(force=False, verbose=False):
    build_library(force=force, verbose=verbose)
    build_torch_extension(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
    print(EXT)
