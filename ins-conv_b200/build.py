"""Builds the native parts in-tree.

  libinsconv_b200.so   CUDA kernels + C ABI (nvcc, sm_100a only)
  sparseconvnet/SCN*.so the torch extension module `sparseconvnet.SCN` (g++ against torch headers),
                       linked against libinsconv_b200.so

Usage: python ins-conv_b200/build.py [--force] [--verbose] [--no-ext]
Nothing is rebuilt when the outputs are newer than every source.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB = os.path.join(HERE, "libinsconv_b200.so")
CU_SOURCES = ["capi.cu", "grid_build.cu", "feature_ops.cu", "gather_gemm_tc.cu", "gather_mma_warp.cu", "halo_exchange.cu", "label_fusion.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc():
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0 or verbose:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("build step failed: " + " ".join(cmd[:4]) + " ...")


def ext_path():
    return os.path.join(HERE, "sparseconvnet", "SCN" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_lib(force=False, verbose=False, ptxas_info=False):
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(INCLUDE, "insconv_b200.h"))
    objs = []
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + headers):
            cmd = [_nvcc()] + NVCC_FLAGS + os.environ.get("INSCONV_NVCC_FLAGS", "").split() + ["-I" + INCLUDE, "-I" + CSRC, "-c", s, "-o", o]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            _run(cmd, verbose or ptxas_info)
        objs.append(o)
    if force or _stale(LIB, objs):
        _run([_nvcc(), "-shared", "-o", LIB] + objs + ["-lcudart"], verbose)
    return LIB


def build_ext(force=False, verbose=False):
    src = os.path.join(CSRC, "scn_ext.cpp")
    out = ext_path()
    if not (force or _stale(out, [src, os.path.join(INCLUDE, "insconv_b200.h"), LIB])):
        return out
    import torch
    from torch.utils import cpp_extension as ce
    inc = ce.include_paths("cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(True)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", src, "-o", out,
           "-DTORCH_EXTENSION_NAME=SCN", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + INCLUDE, "-I" + sysconfig.get_paths()["include"]]
    cmd += ["-I" + i for i in inc]
    cmd += ["-L" + p for p in ce.library_paths()] + ["-L" + HERE]
    cmd += ["-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda", "-linsconv_b200",
            "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath," + ce.library_paths()[0]]
    _run(cmd, verbose)
    return out


def build_all(force=False, verbose=False, ext=True):
    build_lib(force, verbose)
    if ext:
        build_ext(force, verbose)


if __name__ == "__main__":
    build_all("--force" in sys.argv, "--verbose" in sys.argv, "--no-ext" not in sys.argv)
    if "--ptxas" in sys.argv:
        build_lib(True, True, True)
    print("built", LIB)
