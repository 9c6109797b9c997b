"""Builds oracle/_ref/libscn_ref.so: the reference's own sources for the hot path, compiled for the host.

TEST INFRASTRUCTURE.  The library this makes is a second checker beside the Python oracle: it runs the
reference implementation itself (THU-luvision/INS-Conv, sparseconvnet/SCN) so that the oracle's
restatement can be pinned against it in a container that has no GPU.  Nothing the product ships loads it.

What is compiled, from where it lies under the reference tree (nothing is copied into this repository):
  Metadata/Metadata.cpp and the rule headers it includes, CUDA/CUDPPWrapper.hpp, CUDA/SubmanifoldRules_cuda.cpp
  CUDA/{CUDPPWrapper,SubmanifoldRules_cuda,IOLayers,BatchNormalization,Convolution,Deconvolution}.cu
  CUDA/{Convolution,Deconvolution,BatchNormalization,IOLayers,NetworkInNetwork}.cpp
  CPU/{Convolution,Deconvolution,BatchNormalization,IOLayers,NetworkInNetwork}.cpp
How a CUDA source becomes host code: one translation unit is assembled in memory and piped to g++ --
ref_prelude.h (ATen, the CUDA-on-host emulation ref_emu.h, the CUDPP stand-in) + the reference files +
ref_exports.cpp (extern "C" entry points).  The only edit made to the reference text on the way through the
pipe is mechanical: a kernel launch `k<<<grid, block[, shmem]>>>(args)` becomes
`REF_EMU_LAUNCH(grid, block, shmem, k(args))`, and `extern __shared__` loses `__shared__` (the dynamic
shared-memory array becomes an ordinary global defined in ref_exports.cpp).  Kernel bodies, host launchers,
rulebook builders and Metadata run as written.  Third-party pieces that are NOT the reference's code are
stood in for by contract: CUDPP (extra/cudpp: sort-based multivalue hash, compact, scan, reduce), google
sparsehash, easy_profiler, the CUDA runtime (ref_shim/, ref_emu.h, ref_cudpp.h).

Usage: python oracle/build_ref.py [--force] [--verbose] [--reference DIR]   (DIR: the reference tree; default below)
"""
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libscn_ref.so")
DEFAULT_REFERENCE = "/root/reference"

HOST_FIRST = ["Metadata/Metadata.cpp"]
CU_FILES = ["CUDA/CUDPPWrapper.cu", "CUDA/SubmanifoldRules_cuda.cu", "CUDA/IOLayers.cu", "CUDA/BatchNormalization.cu",
            "CUDA/Convolution.cu", "CUDA/Deconvolution.cu"]
HOST_AFTER = ["CUDA/Convolution.cpp", "CUDA/Deconvolution.cpp", "CUDA/BatchNormalization.cpp", "CUDA/IOLayers.cpp",
              "CUDA/NetworkInNetwork.cpp",
              "CPU/Convolution.cpp", "CPU/Deconvolution.cpp", "CPU/BatchNormalization.cpp", "CPU/IOLayers.cpp",
              "CPU/NetworkInNetwork.cpp", "Metadata/resultHash.h"]
OWN = ["ref_prelude.h", "ref_emu.h", "ref_cudpp.h", "ref_exports.cpp", "build_ref.py"]


def _match_back_angle(text, i):
    """text[i] == '>': index of the '<' that opens it."""
    depth = 0
    while i >= 0:
        c = text[i]
        if c == ">":
            depth += 1
        elif c == "<":
            depth -= 1
            if depth == 0:
                return i
        i -= 1
    raise ValueError("unbalanced template arguments before a launch")


def _match_fwd_paren(text, i):
    """text[i] == '(': index of the ')' that closes it."""
    depth = 0
    while i < len(text):
        c = text[i]
        if c == "(":
            depth += 1
        elif c == ")":
            depth -= 1
            if depth == 0:
                return i
        i += 1
    raise ValueError("unbalanced launch arguments")


def rewrite_launches(text):
    """kernel<<<cfg>>>(args) -> REF_EMU_LAUNCH(grid, block, shmem, kernel(args)); comments are left alone
    because a rewritten launch inside a comment is still a comment."""
    out = []
    pos = 0
    while True:
        a = text.find("<<<", pos)
        if a < 0:
            break
        b = text.index(">>>", a)
        # kernel expression: identifier, optionally followed by template arguments
        j = a - 1
        while text[j].isspace() or text[j] == "\\":  # a launch inside a macro continues over lines with '\'
            j -= 1
        if text[j] == ">":
            j = _match_back_angle(text, j) - 1
            while text[j].isspace() or text[j] == "\\":
                j -= 1
        k = j
        while k >= 0 and (text[k].isalnum() or text[k] in "_:"):
            k -= 1
        name_start = k + 1
        kernel = text[name_start:a]
        p = b + 3
        while text[p].isspace():
            p += 1
        assert text[p] == "(", text[a - 40:p + 10]
        q = _match_fwd_paren(text, p)
        cfg = text[a + 3:b]
        # split the configuration at top-level commas
        parts, depth, cur = [], 0, ""
        for c in cfg:
            if c in "([{":
                depth += 1
            elif c in ")]}":
                depth -= 1
            if c == "," and depth == 0:
                parts.append(cur)
                cur = ""
            else:
                cur += c
        parts.append(cur)
        while len(parts) < 3:
            parts.append("0")
        out.append(text[pos:name_start])
        one_line = lambda t: re.sub(r"\\\s*\n", " ", t).strip()  # drop the line continuations of a macro body
        out.append("REF_EMU_LAUNCH((%s), (%s), (%s), (%s%s))" % (one_line(parts[0]), one_line(parts[1]), one_line(parts[2]),
                                                                 one_line(kernel), text[p:q + 1]))
        pos = q + 1
    out.append(text[pos:])
    return "".join(out)


def translation_unit(ref_scn):
    parts = ['#include "ref_prelude.h"\n']
    for rel in HOST_FIRST:
        parts.append('#include "%s"\n' % rel)
    for rel in CU_FILES:
        path = os.path.join(ref_scn, rel)
        with open(path) as f:
            text = f.read()
        text = rewrite_launches(text).replace("extern __shared__", "extern")
        parts.append('#line 1 "%s"\n%s\n' % (path, text))
    parts.append('#line 1 "ref_tail"\n')
    for rel in HOST_AFTER:
        parts.append('#include "%s"\n' % rel)
    parts.append('#include "ref_cudpp.h"\n#include "ref_exports.cpp"\n')
    return "".join(parts)


def build(reference=DEFAULT_REFERENCE, force=False, verbose=False):
    """Returns the path of the library, or None when the reference tree is not there (the GPU box: the
    prebuilt file travels instead)."""
    ref_scn = os.path.join(reference, "sparseconvnet", "SCN")
    if not os.path.isdir(ref_scn):
        return OUT if os.path.exists(OUT) else None
    deps = [os.path.join(HERE, f) for f in OWN]
    deps += [os.path.join(ref_scn, f) for f in HOST_FIRST + CU_FILES + HOST_AFTER]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(d) <= os.path.getmtime(OUT) for d in deps):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    import torch
    from torch.utils import cpp_extension as ce
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-x", "c++", "-", "-std=c++17", "-O1", "-fPIC", "-shared", "-w", "-fpermissive", "-o", OUT,
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + HERE, "-I" + os.path.join(HERE, "ref_shim"), "-I" + ref_scn, "-I" + os.path.join(ref_scn, "CUDA"),
           "-I" + os.path.join(reference, "extra", "cudpp", "include")]
    cmd += ["-I" + p for p in ce.include_paths() if "cuda" not in p.lower().split(os.sep)[-2:]]
    import sysconfig
    cmd += ["-I" + sysconfig.get_paths()["include"]]  # resultHash.h includes torch/extension.h, which wants Python.h
    cmd += ["-L" + lib_dir, "-ltorch_cpu", "-ltorch", "-lc10", "-Wl,-rpath," + lib_dir]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, input=translation_unit(ref_scn), capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stderr[-20000:])
        raise RuntimeError("building the reference for the host failed")
    return OUT


if __name__ == "__main__":
    ref = DEFAULT_REFERENCE
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    if "--tu" in sys.argv:
        sys.stdout.write(translation_unit(os.path.join(ref, "sparseconvnet", "SCN")))
    else:
        print(build(ref, "--force" in sys.argv, "--verbose" in sys.argv))
