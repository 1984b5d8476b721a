"""Builds the backend's shared library in-tree.

    python -m ocannl_b200.build            # libb200.so + sm_100a compile check of the kernels

The host library is plain C++ (g++): it opens the CUDA driver, NVRTC and NCCL at run time.
The device code lives in `csrc/kernels/*.cuh`; the library embeds those sources and compiles
each routine's kernels for sm_100a through NVRTC when the routine is compiled.  `nvcc` is
used here to prove, at build time and without a GPU, that every kernel source compiles for
`-gencode arch=compute_100a,code=sm_100a` (the check translation units are in
`csrc/kernels/check_*.cu`).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "libb200.so")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")

HOST_SOURCES = ["ir.cpp", "emit.cpp", "compile.cpp", "gemm_match.cpp", "attn_match.cpp", "driver.cpp", "runtime.cpp",
                "gemm_launch.cpp", "api.cpp"]
CUDA_SOURCES = ["sum_static.cu"]
EMBED = {"kNumericsSource": "kernels/numerics.cuh", "kTcSource": "kernels/tc_sm100.cuh",
         "kGemmSource": "kernels/gemm_sm100.cuh", "kAttnSource": "kernels/attn_sm100.cuh"}


def _embed() -> str:
    path = os.path.join(OUT, "embedded_sources.cpp")
    parts = ['#include "compile.hpp"\nnamespace b200 {\n']
    for sym, rel in EMBED.items():
        text = open(os.path.join(CSRC, rel)).read()
        # split into chunks below the compilers' string-literal limits
        chunks = [text[i:i + 8000] for i in range(0, len(text), 8000)] or [""]
        lit = "\n".join('  R"B200SRC(' + c + ')B200SRC"' for c in chunks)
        parts.append("const char* %s =\n%s;\n" % (sym, lit))
    parts.append("}  // namespace b200\n")
    new = "".join(parts)
    if not os.path.exists(path) or open(path).read() != new:
        with open(path, "w") as f:
            f.write(new)
    return path


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(verbose=False) -> str:
    os.makedirs(OUT, exist_ok=True)
    emb = _embed()
    srcs = [os.path.join(CSRC, s) for s in HOST_SOURCES] + [emb]
    hdrs = [os.path.join(CSRC, h) for h in os.listdir(CSRC) if h.endswith(".hpp")]
    hdrs.append(os.path.join(HERE, "..", "include", "b200.h"))
    objs = []
    for s in srcs:
        o = os.path.join(OUT, os.path.basename(s)[:-4] + ".o")
        if _newer(o, [s] + hdrs):
            cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-Wall", "-Wno-unused-function", "-I", CSRC,
                   "-I", os.path.join(CUDA, "include"), "-c", s, "-o", o]
            if verbose:
                print(" ".join(cmd))
            subprocess.run(cmd, check=True)
        objs.append(o)
    # translation units that hold ahead-of-time kernels: nvcc, sm_100a only
    for s in CUDA_SOURCES:
        src = os.path.join(CSRC, s)
        o = os.path.join(OUT, s[:-3] + ".o")
        if _newer(o, [src] + hdrs):
            cmd = [os.path.join(CUDA, "bin", "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
                   "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-I", CSRC, "-c", src, "-o", o]
            if verbose:
                print(" ".join(cmd))
            subprocess.run(cmd, check=True)
        objs.append(o)
    if _newer(LIB, objs):
        cmd = ["g++", "-shared", "-o", LIB] + objs + ["-L", os.path.join(CUDA, "lib64"), "-lcudart_static", "-lrt",
                                                       "-ldl", "-lpthread"]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return LIB


def check_kernels(verbose=False) -> None:
    """nvcc cross-compiles every kernel source for sm_100a (no GPU needed)."""
    kdir = os.path.join(CSRC, "kernels")
    for f in sorted(os.listdir(kdir)):
        if not (f.startswith("check_") and f.endswith(".cu")):
            continue
        src = os.path.join(kdir, f)
        out = os.path.join(OUT, f[:-3] + ".cubin")
        deps = [os.path.join(kdir, x) for x in os.listdir(kdir)]
        if not _newer(out, deps):
            continue
        cmd = [os.path.join(CUDA, "bin", "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
               "-O3", "-std=c++17", "-Xptxas", "-v", "-cubin", "-I", kdir, src, "-o", out]
        if verbose:
            print(" ".join(cmd))
        r = subprocess.run(cmd, capture_output=True, text=True)
        with open(out[:-6] + ".ptxas.txt", "w") as lf:
            lf.write(r.stderr)
        if r.returncode != 0:
            sys.stderr.write(r.stderr)
            raise RuntimeError("nvcc failed on " + f)


def main():
    build_library(verbose=True)
    check_kernels(verbose=True)
    print("built", LIB)


if __name__ == "__main__":
    main()
