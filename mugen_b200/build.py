"""Builds libmugen_mla.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc."""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmugen_mla.so")
SOURCES = ["mla_api.cu", "mla_kernels.cu", "mla_decode_mma.cu", "mla_decode_tc5.cu", "mla_decode_tc5_pair2.cu", "mla_decode_tc5_t16.cu", "mla_merge_tc5.cu", "mla_absorb_tc5.cu", "mla_noalloc.cu", "mla_selftest.cu", "mla_gguf.cu", "mla_gemm_tc5.cu", "mla_prefill_tc5.cu"]
HEADERS = ["mla_common.cuh", "mla_launch.h", "mla_tc5.cuh", "../host/page_table.hpp", "../host/rope_table.hpp", "../host/gguf_reader.hpp",
           "../../include/mugen_mla.h"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++20",
              "-Xcompiler", "-fPIC,-ffp-contract=off,-Wall", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libmugen_mla.so")
    return path


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compiles every .cu of the package for sm_100a into one shared object; returns its path."""
    if not force and not needs_build():
        return LIB
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    subprocess.run([_nvcc(), "-shared", "-o", LIB, *objs], check=True)
    return LIB


if __name__ == "__main__":
    import sys
    print(build_library(force=True, verbose="-v" in sys.argv))
