"""Build libnfai_cuda.so (hand-written CUDA for sm_100a) in-tree with nvcc.

    python -m nfai_b200.build [--force] [--verbose]

Objects go to nfai_b200/build/, the library to nfai_b200/lib/libnfai_cuda.so. nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libnfai_cuda.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

SOURCES = ["api.cu", "gemv.cu", "gemv_ring.cu", "gemm_tc.cu", "attn.cu", "attn_ring.cu", "attn_mma.cu", "attn_prefill_tc.cu", "attn_static.cu", "misc.cu", "tp.cu", "gguf_loader.cu", "sample.cu", "tokenizer.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _host_compiler_flags() -> List[str]:
    # the environment may export CXX as a wrapper that nvcc cannot drive; use the system g++
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def _sources() -> List[str]:
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _deps_mtime() -> float:
    t = 0.0
    for root in (CSRC, INCLUDE):
        for f in os.listdir(root):
            if f.endswith((".cu", ".cpp", ".cuh", ".h")):
                t = max(t, os.path.getmtime(os.path.join(root, f)))
    return t


def needs_build() -> bool:
    return not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < _deps_mtime()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []
    header_t = max(os.path.getmtime(os.path.join(r, f)) for r in (CSRC, INCLUDE) for f in os.listdir(r)
                   if f.endswith((".cuh", ".h")))

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
        srcp = os.path.join(CSRC, src)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(srcp), header_t):
            return obj
        cmd = [nvcc, *_host_compiler_flags(), *NVCC_FLAGS, *extra, "-I", INCLUDE, "-c", srcp, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, _sources()))
    cmd = [nvcc, *_host_compiler_flags(), "-gencode", "arch=compute_100a,code=sm_100a", "--shared",
           "-Xcompiler", "-fPIC", "-o", LIB_PATH, *objs, "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


def build_step_model() -> str:
    """The stand-alone model of the decode step (csrc/step_model.cu): a diagnostic program, not part of the library."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    exe = os.path.join(OBJ_DIR, "step_model")
    cmd = [_nvcc(), *_host_compiler_flags(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           os.path.join(CSRC, "step_model.cu"), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for step_model.cu:\n{r.stdout}\n{r.stderr}")
    return exe


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--step-model", action="store_true", help="also build the decode-step timing model (build/step_model)")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    if a.step_model:
        print(build_step_model())
