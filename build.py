#!/usr/bin/env python3
"""Build the native libraries in-tree (no pip, no JIT cache):

  distributed-llama-multiusers_b200/lib/libdllama_b200_cuda.so   nvcc, sm_100a only: the Q40 / f32 Llama kernels
  distributed-llama-multiusers_b200/lib/libdllama_b200_layers.so nvcc, sm_100a only: the kernels of layer-list models
                                                                 (dense bf16 / f32 weights, latent, windowed and linear attention, Mamba-2)
  distributed-llama-multiusers_b200/lib/libdllama_b200_host.so   g++, CPU runtime (tokenizer,
                                                                 sampler, codecs, scheduler ...)

Usage: python build.py [--force] [--verbose] [cuda|layers|host ...]   (no target: all three)
Objects are rebuilt only when a source or header is newer (so repeated calls are cheap).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "distributed-llama-multiusers_b200")
CUDA_SRC = os.path.join(PKG, "csrc", "cuda")
HOST_SRC = os.path.join(PKG, "csrc", "host")
LIB = os.path.join(PKG, "lib")
OBJ = os.path.join(ROOT, "build", "obj")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-pthread"]
# Debug / sanitizer builds (reference: `make DEBUG=1` -> -g -fsanitize=address, Makefile:8-9): extra flags from the
# environment are appended, e.g.  CXXFLAGS="-g -O1 -fsanitize=address" python build.py --force   (run python with
# LD_PRELOAD=$(g++ -print-file-name=libasan.so)), NVCCFLAGS="-G" for device debug info.
CXX_FLAGS += os.environ.get("CXXFLAGS", "").split()
NVCC_FLAGS += os.environ.get("NVCCFLAGS", "").split()


def _find_nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose, log_path=None):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path:
        with open(log_path, "w") as f:
            f.write(" ".join(cmd) + "\n" + p.stdout)
    if p.returncode != 0:
        sys.stderr.write(p.stdout)
        raise RuntimeError("build failed: " + " ".join(cmd))
    if verbose:
        sys.stdout.write(p.stdout)


# sources of the layer-list model library; prep.cu (error plumbing, argmax), sampler.cu and gemm_wh_tc.cu (the tcgen05
# GEMM on pre-tiled operands) are shared with the other one (their objects are compiled once), the rest is its own
LAYERS_OWN = ["dense.cu", "hyper.cu", "latent_attention.cu", "lightning.cu", "mamba2.cu", "moe.cu", "norms.cu", "talk_attention.cu", "window_attention.cu"]
LAYERS_SHARED = ["gemm_wh_tc.cu", "prep.cu", "sampler.cu"]


def build_cuda(force=False, verbose=False) -> str:
    srcs = sorted(f for f in os.listdir(CUDA_SRC) if f.endswith(".cu") and f not in LAYERS_OWN)
    return _build_cuda_lib("libdllama_b200_cuda.so", srcs, force, verbose)


def build_layers(force=False, verbose=False) -> str:
    """Only what a layer-list model needs: a fresh checkout serves one without compiling the Q40 kernels."""
    return _build_cuda_lib("libdllama_b200_layers.so", sorted(LAYERS_OWN + LAYERS_SHARED), force, verbose)


def _build_cuda_lib(name, srcs, force, verbose) -> str:
    nvcc = _find_nvcc()
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    headers = [os.path.join(CUDA_SRC, f) for f in os.listdir(CUDA_SRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "dllama_b200.h"))
    objs, jobs = [], []
    for s in srcs:
        src = os.path.join(CUDA_SRC, s)
        obj = os.path.join(OBJ, s[:-3] + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            jobs.append(([nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj], obj[:-2] + ".ptxas.log"))
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(lambda j: _run(j[0], verbose, j[1]), jobs))
    out = os.path.join(LIB, name)
    if force or jobs or _newer(out, objs):
        _run([nvcc, "-shared", "-o", out] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"], verbose)
    return out


def build_host(force=False, verbose=False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    if not os.path.isdir(HOST_SRC):
        return ""
    headers = [os.path.join(HOST_SRC, f) for f in os.listdir(HOST_SRC) if f.endswith((".hpp", ".h"))]
    srcs = sorted(f for f in os.listdir(HOST_SRC) if f.endswith(".cpp"))
    if not srcs:
        return ""
    objs, jobs = [], []
    for s in srcs:
        src = os.path.join(HOST_SRC, s)
        obj = os.path.join(OBJ, "host_" + s[:-4] + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            jobs.append((["g++"] + CXX_FLAGS + ["-c", src, "-o", obj], None))
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(lambda j: _run(j[0], verbose, j[1]), jobs))
    out = os.path.join(LIB, "libdllama_b200_host.so")
    if force or jobs or _newer(out, objs):
        _run(["g++", "-shared", "-o", out] + objs + ["-pthread"] + [f for f in CXX_FLAGS if f.startswith("-fsanitize")], verbose)
    return out


def build_all(force=False, verbose=False):
    cuda = build_cuda(force, verbose)
    build_layers(False, verbose)          # after the first library: the shared objects are fresh by now
    return cuda, build_host(force, verbose)


if __name__ == "__main__":
    force, verbose = "--force" in sys.argv, "--verbose" in sys.argv
    targets = [a for a in sys.argv[1:] if not a.startswith("-")]
    if not targets:
        a, b = build_all(force, verbose)
        print("built:", a, b, os.path.join(LIB, "libdllama_b200_layers.so"))
    else:
        fns = {"cuda": build_cuda, "layers": build_layers, "host": build_host}
        for t in targets:
            print("built:", fns[t](force, verbose))
