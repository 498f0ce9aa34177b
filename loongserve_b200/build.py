"""Build the CUDA libraries in-tree with nvcc for sm_100a.

    python -m loongserve_b200.build [--force]

Produces, next to this file:
  libesp_attention.so  -- kernels + C ABI declared in include/esp_attention.h
  libesp_rnccl.so      -- raw NCCL point-to-point layer declared in include/esp_rnccl.h
Both link the shared CUDA runtime, so they use the same runtime instance as PyTorch in one process.
`build_selftest()` builds the test-suite's own kernels (tests/csrc/selftest_kernels.cu) into tests/libesp_selftest.so;
they are not part of the product library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)

ATTN_SOURCES = ["kv_scatter.cu", "decode_attention.cu", "prefill_attention.cu", "layer_ops.cu",
                "pool_allocator.cpp", "prefill_scheduler.cpp"]
ATTN_LIB = os.path.join(HERE, "libesp_attention.so")
RNCCL_LIB = os.path.join(HERE, "libesp_rnccl.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-cudart", "shared"]


def reference_dir():
    """A checkout of the reference project, for the builds and tests that compare against it: the directory named by
    ESP_REFERENCE_DIR, else a sibling directory `reference` next to this repository.  None when neither exists."""
    for cand in (os.environ.get("ESP_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "loongserve")):
            return os.path.abspath(cand)
    return None


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd: list[str]) -> None:
    print("+", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build_attention(force: bool = False, verbose_ptxas: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in ATTN_SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in ("esp_common.cuh", "sm100_ptx.cuh")] + \
        [os.path.join(ROOT, "include", "esp_attention.h")]
    if force or _newer(ATTN_LIB, deps):
        objs = []
        bdir = os.path.join(HERE, "build")
        os.makedirs(bdir, exist_ok=True)
        for s in srcs:
            o = os.path.join(bdir, os.path.basename(s) + ".o")
            if force or _newer(o, deps):
                host_only = ["-Xcompiler", "-ffp-contract=off"] if s.endswith(".cpp") else []
                _run([_nvcc()] + NVCC_FLAGS + host_only + (["-Xptxas", "-v"] if verbose_ptxas else []) + ["-c", s, "-o", o])
            objs.append(o)
        _run([_nvcc(), "-shared", "-cudart", "shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", ATTN_LIB] + objs)
    return ATTN_LIB


SELFTEST_SRC = os.path.join(ROOT, "tests", "csrc", "selftest_kernels.cu")
SELFTEST_LIB = os.path.join(ROOT, "tests", "libesp_selftest.so")


def build_selftest(force: bool = False) -> str:
    deps = [SELFTEST_SRC] + [os.path.join(CSRC, h) for h in ("esp_common.cuh", "sm100_ptx.cuh")]
    if force or _newer(SELFTEST_LIB, deps):
        _run([_nvcc()] + NVCC_FLAGS + ["-shared", SELFTEST_SRC, "-o", SELFTEST_LIB])
    return SELFTEST_LIB


def build_rnccl(force: bool = False) -> str:
    src = os.path.join(CSRC, "rnccl.cpp")
    deps = [src, os.path.join(ROOT, "include", "esp_rnccl.h")]
    if force or _newer(RNCCL_LIB, deps):
        cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-I{cuda_home}/include", src, "-o", RNCCL_LIB,
              f"-L{cuda_home}/lib64", "-lcudart", "-l:libnccl.so.2"])
    return RNCCL_LIB


def build_all(force: bool = False) -> None:
    build_attention(force)
    build_rnccl(force)
    if os.path.exists(SELFTEST_SRC):
        build_selftest(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
