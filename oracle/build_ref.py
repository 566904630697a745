"""Builds the reference's own CPU operators into ``oracle/_ref/libcgpt_ref_cpu.so`` and its own CUDA operators, for
sm_100a, into ``oracle/_ref/libcgpt_ref_cuda.so`` (TEST INFRASTRUCTURE).

Sources are compiled where they lie under the reference checkout (``--reference`` or ``$CGPT_REFERENCE``); nothing
is copied. The only file of this repository in the link is ``oracle/ref_wrap.cpp``, a flat C wrapper.
The recipe replaces the reference's CMake build (which pins sm_86/sm_90a and needs CMake >= 4.3) with
direct compiler calls and the flags of its ``CMakeLists.txt:57-66`` (``-O3 -mavx2 -mfma -mf16c``,
OpenMP on), plus ``-include cstdint`` because ``include/core/dtype.h:12`` uses ``std::uint8_t`` without
including ``<cstdint>``.

Usage: ``python oracle/build_ref.py [--reference <checkout>]``. Does nothing (and says so) when the
reference checkout is absent, e.g. on a GPU box, where the prebuilt library is used.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
LIB = OUT / "libcgpt_ref_cpu.so"

CPU_SOURCES = [
    "src/ops/cpu/attention_cpu.cpp", "src/ops/cpu/cross_entropy_cpu.cpp", "src/ops/cpu/embedding_cpu.cpp",
    "src/ops/cpu/linear_cpu.cpp", "src/ops/cpu/rmsnorm_cpu.cpp", "src/ops/cpu/rope_cpu.cpp",
    "src/ops/cpu/softmax_cpu.cpp", "src/ops/cpu/swiglu_cpu.cpp",
    "src/ops/cpu/backward/attention_backward_cpu.cpp", "src/ops/cpu/backward/cross_entropy_backward_cpu.cpp",
    "src/ops/cpu/backward/embedding_backward_cpu.cpp", "src/ops/cpu/backward/linear_backward_cpu.cpp",
    "src/ops/cpu/backward/rmsnorm_backward_cpu.cpp", "src/ops/cpu/backward/rope_backward_cpu.cpp",
    "src/ops/cpu/backward/swiglu_backward_cpu.cpp",
]
CUDA_SOURCES = ["src/core/tensor.cu", "src/optim/adamw.cu"]  # host code paths only are exercised

# The reference's GPU code on the path, for the second library oracle/_ref/libcgpt_ref_cuda.so: its own operators, block,
# model, optimizer and graph wrapper, rebuilt for sm_100a. src/ops/linear.cu goes in as a build-time copy (below).
LIB_CUDA = OUT / "libcgpt_ref_cuda.so"
GPU_SOURCES = [
    "src/core/tensor.cu", "src/ops/attention.cu", "src/ops/cross_entropy.cu", "src/ops/cut_cross_entropy.cu",
    "src/ops/embedding.cu", "src/ops/rmsnorm.cu", "src/ops/rope.cu", "src/ops/softmax.cu", "src/ops/swiglu.cu",
    "src/ops/backward/attention_backward.cu", "src/ops/backward/embedding_backward.cu",
    "src/ops/backward/rmsnorm_backward.cu", "src/ops/backward/rope_backward.cu", "src/ops/backward/swiglu_backward.cu",
    "src/ops/backward/linear_backward.cu", "src/core/transformer_block.cu", "src/core/transformer_model.cu",
    "src/core/kv_cache.cu", "src/core/cuda_graph.cu", "src/core/weight_initialization.cu", "src/optim/adamw.cu",
]
# src/ops/linear.cu stops nvcc 12.9's front end with an internal error at the declaration
# `std::vector<cublasLtMatmulHeuristicResult_t> heuristics(max_algorithms);` (linear.cu:271). The build writes a copy under
# oracle/_ref/ in which that vector is a C array (two textual edits, :271 and :282) and compiles the copy; the checkout is
# not touched and the copy is never committed.
LINEAR_SOURCE = "src/ops/linear.cu"
LINEAR_EDITS = [
    ("std::vector<cublasLtMatmulHeuristicResult_t> heuristics(max_algorithms);",
     "cublasLtMatmulHeuristicResult_t heuristics[max_algorithms];"),
    ("heuristics.data(),", "heuristics,"),
]
WRAPPERS = ["ref_wrap_cuda.cpp", "ref_wrap_model.cpp"]


def patched_linear(reference: Path) -> Path:
    text = (reference / LINEAR_SOURCE).read_text()
    for old, new in LINEAR_EDITS:
        if text.count(old) != 1:
            raise RuntimeError(f"{LINEAR_SOURCE}: expected exactly one occurrence of {old!r}")
        text = text.replace(old, new)
    out = OUT / "linear_patched.cu"
    out.write_text(text)
    return out
# per-file options of the reference's CMakeLists.txt:54
FAST_MATH = {"src/ops/cross_entropy.cu", "src/ops/softmax.cu"}


def build(reference: Path, force: bool = False) -> Path | None:
    if not (reference / "src" / "ops" / "cpu").is_dir():
        print(f"[oracle/_ref] reference checkout not found at {reference}; keeping prebuilt files", file=sys.stderr)
        return LIB if LIB.exists() else None
    OUT.mkdir(parents=True, exist_ok=True)
    wrap = HERE / "ref_wrap.cpp"
    inputs = [reference / s for s in CPU_SOURCES + CUDA_SOURCES] + [wrap]
    if LIB.exists() and not force and all(LIB.stat().st_mtime > p.stat().st_mtime for p in inputs):
        build_cuda(reference, force)
        return LIB
    inc = ["-I", str(reference / "include"), "-I", str(reference / "include" / "core"), "-I", "/usr/local/cuda/include"]
    cxx = ["/usr/bin/g++", "-std=c++20", "-O3", "-mavx2", "-mfma", "-mf16c", "-fopenmp", "-fPIC", "-include", "cstdint",
           "-DCGPT_ENABLE_OPENMP=1", *inc]
    nvcc = ["/usr/local/cuda/bin/nvcc", "-ccbin", "/usr/bin/g++", "-std=c++20", "-O3", "-include", "cstdint",
            "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC,-fopenmp", *inc]
    jobs = []
    objects = []
    for rel in CPU_SOURCES:
        obj = OUT / (rel.replace("/", "_") + ".o")
        objects.append(obj)
        jobs.append([*cxx, "-c", str(reference / rel), "-o", str(obj)])
    for rel in CUDA_SOURCES:
        obj = OUT / (rel.replace("/", "_") + ".o")
        objects.append(obj)
        jobs.append([*nvcc, "-c", str(reference / rel), "-o", str(obj)])
    obj = OUT / "ref_wrap.o"
    objects.append(obj)
    jobs.append([*cxx, "-c", str(wrap), "-o", str(obj)])

    def run(cmd):
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(run, jobs))
    run(["/usr/local/cuda/bin/nvcc", "-ccbin", "/usr/bin/g++", "-shared", "-cudart", "shared", "-Xcompiler", "-fopenmp",
         "-gencode", "arch=compute_100a,code=sm_100a", "-Xlinker", "-rpath,/usr/local/cuda/lib64", "-o", str(LIB),
         *map(str, objects)])
    for o in objects:
        o.unlink(missing_ok=True)
    build_cuda(reference, force)
    return LIB


def build_cuda(reference: Path, force: bool = False) -> Path | None:
    """The reference's CUDA operators + oracle/ref_wrap_cuda.cpp -> oracle/_ref/libcgpt_ref_cuda.so (sm_100a)."""
    wraps = [HERE / w for w in WRAPPERS]
    inputs = [reference / s for s in GPU_SOURCES + CPU_SOURCES + [LINEAR_SOURCE]] + wraps + [Path(__file__)]
    if LIB_CUDA.exists() and not force and all(LIB_CUDA.stat().st_mtime > p.stat().st_mtime for p in inputs):
        return LIB_CUDA
    inc = ["-I", str(reference / "include"), "-I", str(reference / "include" / "core"), "-I", "/usr/local/cuda/include"]
    nvcc = ["/usr/local/cuda/bin/nvcc", "-ccbin", "/usr/bin/g++", "-std=c++20", "-O3", "-include", "cstdint",
            "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC,-fopenmp", "-DCGPT_ENABLE_OPENMP=1", *inc]
    cxx = ["/usr/bin/g++", "-std=c++20", "-O3", "-mavx2", "-mfma", "-mf16c", "-fopenmp", "-fPIC", "-include", "cstdint",
           "-DCGPT_ENABLE_OPENMP=1", *inc]
    jobs, objects = [], []
    for rel in GPU_SOURCES:
        obj = OUT / ("gpu_" + rel.replace("/", "_") + ".o")
        objects.append(obj)
        jobs.append([*nvcc, *(["--use_fast_math"] if rel in FAST_MATH else []), "-c", str(reference / rel), "-o", str(obj)])
    linear_copy = patched_linear(reference)
    obj = OUT / "gpu_linear_patched.o"
    objects.append(obj)
    jobs.append([*nvcc, "-c", str(linear_copy), "-o", str(obj)])
    for rel in CPU_SOURCES:   # the GPU entry points dispatch to these for CPU tensors, so the symbols must resolve
        obj = OUT / ("gpu_" + rel.replace("/", "_") + ".o")
        objects.append(obj)
        jobs.append([*cxx, "-c", str(reference / rel), "-o", str(obj)])
    for wrap in wraps:
        obj = OUT / (wrap.stem + ".o")
        objects.append(obj)
        jobs.append([*cxx, "-c", str(wrap), "-o", str(obj)])

    def run(cmd):
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(run, jobs))
    run(["/usr/local/cuda/bin/nvcc", "-ccbin", "/usr/bin/g++", "-shared", "-cudart", "shared", "-Xcompiler", "-fopenmp",
         "-gencode", "arch=compute_100a,code=sm_100a", "-Xlinker", "-rpath,/usr/local/cuda/lib64", "-Xlinker", "--no-undefined",
         "-o", str(LIB_CUDA), *map(str, objects), "-lcublasLt", "-lcublas"])
    for o in objects:
        o.unlink(missing_ok=True)
    linear_copy.unlink(missing_ok=True)
    return LIB_CUDA


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", default=os.environ.get("CGPT_REFERENCE", str(HERE.parent.parent / "reference")))
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    print(build(Path(args.reference), args.force))


if __name__ == "__main__":
    main()
