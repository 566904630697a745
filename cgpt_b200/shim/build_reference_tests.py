"""Builds CGPT's own test executables, UNCHANGED, against the drop-in: ``cgpt_b200_shim.cpp`` + ``libcgpt_b200.so``.

What a maintainer does with CMake is done here with direct compiler calls (CGPT's CMakeLists.txt pins sm_86/sm_90a and
needs CMake >= 4.3). From a CGPT checkout (``--reference`` or ``$CGPT_REFERENCE``; nothing in it is modified, nothing is
copied into this repository) it compiles, for sm_100a:

* the sources of ``cgpt_core`` that STAY CGPT's (CMakeLists.txt:36-56 minus the replaced files): Tensor, KV cache, CUDA
  graph wrapper, weight initialisation, the forward operators, the CPU operators, and a build-time copy of
  ``src/ops/linear.cu`` with the one declaration nvcc 12.9 cannot parse rewritten (see ``LINEAR_EDITS``);
* ``cgpt_b200_shim.cpp`` in place of the replaced files (listed in ``REPLACED``), against CGPT's unmodified headers;
* each test source of ``TESTS`` plus CGPT's CUPTI profiler unit ``tests/cuda_kernel_profiler.cpp`` (built with
  ``-DCUpti_ActivityKernel12=CUpti_ActivityKernel9``: it names a CUDA 13 record type, CUDA 12.9 has version 9),

and links every test twice into ``cgpt_b200/shim/_build/``:

* ``shim/<test>``      = test + kept CGPT objects + shim + ``libcgpt_b200.so``  (the drop-in under test)
* ``reference/<test>`` = test + kept CGPT objects + the replaced CGPT files themselves (the control: how CGPT's own code
  fares on the same GPU, so that a failure that both share is seen as CGPT's)

``tests/test_reference_tests_gpu.py`` runs them on a GPU. Usage: ``python -m cgpt_b200.shim.build_reference_tests``.
Does nothing (and says so) when the checkout is absent, e.g. on a GPU box, where the prebuilt executables are used.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
OUT = HERE / "_build"
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

KEPT = [
    "src/core/tensor.cu", "src/core/kv_cache.cu", "src/core/cuda_graph.cu", "src/core/weight_initialization.cu",
    "src/ops/attention.cu", "src/ops/embedding.cu", "src/ops/rmsnorm.cu", "src/ops/rope.cu", "src/ops/swiglu.cu", "src/ops/softmax.cu",
    "src/ops/cpu/attention_cpu.cpp", "src/ops/cpu/cross_entropy_cpu.cpp", "src/ops/cpu/embedding_cpu.cpp", "src/ops/cpu/linear_cpu.cpp",
    "src/ops/cpu/rmsnorm_cpu.cpp", "src/ops/cpu/rope_cpu.cpp", "src/ops/cpu/softmax_cpu.cpp", "src/ops/cpu/swiglu_cpu.cpp",
    "src/ops/cpu/backward/attention_backward_cpu.cpp", "src/ops/cpu/backward/cross_entropy_backward_cpu.cpp",
    "src/ops/cpu/backward/embedding_backward_cpu.cpp", "src/ops/cpu/backward/linear_backward_cpu.cpp",
    "src/ops/cpu/backward/rmsnorm_backward_cpu.cpp", "src/ops/cpu/backward/rope_backward_cpu.cpp",
    "src/ops/cpu/backward/swiglu_backward_cpu.cpp",
]
REPLACED = [
    "src/ops/backward/attention_backward.cu", "src/ops/backward/linear_backward.cu", "src/ops/backward/rmsnorm_backward.cu",
    "src/ops/backward/rope_backward.cu", "src/ops/backward/swiglu_backward.cu", "src/ops/backward/embedding_backward.cu",
    "src/ops/cross_entropy.cu", "src/ops/cut_cross_entropy.cu", "src/optim/adamw.cu", "src/core/transformer_block.cu",
    "src/core/transformer_model.cu",
]
FAST_MATH = {"src/ops/cross_entropy.cu", "src/ops/softmax.cu"}   # CMakeLists.txt:54
LINEAR_SOURCE = "src/ops/linear.cu"
LINEAR_EDITS = [   # nvcc 12.9's front end stops with an internal error at this std::vector declaration (linear.cu:271)
    ("std::vector<cublasLtMatmulHeuristicResult_t> heuristics(max_algorithms);", "cublasLtMatmulHeuristicResult_t heuristics[max_algorithms];"),
    ("heuristics.data(),", "heuristics,"),
]
TESTS = ["flash_attention_test", "linear_backward_test", "rmsnorm_test", "rope_test", "embedding_test", "cut_cross_entropy_test",
         "cross_entropy_test", "adamw_test", "fp16_numerical_stability_test", "transformer_model_test", "transformer_block_test"]


def _run(cmd):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + proc.stdout + proc.stderr)


def build(reference: Path, force: bool = False) -> Path | None:
    if not (reference / "tests" / "adamw_test.cu").is_file():
        print(f"[shim] CGPT checkout not found at {reference}; keeping prebuilt executables", file=sys.stderr)
        return OUT if OUT.is_dir() else None
    lib = ROOT / "cgpt_b200" / "libcgpt_b200.so"
    if not lib.exists():
        raise RuntimeError("build libcgpt_b200.so first (python -m cgpt_b200.build)")
    obj = OUT / "obj"
    for d in (obj, OUT / "shim", OUT / "reference"):
        d.mkdir(parents=True, exist_ok=True)
    inc = ["-I", str(reference / "include"), "-I", str(reference / "include" / "core"), "-I", str(CUDA / "include")]
    cxx = ["/usr/bin/g++", "-std=c++20", "-O3", "-mavx2", "-mfma", "-mf16c", "-fopenmp", "-fPIC", "-include", "cstdint",
           "-DCGPT_ENABLE_OPENMP=1", *inc]
    nvcc = [str(CUDA / "bin" / "nvcc"), "-ccbin", "/usr/bin/g++", "-std=c++20", "-O3", "-include", "cstdint",
            "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC,-fopenmp", "-DCGPT_ENABLE_OPENMP=1", *inc]

    linear_copy = obj / "linear_patched.cu"
    text = (reference / LINEAR_SOURCE).read_text()
    for old, new in LINEAR_EDITS:
        if text.count(old) != 1:
            raise RuntimeError(f"{LINEAR_SOURCE}: expected exactly one occurrence of {old!r}")
        text = text.replace(old, new)
    linear_copy.write_text(text)

    jobs = []

    def add(src: Path, out: Path, cmd_prefix, extra=()):
        newest = max(src.stat().st_mtime, Path(__file__).stat().st_mtime)
        if force or not out.exists() or out.stat().st_mtime < newest:
            jobs.append([*cmd_prefix, *extra, "-c", str(src), "-o", str(out)])
        return out

    def compile_list(rels):
        outs = []
        for rel in rels:
            src = reference / rel
            out = obj / (rel.replace("/", "_") + ".o")
            outs.append(add(src, out, nvcc if rel.endswith(".cu") else cxx, ["--use_fast_math"] if rel in FAST_MATH else []))
        return outs

    kept = compile_list(KEPT) + [add(linear_copy, obj / "linear_patched.o", nvcc)]
    replaced = compile_list(REPLACED)
    shim_src = HERE / "cgpt_b200_shim.cpp"
    shim = obj / "cgpt_b200_shim.o"
    if force or not shim.exists() or shim.stat().st_mtime < max(shim_src.stat().st_mtime, (ROOT / "include" / "cgpt_b200.h").stat().st_mtime):
        jobs.append([*cxx, "-I", str(ROOT / "include"), "-c", str(shim_src), "-o", str(shim)])
    profiler = add(reference / "tests" / "cuda_kernel_profiler.cpp", obj / "cuda_kernel_profiler.o", cxx,
                   ["-DCUpti_ActivityKernel12=CUpti_ActivityKernel9", "-I", str(CUDA / "extras" / "CUPTI" / "include")])
    tests = {t: add(reference / "tests" / f"{t}.cu", obj / f"{t}.o", nvcc, ["-I", str(reference / "tests")]) for t in TESTS}

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(_run, jobs))

    libs = ["-L", str(CUDA / "lib64"), "-L", str(CUDA / "extras" / "CUPTI" / "lib64"), "-lcublasLt", "-lcudart", "-lcupti", "-lgomp",
            "-Wl,-rpath," + str(CUDA / "lib64"), "-Wl,-rpath," + str(CUDA / "extras" / "CUPTI" / "lib64")]
    links = []
    for t, o in tests.items():
        # the drop-in: $ORIGIN/../../.. is the package directory that holds libcgpt_b200.so
        links.append(["/usr/bin/g++", "-o", str(OUT / "shim" / t), str(o), str(profiler), str(shim), *map(str, kept),
                      "-L", str(lib.parent), "-lcgpt_b200", "-Wl,-rpath,$ORIGIN/../../..", *libs])
        links.append(["/usr/bin/g++", "-o", str(OUT / "reference" / t), str(o), str(profiler), *map(str, replaced), *map(str, kept), *libs])
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(_run, links))
    linear_copy.unlink(missing_ok=True)
    return OUT


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--reference", default=os.environ.get("CGPT_REFERENCE", str(ROOT.parent / "reference")))
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    print(build(Path(args.reference), args.force))


if __name__ == "__main__":
    main()
