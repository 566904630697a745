"""Builds ``cgpt_b200/libcgpt_b200.so`` (sm_100a only) from ``cgpt_b200/csrc`` with nvcc.

Run as ``python -m cgpt_b200.build`` (add ``--force`` to rebuild everything, ``--verbose`` to see
``-Xptxas -v`` register/shared-memory reports, ``--diagnosis`` to compile in the environment-driven diagnosis
switches, which the normal build leaves out). Objects are cached under ``build/obj`` and rebuilt
when the source or any header under ``csrc``/``include`` is newer. No GPU is needed to build.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "cgpt_b200" / "csrc"
OBJ = ROOT / "build" / "obj"
LIB = ROOT / "cgpt_b200" / "libcgpt_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = [
    "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
    "-cudart", "shared", "-ccbin", "/usr/bin/g++",
    "-diag-suppress", "177",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: cgpt_b200 cannot be built without the CUDA toolkit")


def _headers_mtime() -> float:
    newest = 0.0
    for pattern, base in (("*.cuh", CSRC), ("*.h", CSRC), ("*.h", ROOT / "include")):
        for path in base.glob(pattern):
            newest = max(newest, path.stat().st_mtime)
    return newest


def _compile(nvcc: str, src: Path, obj: Path, verbose: bool, diagnosis: bool = False) -> str:
    cmd = [nvcc, *ARCH_FLAGS, *COMMON, "-I", str(ROOT / "include"), "-c", str(src), "-o", str(obj)]
    if diagnosis:
        cmd[1:1] = ["-DCGPT_B200_DIAGNOSIS"]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False, diagnosis: bool = False) -> Path:
    force = force or diagnosis
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    sources = sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))
    if not sources:
        raise RuntimeError(f"no sources under {CSRC}")
    hdr_time = _headers_mtime()
    jobs = []
    objects = []
    for src in sources:
        obj = OBJ / (src.name + ".o")
        objects.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            jobs.append((src, obj))
    if jobs:
        workers = min(len(jobs), os.cpu_count() or 4)
        with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
            futures = {pool.submit(_compile, nvcc, s, o, verbose, diagnosis): s for s, o in jobs}
            for fut in concurrent.futures.as_completed(futures):
                report = fut.result()
                if report:
                    print(f"== {futures[fut].name}\n{report}", file=sys.stderr)
    relink = bool(jobs) or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objects)
    if relink:
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-cudart", "shared", "-ccbin", "/usr/bin/g++",
               "-Xlinker", "-rpath,/usr/local/cuda/lib64", "-o", str(LIB), *map(str, objects)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--diagnosis", action="store_true",
                    help="define CGPT_B200_DIAGNOSIS (rebuild with --force afterwards to return to the normal library)")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose, diagnosis=args.diagnosis))


if __name__ == "__main__":
    main()
