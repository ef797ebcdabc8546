"""Builds librns_b200.so in-tree with nvcc for sm_100a.

Usage: ``python -m rns_llm_b200.csrc.build [--force]``.  The build is skipped
when the library is newer than every source file.  nvcc cross-compiles, so no
GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
SOURCES = ("rns_host.cu", "rns_aux.cu", "rns_gemm_sm100.cu", "rns_gemm_tmem_sm100.cu",
           "rns_gemm_pair_sm100.cu", "rns_gemm_pair_raw_sm100.cu", "rns_small_sm100.cu", "rns_stream_sm100.cu", "rns_static_scratch.cu")
HEADERS = (HERE / "rns_common.cuh", HERE / "rns_ptx.cuh", HERE / "rns_pair.cuh", HERE / "rns_mma_sync.cuh", REPO / "include" / "rns_b200.h")
LIBRARY = HERE / "librns_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build librns_b200.so")
    return found


def sources() -> list[Path]:
    return [HERE / name for name in SOURCES if (HERE / name).exists()]


def up_to_date() -> bool:
    if not LIBRARY.exists():
        return False
    built = LIBRARY.stat().st_mtime
    deps = sources() + [h for h in HEADERS if h.exists()]
    return all(dep.stat().st_mtime <= built for dep in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and up_to_date():
        return LIBRARY
    nvcc = _nvcc()
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
        if verbose:
            sys.stderr.write(proc.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(4, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, sources()))
    link = [nvcc, "-shared", "-o", str(LIBRARY), *map(str, objects)]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return LIBRARY


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
