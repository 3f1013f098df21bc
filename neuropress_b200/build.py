"""Ahead-of-time build of ``libneuropress_b200.so`` (sm_100a only) with plain nvcc.

The reference JIT-builds one torch extension per ``.cu`` at first use
(neuropress/kernels/__init__.py:58-106).  Here a single C-ABI shared library is built once,
in-tree, next to this file; it has no torch or Python dependency.

Usage: ``python -m neuropress_b200.build [--force] [--verbose]``
"""

from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
OBJ_DIR = CSRC / "build"
LIB_PATH = PKG_DIR / "libneuropress_b200.so"
# Measurement probes of the benchmark: a library of their own, outside the product's C ABI.
BENCH_LIB_PATH = PKG_DIR / "libneuropress_b200_bench.so"
BENCH_SOURCES = ["bench_probes.cu"]

SOURCES = [
    "c_api.cu",
    "vq_decode.cu",
    "vq_gemv.cu",
    "q_kernels.cu",
    "q_gemv_mma.cu",
    "q_gemv_ring.cu",
    "gemm_tcgen05.cu",
    "vq_gemm_fused.cu",
    "static_scratch.cu",
    "allgather_push.cu", "rms_norm.cu", "vq_gemv_mma.cu", "embedding.cu", "vq_entropy.cu", "vq_decode_copy.cu", "q_gemm_staged.cu", "vq_lut.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def find_nvcc() -> str:
    """Locate nvcc: PATH, then CUDA_HOME / CUDA_PATH, then /usr/local/cuda."""
    found = shutil.which("nvcc")
    if found:
        return found
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home and (Path(home) / "bin" / "nvcc").is_file():
            return str(Path(home) / "bin" / "nvcc")
    raise RuntimeError("nvcc not found (PATH, CUDA_HOME, /usr/local/cuda)")


def _newest_header_mtime() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    log = proc.stderr
    (obj.with_suffix(".ptxas.log")).write_text(log)
    if verbose:
        print(log)
    return log


def _build_library(nvcc: str, names: list[str], lib_path: Path, force: bool, verbose: bool) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    hdr_m = _newest_header_mtime()
    sources = [CSRC / s for s in names]
    jobs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        stale = force or not obj.is_file() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            futs = [ex.submit(_compile_one, nvcc, s, o, verbose) for s, o in jobs]
            for f in futs:
                f.result()
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    relink = bool(jobs) or not lib_path.is_file() or any(
        o.stat().st_mtime > lib_path.stat().st_mtime for o in objs
    )
    if relink:
        cmd = [nvcc, "-shared", "-o", str(lib_path), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "shared"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return lib_path


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` listed in ``SOURCES`` and link the shared library; then the
    benchmark's probe library (``BENCH_SOURCES``).

    Returns the path of the product library.  Objects are rebuilt only when their source or any
    header is newer (``force`` rebuilds everything).
    """
    nvcc = find_nvcc()
    path = _build_library(nvcc, SOURCES, LIB_PATH, force, verbose)
    _build_library(nvcc, BENCH_SOURCES, BENCH_LIB_PATH, force, verbose)
    return path


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args(argv)
    print(build(force=args.force, verbose=args.verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main())
