"""Build libb200moe.so (sm_100a only) in-tree with plain nvcc.

    python b300-moe-decode-fastpath_b200/build.py [--force] [--verbose]

The library has no Python, PyTorch, CUTLASS or pybind dependency: ten `.cu`
files, the CUDA runtime (static) and nothing else.  Exactly one `-gencode` is
passed, like the reference's single-architecture build
(fastpath/build.py:52-57, setup.py:49-54), but for `sm_100a`.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_ROOT = Path(__file__).resolve().parent
CSRC = PACKAGE_ROOT / "csrc"
INCLUDE = PACKAGE_ROOT.parent / "include"
SOURCES = ("api.cu", "routing.cu", "rows.cu", "grouped_gemm.cu", "grouped_gemm_fp8.cu",
           "grouped_gemm_nvfp4.cu", "quant.cu", "nvfp4_quant.cu", "ep_reduce.cu", "router.cu")
HEADERS = (CSRC / "common.cuh", INCLUDE / "b200moe.h")
LIBRARY = PACKAGE_ROOT / "b200moe" / "libb200moe.so"
GENCODE = "arch=compute_100a,code=sm_100a"


def nvcc_path() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    if candidate.exists():
        return str(candidate)
    found = shutil.which("nvcc")
    if found is None:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def is_stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    inputs = [CSRC / name for name in SOURCES] + list(HEADERS)
    return any(path.stat().st_mtime > built for path in inputs)


def command(verbose: bool = False) -> list[str]:
    cmd = [
        nvcc_path(),
        "-std=c++17",
        "-O3",
        "-gencode",
        GENCODE,
        "-lineinfo",
        "-shared",
        "-Xcompiler",
        "-fPIC",
        "-I",
        str(INCLUDE),
        "-o",
        str(LIBRARY),
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(CSRC / name) for name in SOURCES]
    return cmd


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources."""

    if not force and not is_stale():
        return LIBRARY
    cmd = command(verbose)
    result = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stderr.write(result.stdout)
        sys.stderr.write(result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}: {' '.join(cmd)}")
    return LIBRARY


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true", help="rebuild even if up to date")
    parser.add_argument("--verbose", action="store_true", help="print ptxas resource usage")
    args = parser.parse_args()
    path = build_library(force=args.force, verbose=args.verbose)
    print(path)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
