"""Builds libqf_hotpath.so (sm_100a only) in-tree with nvcc.

    python qwen-frence_b200/build.py            # incremental
    python qwen-frence_b200/build.py --force    # rebuild everything
    python qwen-frence_b200/build.py --verbose  # show ptxas resource usage

nvcc cross-compiles for sm_100a, so this works on a machine without a GPU.
The CUDA runtime is linked statically: the library has no torch dependency and
shares the primary context (and therefore streams and device pointers) with any
other runtime in the process.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
BUILD_DIR = PACKAGE_DIR / "build"
LIBRARY = PACKAGE_DIR / "libqf_hotpath.so"

SOURCES = ("qf_api.cu", "qf_rope_kv_write.cu", "qf_decode_attention.cu", "qf_decode_metadata.cu", "qf_rms_norm.cu", "qf_qkv_gemm_rope.cu")

ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
COMMON_FLAGS = ("-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-O2")


def find_nvcc() -> str:
    candidates = [os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for candidate in candidates:
        if candidate and Path(candidate).is_file():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or put the CUDA toolkit on PATH")


def _newest_dependency(source: Path) -> float:
    deps = [source, *CSRC.glob("*.cuh"), *INCLUDE.glob("*.h"), Path(__file__)]
    return max(path.stat().st_mtime for path in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel translation unit and link the shared library."""
    nvcc = find_nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    objects = []
    rebuilt = False
    for name in SOURCES:
        source = CSRC / name
        obj = BUILD_DIR / (source.stem + ".o")
        objects.append(obj)
        if not force and obj.is_file() and obj.stat().st_mtime >= _newest_dependency(source):
            continue
        command = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, "-I", str(INCLUDE), "-c", str(source), "-o", str(obj)]
        if verbose:
            command[1:1] = ["-Xptxas", "-v"]
        result = subprocess.run(command, capture_output=True, text=True)
        if verbose or result.returncode:
            sys.stderr.write(result.stdout + result.stderr)
        if result.returncode:
            raise RuntimeError(f"nvcc failed on {source.name}")
        rebuilt = True
    if rebuilt or force or not LIBRARY.is_file():
        command = [nvcc, *ARCH_FLAGS, "-shared", "-cudart", "static", "-o", str(LIBRARY), *map(str, objects)]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode:
            sys.stderr.write(result.stdout + result.stderr)
            raise RuntimeError("linking libqf_hotpath.so failed")
    return LIBRARY


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    print(build_library(force=args.force, verbose=args.verbose))


if __name__ == "__main__":
    main()
