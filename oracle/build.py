"""Builds the C oracle (oracle/libqf_oracle.so) with gcc.

    python oracle/build.py [--force]

Test infrastructure only: nothing in the product imports or links this.
The hot loops are compiled twice (x86-64-v3 and baseline) and dispatched by
the dynamic loader, so one binary runs on any x86-64 host; fp contraction is
off so both clones give identical bits.
"""

from __future__ import annotations

import shutil
import subprocess
import sys
from pathlib import Path

ORACLE_DIR = Path(__file__).resolve().parent
SOURCE = ORACLE_DIR / "qf_oracle.c"
LIBRARY = ORACLE_DIR / "libqf_oracle.so"
FLAGS = ["-O3", "-fPIC", "-shared", "-std=gnu11", "-ffp-contract=off", "-fno-math-errno",
         "-fopenmp", "-Wall"]


def build_oracle(force: bool = False) -> Path:
    if not force and LIBRARY.is_file() and LIBRARY.stat().st_mtime >= max(
            SOURCE.stat().st_mtime, Path(__file__).stat().st_mtime):
        return LIBRARY
    gcc = shutil.which("gcc") or shutil.which("cc")
    if gcc is None:
        raise RuntimeError("gcc not found; the oracle needs a C compiler")
    command = [gcc, *FLAGS, str(SOURCE), "-o", str(LIBRARY), "-lm"]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode:
        # Some toolchains cannot clone functions that contain OpenMP regions.
        result = subprocess.run(command[:1] + ["-DQFO_NO_CLONES"] + command[1:],
                                capture_output=True, text=True)
    if result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
        raise RuntimeError("building the oracle failed")
    return LIBRARY


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
