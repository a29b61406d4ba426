"""Build the C-ABI shared library (dmf_b200/libdmf_attn.so) with nvcc for sm_100a.

The library is built in-tree so that it travels with the source snapshot; it has
no Python or torch dependency.  ``python -m dmf_b200.build`` builds it by hand.
"""

from __future__ import annotations

import fcntl
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libdmf_attn.so"

SOURCES = ["dmf_attn.cu", "dmf_adaln.cu", "dmf_step.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "-shared",
]


def find_nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and Path(cand).exists() else None


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources.

    Several processes may get here at once (one rank per GPU under torchrun, spawned test workers): the stale
    check and the compile run under an exclusive lock on a sidecar file, so one process builds and the others
    wait and then find the library fresh; nvcc writes to a temporary name that is moved onto the library in
    one step, so nobody ever loads a half-written file.
    """
    if not force and not _stale():
        return LIB
    with open(PKG / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not _stale():      # somebody else built it while this process waited
                return LIB
            nvcc = find_nvcc()
            if nvcc is None:
                raise RuntimeError("nvcc not found: cannot build dmf_b200/libdmf_attn.so")
            tmp = LIB.with_name(f".{LIB.name}.{os.getpid()}.tmp")
            cmd = [nvcc, *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "--threads", "0"]
            if verbose:
                cmd += ["-Xptxas", "-v"]
            cmd += ["-o", str(tmp), *[str(CSRC / s) for s in SOURCES]]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
            os.replace(tmp, LIB)
            if verbose:
                sys.stderr.write(res.stderr)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
