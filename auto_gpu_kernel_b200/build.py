"""Build libdsa_b200.so (sm_100a only) from csrc/*.cu with nvcc, in-tree.

    python -m auto_gpu_kernel_b200.build [--force] [--verbose]

The library is rebuilt when any source or header is newer than it.  nvcc cross-compiles without a
GPU.  The same function is used by the solution directory that ships through kbench as text: there
the sources are compiled on first import.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_NAME = "libdsa_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: set NVCC or put the CUDA toolkit on PATH")
    return cand


def sources(csrc: Path = CSRC):
    return sorted(csrc.glob("*.cu"))


def needs_build(out: Path, csrc: Path = CSRC) -> bool:
    if not out.exists():
        return True
    stamp = out.stat().st_mtime
    deps = list(csrc.glob("*.cu")) + list(csrc.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(p.stat().st_mtime > stamp for p in deps)


def build(out: Path | None = None, csrc: Path = CSRC, force: bool = False, verbose: bool = False,
          extra_flags=()) -> Path:
    """Compile the library when it is missing or older than a source.  Safe when several
    processes (one rank per GPU) call it at once: one of them compiles, into a scratch file that
    is renamed into place, the others wait at a lock file and find the work done."""
    import fcntl
    out = Path(out) if out else PKG_DIR / LIB_NAME
    if not force and not needs_build(out, csrc):
        return out
    out.parent.mkdir(parents=True, exist_ok=True)
    with open(out.with_name(out.name + ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not needs_build(out, csrc):
                return out                       # another process built it while we waited
            scratch = out.with_name(f"{out.name}.{os.getpid()}.tmp")
            cmd = [find_nvcc(), *NVCC_FLAGS, *extra_flags]
            if verbose:
                cmd += ["-Xptxas", "-v"]
            cmd += [str(p) for p in sources(csrc)] + ["-o", str(scratch)]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or proc.returncode != 0:
                sys.stderr.write(proc.stdout + proc.stderr)
            if proc.returncode != 0:
                scratch.unlink(missing_ok=True)
                raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}")
            os.replace(scratch, out)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return out


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
