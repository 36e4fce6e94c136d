"""Compile the sm_100a kernels with nvcc into one shared library, at first use.

The sources under ``tokenmill_b200/csrc`` have no dependency beyond the CUDA toolkit (no torch or
pybind headers), so a cold build takes well under a minute. The library is written next to the
sources (``csrc/_build``) when that folder can be written, else under the system's temporary folder;
its name carries a hash of the sources and flags, so an edited source is rebuilt and a stale library
is never loaded. While nvcc runs, a line is printed to stderr every few seconds.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# Precise math (no --use_fast_math): division, sqrt and expf keep their IEEE / documented accuracy.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


class KernelBuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc); the "
                           "engine has no path that runs without its compiled sm_100a kernels")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest(files: list[Path]) -> str:
    h = hashlib.sha256()
    for f in files + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> Path:
    override = os.environ.get("TOKENMILL_BUILD_DIR")
    cands = [Path(override)] if override else []
    cands += [CSRC / "_build", Path(tempfile.gettempdir()) / f"tokenmill_b200_build_{os.getuid()}"]
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".write_probe_{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for the kernel library (tried {[str(c) for c in cands]})")


def library_path() -> Path:
    """Where the library for the present sources lives (it may not be built yet)."""
    return _build_dir() / f"libtokenmill_kernels_{_digest(sources())}.so"


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}\n{proc.stdout}")


def build(verbose: bool = True, force: bool = False) -> Path:
    """Build the library if it is missing; return its path."""
    files = sources()
    if not files:
        raise KernelBuildError(f"no .cu sources in {CSRC}")
    out_dir = _build_dir()
    lib = out_dir / f"libtokenmill_kernels_{_digest(files)}.so"
    if lib.exists() and not force:
        return lib
    nvcc = find_nvcc()
    obj_dir = out_dir / f"obj_{lib.stem}_{os.getpid()}"
    obj_dir.mkdir(parents=True, exist_ok=True)
    t0 = time.time()
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(5.0):
            print(f"[tokenmill_b200] compiling sm_100a kernels ({len(files)} files) ... {time.time() - t0:.0f} s",
                  file=sys.stderr, flush=True)

    if verbose:
        print(f"[tokenmill_b200] compiling sm_100a kernels ({len(files)} files) into {lib}", file=sys.stderr,
              flush=True)
        threading.Thread(target=heartbeat, daemon=True).start()
    try:
        objs = [obj_dir / (f.stem + ".o") for f in files]
        with ThreadPoolExecutor(max_workers=min(8, len(files))) as pool:
            jobs = [pool.submit(_run, [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(f), "-o", str(o)])
                    for f, o in zip(files, objs)]
            for j in jobs:
                j.result()
        tmp = out_dir / f".{lib.name}.{os.getpid()}.tmp"
        _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *[str(o) for o in objs], "-lcuda", "-ldl"])
        os.replace(tmp, lib)  # atomic: a concurrent builder never sees half a library
        for stale in out_dir.glob("libtokenmill_kernels_*.so"):     # libraries of earlier source states
            if stale != lib:
                stale.unlink(missing_ok=True)   # a process that has one mapped keeps its copy
    finally:
        done.set()
        shutil.rmtree(obj_dir, ignore_errors=True)
    if verbose:
        print(f"[tokenmill_b200] kernels built in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return lib
