"""Builds the CUDA kernels of this package into one shared library for sm_100a.

Plain ``nvcc`` on the ``.cu`` files beside this module (no torch headers: the
entry points are ``extern "C"`` and are called through ``ctypes`` with raw device
pointers), objects and library under ``_build/`` beside the sources, or under a
per-user temporary folder when the package folder cannot be written.  The library
is rebuilt when the hash of the sources and flags changes.  Progress goes to
stderr, a line per file and a line every few seconds while waiting.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path
from typing import List, Optional

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libbspec_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]


def bounds_requested() -> bool:
    """``BSPEC_BOUNDS=1`` in the environment: the checked build (``-DBSPEC_BOUNDS``: indices that come from data are
    compared with their ranges, recorded and skipped when outside), kept in a build folder of its own."""
    return os.environ.get("BSPEC_BOUNDS", "0") == "1"


def _flags() -> List[str]:
    return NVCC_FLAGS + (["-DBSPEC_BOUNDS"] if bounds_requested() else [])


def _log(msg: str) -> None:
    print(f"[batchspec_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("BSPEC_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError("nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels cannot be built")


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def _source_hash() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + _flags()).encode())
    return h.hexdigest()


def _build_dir() -> Path:
    override = os.environ.get("BSPEC_BUILD_DIR")
    if override:
        d = Path(override)
        d.mkdir(parents=True, exist_ok=True)
        return d
    d = CSRC / ("_build_checked" if bounds_requested() else "_build")
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"batchspec_b200_build_{os.getuid()}{'_checked' if bounds_requested() else ''}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def library_path(build: bool = True) -> Path:
    """Path of an up-to-date library, building it first if need be."""
    bdir = _build_dir()
    lib, stamp = bdir / LIB_NAME, bdir / (LIB_NAME + ".hash")
    want = _source_hash()
    if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == want:
        return lib
    if not build:
        raise FileNotFoundError(f"{lib} is missing or stale")
    _compile(bdir, lib)
    stamp.write_text(want + "\n")
    return lib


def _compile(bdir: Path, lib: Path) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    _log(f"compiling {len(srcs)} CUDA files for sm_100a with {nvcc} into {bdir}")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", str(bdir))
    procs = []
    for src in srcs:
        obj = bdir / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *_flags(), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)))
    pending = list(procs)
    last = time.time()
    while pending:
        for item in list(pending):
            src, obj, p = item
            if p.poll() is not None:
                out = p.stdout.read().decode(errors="replace")
                if p.returncode != 0:
                    for _, _, q in pending:
                        if q.poll() is None:
                            q.kill()
                    raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
                _log(f"compiled {src.name} ({time.time() - t0:.0f}s)")
                pending.remove(item)
        if pending:
            time.sleep(0.2)
            if time.time() - last > 10:
                _log(f"still compiling {', '.join(s.name for s, _, _ in pending)} ({time.time() - t0:.0f}s)")
                last = time.time()
    tmp = lib.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *[str(o) for _, o, _ in procs]]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout.decode(errors='replace')}")
    os.replace(tmp, lib)
    _log(f"built {lib.name} in {time.time() - t0:.0f}s")


if __name__ == "__main__":
    print(library_path())
