"""Builds the CUDA sources of this folder into one shared library for sm_100a.

`library_path()` returns the path of an up-to-date library, compiling first
when the sources or flags changed (a stamp file beside the library holds
their hash).  The library is built inside the package, in `csrc/_build/`; if
that folder cannot be written it goes to a per-user folder under the system's
temporary directory.  Nothing is read from or written to the home directory.
While it compiles it prints a line per file and a line every few seconds to
stderr, so that a first call does not look hung.

Upstream builds one executable with CMake for sm_120a (CMakeLists.txt:12-35).
"""
from __future__ import annotations

import fcntl
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

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libgarlic_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
                           "--expt-relaxed-constexpr", "-Xcompiler", "-fvisibility=default"]


class BuildError(RuntimeError):
    pass


def timeline_build() -> bool:
    """GARLIC_B200_TIMELINE=1: a build of its own (folder `_build_timeline`) whose kernels note when they start
    and when they are released (common.cuh); `python -m garlic_inference_b200.engine.timeline` reads it."""
    return os.environ.get("GARLIC_B200_TIMELINE", "0") == "1"


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, $CUDA_HOME/bin, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of this library have to be compiled before anything can run")


def _fingerprint() -> str:
    h = hashlib.sha256()
    for p in sources() + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(b"timeline" if timeline_build() else b"")
    return h.hexdigest()


def _build_dir() -> Path:
    override = os.environ.get("GARLIC_B200_BUILD_DIR")
    if override:
        d = Path(override)
        d.mkdir(parents=True, exist_ok=True)
        return d
    d = CSRC / ("_build_timeline" if timeline_build() else "_build")
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"garlic_b200_build_{os.getuid()}{'_timeline' if timeline_build() else ''}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[garlic_inference_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: Path, obj: Path, extra: list[str]) -> None:
    tl = ["-DGI_TIMELINE", f"-DGI_TU={src.stem}"] if timeline_build() else []
    cmd = [nvcc, *NVCC_FLAGS, *tl, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    t0 = time.time()
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    _say(f"compiled {src.name} in {time.time() - t0:.0f} s")
    if extra and r.stderr.strip():
        print(r.stderr, file=sys.stderr)


def build(force: bool = False, verbose_ptxas: bool = False) -> Path:
    """Compile what is stale and return the library's path."""
    bdir = _build_dir()
    lib = bdir / LIB_NAME
    stamp = bdir / (LIB_NAME + ".stamp")
    want = _fingerprint()
    if not force and lib.is_file() and stamp.is_file() and stamp.read_text().strip() == want:
        return lib
    with open(bdir / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and lib.is_file() and stamp.is_file() and stamp.read_text().strip() == want:
            return lib
        nvcc = find_nvcc()
        srcs = sources()
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} (first call only)")
        done = threading.Event()

        def heartbeat():
            t0 = time.time()
            while not done.wait(10.0):
                _say(f"still compiling ... {time.time() - t0:.0f} s")

        hb = threading.Thread(target=heartbeat, daemon=True)
        hb.start()
        try:
            extra = ["-Xptxas", "-v"] if verbose_ptxas else []
            objs = [bdir / (s.stem + ".o") for s in srcs]
            with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
                list(pool.map(lambda so: _compile_one(nvcc, so[0], so[1], extra), zip(srcs, objs)))
            tmp = bdir / (LIB_NAME + f".tmp{os.getpid()}")
            cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs), "-lcuda"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise BuildError(f"link failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
            os.replace(tmp, lib)
            stamp.write_text(want)
        finally:
            done.set()
        _say(f"built {lib}")
    return lib


def library_path() -> Path:
    return build()


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose_ptxas="--ptxas" in sys.argv))
