"""Compiles the CUDA sources of this folder for sm_100a and loads them with ctypes.

There is one shared library per group of sources, so that a model compiles
only what it needs at its first call.  A library is rebuilt when the hash of
its sources and flags changes.  It is written next to the sources; where that
folder cannot be written (a read-only install) a per-user folder under the
system's temporary directory is used instead.  Nothing is read from or written
to the home directory.  While nvcc runs, a line is printed every few seconds.
"""

from __future__ import annotations

import ctypes
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

SOURCE_DIR = Path(__file__).resolve().parent

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]

# library name -> sources.  "core" holds the kernels that take every size; the
# others hold the tensor-core kernels for the sizes they are specialised for.
LIBRARIES: dict[str, list[str]] = {
    "core": ["elementwise.cu", "gemm_simt.cu", "attention_simt.cu", "sampling.cu"],
    "tc": ["gemm_tc.cu", "attention_decode_mma.cu", "attention_prefill_tc.cu"],
}

_HEADERS = ["common.cuh", "tc_common.cuh", "no_alloc.h", "rope.cuh", "attention_fold.cuh"]
_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    """nvcc is missing or a source did not compile."""


def _say(msg: str) -> None:
    print(f"[lockstep_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("LOCKSTEP_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError(
        "nvcc was not found (looked at $LOCKSTEP_NVCC, PATH and /usr/local/cuda/bin); "
        "the engine has no CPU fallback and cannot run without its CUDA extension"
    )


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for src in _HEADERS + sorted(set(LIBRARIES[name])):
        path = SOURCE_DIR / src
        if path.exists():
            h.update(src.encode())
            h.update(path.read_bytes())
    return h.hexdigest()[:16]


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe-{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def output_dir() -> Path:
    """Folder that holds the built libraries."""
    if _writable(SOURCE_DIR / "_build"):
        return SOURCE_DIR
    alt = Path(tempfile.gettempdir()) / f"lockstep_b200-{os.getuid()}"
    if not _writable(alt / "_build"):
        raise BuildError(f"neither {SOURCE_DIR} nor {alt} can be written to build the CUDA extension")
    return alt


def library_path(name: str) -> Path:
    return output_dir() / f"liblockstep_{name}.so"


def _run_with_heartbeat(cmd: list[str], what: str) -> None:
    started = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            cwd=str(SOURCE_DIR))
    done = threading.Event()

    def beat():
        while not done.wait(8.0):
            _say(f"still compiling {what} ({time.time() - started:.0f} s)")

    t = threading.Thread(target=beat, daemon=True)
    t.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {what}:\n{' '.join(cmd)}\n{out}")


def build(name: str, force: bool = False) -> Path:
    """Compile library `name` if it is missing or stale; return its path."""
    if name not in LIBRARIES:
        raise KeyError(f"unknown library {name!r}; known: {sorted(LIBRARIES)}")
    out_dir = output_dir()
    target = out_dir / f"liblockstep_{name}.so"
    stamp = out_dir / f"liblockstep_{name}.stamp"
    digest = _digest(name)
    if not force and target.exists() and stamp.exists() and stamp.read_text().strip() == digest:
        return target

    nvcc = find_nvcc()
    obj_dir = out_dir / "_build"
    obj_dir.mkdir(parents=True, exist_ok=True)
    with open(obj_dir / f".{name}.lock", "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        try:
            if not force and target.exists() and stamp.exists() and stamp.read_text().strip() == digest:
                return target
            _say(f"compiling CUDA library '{name}' for sm_100a ({len(LIBRARIES[name])} sources), once")
            started = time.time()
            objects = []

            def compile_one(src: str) -> Path:
                obj = obj_dir / f"{name}-{Path(src).stem}-{digest}.o"
                cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-c", str(SOURCE_DIR / src), "-o", str(obj)]
                _run_with_heartbeat(cmd, src)
                _say(f"compiled {src}")
                return obj

            with ThreadPoolExecutor(max_workers=min(4, len(LIBRARIES[name]))) as pool:
                objects = list(pool.map(compile_one, LIBRARIES[name]))
            tmp = out_dir / f".liblockstep_{name}.{os.getpid()}.so"
            cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objects)]
            _run_with_heartbeat(cmd, f"link {name}")
            os.replace(tmp, target)
            stamp.write_text(digest + "\n")
            for obj in objects:
                try:
                    obj.unlink()
                except OSError:
                    pass
            _say(f"built {target.name} in {time.time() - started:.0f} s")
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)
    return target


def load(name: str) -> ctypes.CDLL:
    """Build if needed and open library `name`."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(str(build(name)))
            _loaded[name] = lib
        return lib


def build_all(force: bool = False) -> list[Path]:
    return [build(name, force=force) for name in LIBRARIES]
