"""Compiles this package's CUDA sources for sm_100a into shared libraries.

Two kinds of library: ``core`` (kernels whose sizes are run-time arguments) and
``attn_d<D>`` (the attention kernels, compiled once per head size D with
``-DKRK_HEAD_DIM=D``, so a model compiles only the head size it has). A library
is rebuilt when a source or a flag changes (its name carries a hash of both) and
is otherwise loaded as it is. Libraries live in ``csrc/_build`` inside the
package when that is writable, else under ``$KRK_BUILD_DIR`` or a per-user
folder in the system's temporary directory; no home directory and no network are
needed. While nvcc runs, a line is printed every few seconds.
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

SRC_DIR = Path(__file__).parent

CORE_SOURCES = ["elementwise.cu", "rope_kv.cu", "gemm_simple.cu", "select.cu", "skinny_bf16.cu", "gemm_tcgen05.cu", "lt_gemm.cu"]
CORE_LIBS = ["-lcublasLt"]  # lt_gemm.cu; the process already holds the copy that torch loaded
ATTN_SOURCES = ["attention_simple.cu", "attention_mma.cu", "attention_tcgen05.cu"]
HEADERS = ["common.cuh", "mma.cuh", "tcgen05.cuh", "attention_noalloc.h"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
# extra flags for performance work, e.g. KRK_EXTRA_NVCC_FLAGS="-DKRK_TRACE"; they are part of the library's hash
NVCC_FLAGS += os.environ.get("KRK_EXTRA_NVCC_FLAGS", "").split()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[kernel_rush_kawk_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("KRK_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $KRK_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                     "the CUDA extension cannot be compiled and this library has no other compute path")


def build_dir() -> Path:
    cands = []
    if os.environ.get("KRK_BUILD_DIR"):
        cands.append(Path(os.environ["KRK_BUILD_DIR"]))
    cands.append(SRC_DIR / "_build")
    cands.append(Path(tempfile.gettempdir()) / f"kernel_rush_kawk_b200_build_{os.getuid()}")
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            fd, probe = tempfile.mkstemp(prefix=".probe_", dir=d)  # a name of its own: threads and processes probe at once
            os.close(fd)
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable folder for compiled kernels among {[str(c) for c in cands]}")


def _existing(sources):
    return [s for s in sources if (SRC_DIR / s).is_file()]


def _key(sources, defines) -> str:
    h = hashlib.sha256()
    for name in list(sources) + _existing(HEADERS):
        h.update(name.encode())
        h.update((SRC_DIR / name).read_bytes())
    h.update(" ".join(NVCC_FLAGS + list(defines) + CORE_LIBS).encode())
    return h.hexdigest()[:12]


def library_path(kind: str, head_dim: int | None = None) -> tuple[Path, list, list]:
    if kind == "core":
        sources, defines, stem = _existing(CORE_SOURCES), [], "libkrk_core"
    else:
        sources, defines, stem = _existing(ATTN_SOURCES), [f"-DKRK_HEAD_DIM={int(head_dim)}"], f"libkrk_attn_d{int(head_dim)}"
    return build_dir() / f"{stem}_{_key(sources, defines)}.so", sources, defines


def _compile_one(nvcc: str, src: Path, obj: Path, defines) -> None:
    cmd = [nvcc, *NVCC_FLAGS, *defines, "-I", str(SRC_DIR), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")


def build_library(kind: str, head_dim: int | None = None, verbose: bool = True) -> Path:
    """Return the path of the library, compiling it first if it is not there."""
    target, sources, defines = library_path(kind, head_dim)
    if target.is_file():
        return target
    nvcc = find_nvcc()
    lock_path = target.with_suffix(".lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)  # one builder at a time per library
        try:
            if target.is_file():
                return target
            t0 = time.time()
            if verbose:
                _say(f"compiling {target.name} from {len(sources)} sources for sm_100a (first use; a minute or so)")
            work = Path(tempfile.mkdtemp(prefix="krk_obj_", dir=str(target.parent)))
            stop = threading.Event()

            def ticker():
                while not stop.wait(10.0):
                    _say(f"  still compiling {target.name} ... {time.time() - t0:.0f}s")

            tick = threading.Thread(target=ticker, daemon=True)
            if verbose:
                tick.start()
            try:
                objs = [work / (Path(s).stem + ".o") for s in sources]
                with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
                    list(pool.map(lambda so: _compile_one(nvcc, SRC_DIR / so[0], so[1], defines), zip(sources, objs)))
                tmp = work / target.name
                libs = []
                if kind == "core":  # the library's directory as a run path too, should the process not hold a copy yet
                    lib_dir = Path(nvcc).resolve().parent.parent / "lib64"
                    libs = [f"-L{lib_dir}", *CORE_LIBS, "-Xlinker", f"-rpath={lib_dir}"]
                r = subprocess.run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode",
                                    "arch=compute_100a,code=sm_100a", *libs], capture_output=True, text=True)
                if r.returncode != 0:
                    raise BuildError(f"linking {target.name} failed:\n{r.stdout}\n{r.stderr}")
                os.replace(tmp, target)
            finally:
                stop.set()
                shutil.rmtree(work, ignore_errors=True)
            if verbose:
                _say(f"built {target.name} in {time.time() - t0:.1f}s")
            return target
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
            try:
                os.unlink(lock_path)
            except OSError:
                pass


def build_all(head_dims=(16, 32, 64, 128), verbose: bool = True) -> list[Path]:
    """Compile the core library and the attention library of every given head size."""
    out = [build_library("core", verbose=verbose)]
    for d in head_dims:
        out.append(build_library("attn", d, verbose=verbose))
    return out
