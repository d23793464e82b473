"""Compiles the CUDA sources under `csrc/` for sm_100a and loads them.

Every `.cu` file is a library of its own with `extern "C"` launchers, built by
plain `nvcc` (no torch headers, so a file compiles in seconds) into
`csrc/_build/<name>-<hash>.so` inside the package and opened with ctypes.  A
library is compiled at its first use, so a program compiles what its model
needs; `build_all()` compiles every library with its default variants.  The
hash covers the source, the shared headers and the flags, so an edited source
never meets a stale binary.  While nvcc runs, a line is printed every few
seconds.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Iterable, Optional, Tuple

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fvisibility=hidden"]

_loaded: Dict[Tuple[str, Tuple[str, ...]], ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise KernelBuildError(
            "nvcc was not found: the CUDA kernels of tokenizer_b200 cannot be built "
            "(there is no fallback path)")
    return found


_build_dir_found = None
_build_dir_lock = threading.Lock()


def _build_dir() -> str:
    """`csrc/_build` inside the package where it can be written, else a folder of this user's
    under the temporary directory.  Decided once per process (threads that compile side by
    side must agree on it)."""
    global _build_dir_found
    with _build_dir_lock:
        if _build_dir_found is None:
            preferred = os.path.join(CSRC, "_build")
            try:
                os.makedirs(preferred, exist_ok=True)
                probe = os.path.join(preferred, f".probe-{os.getpid()}-{threading.get_ident()}")
                with open(probe, "w"):
                    pass
                os.remove(probe)
                _build_dir_found = preferred
            except OSError:
                fallback = os.path.join(tempfile.gettempdir(), f"tokenizer_b200_build_{os.getuid()}")
                os.makedirs(fallback, exist_ok=True)
                _build_dir_found = fallback
        return _build_dir_found


def _digest(source: str, defines: Tuple[str, ...], extra: Tuple[str, ...]) -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cuh", ".h")) or name == source:
            with open(os.path.join(CSRC, name), "rb") as fh:
                h.update(name.encode())
                h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + list(defines) + list(extra)).encode())
    return h.hexdigest()[:16]


def library_path(source: str, defines: Iterable[str] = (), extra: Iterable[str] = ()) -> str:
    defines, extra = tuple(defines), tuple(extra)
    stem = os.path.splitext(source)[0]
    tag = "".join(c if c.isalnum() else "_" for c in "_".join(defines))
    name = f"libtokb200_{stem}{('_' + tag) if tag else ''}-{_digest(source, defines, extra)}.so"
    return os.path.join(_build_dir(), name)


def compile_library(source: str, defines: Iterable[str] = (), extra: Iterable[str] = (),
                    verbose: bool = True) -> str:
    """Compile `csrc/<source>` if its library is not there yet; return the path."""
    defines, extra = tuple(defines), tuple(extra)
    target = library_path(source, defines, extra)
    if os.path.exists(target):
        return target
    cmd = [_nvcc()] + ARCH_FLAGS + BASE_FLAGS + [f"-D{d}" for d in defines] + list(extra) + [
        "-I", CSRC, os.path.join(CSRC, source)]
    tmp = f"{target}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd += ["-o", tmp]
    label = source + (f" [{' '.join(defines)}]" if defines else "")
    if verbose:
        print(f"[tokenizer_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    started = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            if verbose:
                print(f"[tokenizer_b200] ... still compiling {label} "
                      f"({time.time() - started:.0f} s)", file=sys.stderr, flush=True)

    thread = threading.Thread(target=ticker, daemon=True)
    thread.start()
    output, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed on {label}:\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, target)
    if verbose:
        print(f"[tokenizer_b200] built {os.path.basename(target)} in "
              f"{time.time() - started:.1f} s", file=sys.stderr, flush=True)
    return target


def load_library(source: str, defines: Iterable[str] = (), extra: Iterable[str] = ()) -> ctypes.CDLL:
    key = (source, tuple(defines) + ("|",) + tuple(extra))
    with _lock:
        if key not in _loaded:
            _loaded[key] = ctypes.CDLL(compile_library(source, defines, extra))
        return _loaded[key]


def compile_many(jobs, verbose: bool = True) -> None:
    """Compile several (source, defines, extra) jobs side by side."""
    errors = []

    def work(job):
        try:
            compile_library(*job, verbose=verbose)
        except Exception as err:  # collected and re-raised below
            errors.append(err)

    threads = [threading.Thread(target=work, args=(job,)) for job in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
