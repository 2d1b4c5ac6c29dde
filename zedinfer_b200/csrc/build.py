"""Compile the CUDA sources of this folder for sm_100a and load them with ctypes.

Each ``<name>.cu`` becomes ``_build/lib<name>.so``, built with ``nvcc`` on first use and
rebuilt when the source, a header or the flags change (a hash is kept beside the
library).  Only what is asked for is compiled, so a run builds what its model needs.
While nvcc runs a line is printed to stderr every few seconds.  The libraries are plain
C: every entry point takes raw device pointers and a stream, returns 0 or an error code,
and ``zi_last_error_<name>()`` gives the message.

There is no fallback: if nvcc is missing or a build fails the import of the op raises.
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
from typing import Dict, List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]
NVCC_FLAGS += os.environ.get("ZEDINFER_NVCC_FLAGS", "").split()      # experiments, e.g. -DZI_PDL_TRIGGER=0
# No --use_fast_math: division, sqrt, expf and sincosf keep their IEEE / full-range versions.

# Libraries of the engine: name -> source file.  Extra nvcc arguments per library.
SOURCES: Dict[str, str] = {
    "elementwise": "elementwise.cu",
    "gemm_simt": "gemm_simt.cu",
    "attention_generic": "attention_generic.cu",
    "sampling": "sampling.cu",
    "attention_mma": "attention_mma.cu",
    "gemm_smallm": "gemm_smallm.cu",
    "gemm_tcgen05": "gemm_tcgen05.cu",
    "attention_tcgen05": "attention_tcgen05.cu",
}
EXTRA_FLAGS: Dict[str, List[str]] = {}
EXTRA_LIBS: Dict[str, List[str]] = {}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def register_source(name: str, filename: str, extra_flags: Optional[List[str]] = None,
                    extra_libs: Optional[List[str]] = None) -> None:
    SOURCES[name] = filename
    if extra_flags:
        EXTRA_FLAGS[name] = list(extra_flags)
    if extra_libs:
        EXTRA_LIBS[name] = list(extra_libs)


def find_nvcc() -> str:
    for cand in (os.environ.get("ZEDINFER_NVCC"),
                 shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $ZEDINFER_NVCC, PATH, $CUDA_HOME/bin and /usr/local/cuda/bin); "
                     "the engine has no path without its CUDA kernels")


def build_dir() -> str:
    """``_build`` beside the sources when that is writable, else a per-user folder under the temp dir."""
    override = os.environ.get("ZEDINFER_BUILD_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(_HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"zedinfer_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe_{os.getpid()}_{threading.get_ident()}")
            with open(probe, "w") as f:
                f.write("x")
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError("no writable folder for compiled kernels: tried " + ", ".join(str(c) for c in cands))


def _source_hash(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + EXTRA_FLAGS.get(name, []) + EXTRA_LIBS.get(name, [])).encode())
    files = [SOURCES[name]] + sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))
    for fn in files:
        with open(os.path.join(_HERE, fn), "rb") as f:
            h.update(fn.encode())
            h.update(f.read())
    return h.hexdigest()


def _existing_library(name: str, digest: str) -> Optional[str]:
    """A library whose recorded hash matches: in the in-tree folder first, then the fallback."""
    for d in (os.path.join(_HERE, "_build"),
              os.environ.get("ZEDINFER_BUILD_DIR") or "",
              os.path.join(tempfile.gettempdir(), f"zedinfer_b200_build_{os.getuid()}")):
        if not d:
            continue
        so = os.path.join(d, f"lib{name}.so")
        tag = so + ".sha256"
        try:
            with open(tag, "r") as f:
                if f.read().strip() == digest and os.path.isfile(so):
                    return so
        except OSError:
            continue
    return None


def compile_library(name: str, verbose: bool = True) -> str:
    """Build ``lib<name>.so`` if it is not up to date; return its path."""
    if name not in SOURCES:
        raise BuildError(f"unknown kernel library '{name}' (known: {', '.join(sorted(SOURCES))})")
    digest = _source_hash(name)
    have = _existing_library(name, digest)
    if have:
        return have
    nvcc = find_nvcc()
    out_dir = build_dir()
    so = os.path.join(out_dir, f"lib{name}.so")
    tmp = os.path.join(out_dir, f".lib{name}.{os.getpid()}.{threading.get_ident()}.so")
    cmd = [nvcc] + NVCC_FLAGS + EXTRA_FLAGS.get(name, []) + \
          ["-I", _HERE, "-o", tmp, os.path.join(_HERE, SOURCES[name])] + EXTRA_LIBS.get(name, [])
    if verbose:
        print(f"[zedinfer_b200] compiling {SOURCES[name]} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, cwd=out_dir)
    done = threading.Event()

    def _tick():
        while not done.wait(10.0):
            if verbose:
                print(f"[zedinfer_b200] ... still compiling {SOURCES[name]} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)

    ticker = threading.Thread(target=_tick, daemon=True)
    ticker.start()
    try:
        output, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed for {SOURCES[name]} (exit {proc.returncode}):\n"
                         f"{' '.join(cmd)}\n{output.decode(errors='replace')}")
    os.replace(tmp, so)
    with open(so + ".sha256", "w") as f:
        f.write(digest)
    if verbose:
        print(f"[zedinfer_b200] built lib{name}.so in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return so


def compile_all(names: Optional[List[str]] = None, verbose: bool = True, jobs: int = 4) -> Dict[str, str]:
    """Build several libraries at once (used by ``__graft_entry__.build`` and before a run)."""
    from concurrent.futures import ThreadPoolExecutor
    names = list(names) if names is not None else sorted(SOURCES)
    with ThreadPoolExecutor(max_workers=max(1, jobs)) as pool:
        paths = list(pool.map(lambda n: compile_library(n, verbose), names))
    return dict(zip(names, paths))


def load_library(name: str) -> ctypes.CDLL:
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from e
            err = getattr(lib, f"zi_last_error_{name}", None)
            if err is not None:
                err.restype = ctypes.c_char_p
            _loaded[name] = lib
        return lib


def last_error(name: str) -> str:
    lib = _loaded.get(name)
    if lib is None:
        return ""
    fn = getattr(lib, f"zi_last_error_{name}", None)
    return fn().decode(errors="replace") if fn is not None else ""
