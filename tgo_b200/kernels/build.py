"""Compile the CUDA sources of `tgo_b200/csrc` for sm_100a and load them.

Each `.cu` file becomes one shared library, built with nvcc the first time one of
its kernels is asked for and kept under `tgo_b200/kernels/_build/` (or, if that
folder cannot be written, under a per-user temporary folder), named by a hash of
the sources and flags so an edit rebuilds it. A model therefore compiles only the
libraries it uses. While nvcc runs, a line is printed to stderr now and then.

There is no fallback: a missing compiler, a failed build or a library that will
not load raises, and the caller stops.
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

CSRC = os.path.normpath(os.path.join(os.path.dirname(__file__), "..", "csrc"))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"] + os.environ.get("TGO_NVCC_DEFS", "").split()

# library name -> (sources, extra link flags)
LIBRARIES = {
    "elementwise": (["elementwise.cu"], []),
    "attention_generic": (["attention_generic.cu"], []),
    "attention_flash": (["attention_flash.cu"], []),
    "attention_tc": (["attention_tc.cu"], []),
    "attention_decode_tma": (["attention_decode_tma.cu"], []),
    "sgemm": (["sgemm.cu"], []),
    "gemm_skinny": (["gemm_skinny.cu"], []),
    "gemm_tc": (["gemm_tc.cu"], []),
    "sampling": (["sampling.cu"], []),
    # host code only (no kernel): the cache books and the packing of a step
    "host_runtime": (["host_runtime.cpp"], []),
}
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden"]

_loaded = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _say(line: str) -> None:
    """One whole line to stderr (several libraries may be compiling side by side)."""
    sys.stderr.write(line + "\n")
    sys.stderr.flush()


def register_library(name: str, sources, link_flags=()) -> None:
    LIBRARIES[name] = (list(sources), list(link_flags))


def find_nvcc() -> str:
    for cand in (os.environ.get("TGO_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $TGO_NVCC, $CUDA_HOME/bin, "
                           "/usr/local/cuda/bin and PATH); the CUDA kernels cannot be built "
                           "and there is no other path")


def find_host_compiler():
    """A C++ compiler for the libraries without kernels, or None (nvcc compiles them then)."""
    for cand in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        path = shutil.which(cand) if cand else None
        if path:
            return path
    return None


_build_dir_found = None


def _build_dir() -> str:
    """Where the libraries go: decided once per process (several threads may be compiling)."""
    global _build_dir_found
    if _build_dir_found is not None:
        return _build_dir_found
    with _dir_lock:
        if _build_dir_found is None:
            here = os.path.join(os.path.dirname(__file__), "_build")
            try:
                os.makedirs(here, exist_ok=True)
                probe = os.path.join(here, f".w{os.getpid()}.{threading.get_ident()}")
                with open(probe, "w"):
                    pass
                os.unlink(probe)
                _build_dir_found = here
            except OSError:
                alt = os.path.join(tempfile.gettempdir(), f"tgo_b200_build_{os.getuid()}")
                os.makedirs(alt, exist_ok=True)
                _build_dir_found = alt
    return _build_dir_found


def _digest(sources, link_flags) -> str:
    h = hashlib.sha256()
    for path in sorted(os.listdir(CSRC)):
        if path.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC, path), "rb") as f:
                h.update(path.encode() + b"\0" + f.read())
    for src in sources:
        with open(os.path.join(CSRC, src), "rb") as f:
            h.update(src.encode() + b"\0" + f.read())
    flags = HOST_FLAGS if all(src.endswith(".cpp") for src in sources) else ARCH_FLAGS + NVCC_FLAGS
    h.update(" ".join(flags + list(link_flags)).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    sources, link_flags = LIBRARIES[name]
    return os.path.join(_build_dir(), f"libtgo_{name}_{_digest(sources, link_flags)}.so")


def compile_library(name: str, verbose: bool = True, ptxas_info: bool = False) -> str:
    """Build the library if its file is not there yet; return its path."""
    if name not in LIBRARIES:
        raise KernelBuildError(f"no kernel library named {name!r}; known: {sorted(LIBRARIES)}")
    sources, link_flags = LIBRARIES[name]
    out = library_path(name)
    if os.path.exists(out) and not ptxas_info:
        return out
    tmp = f"{out}.{os.getpid()}.tmp"
    host_only = all(src.endswith(".cpp") for src in sources)
    cxx = find_host_compiler() if host_only else None
    if cxx:
        cmd = [cxx] + HOST_FLAGS + ["-I", CSRC, "-o", tmp] + \
            [os.path.join(CSRC, s) for s in sources] + list(link_flags)
    else:
        nvcc = find_nvcc()
        cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + \
            ["-I", CSRC, "-o", tmp] + [os.path.join(CSRC, s) for s in sources] + list(link_flags)
    if verbose:
        _say(f"[tgo_b200] compiling {name} ({', '.join(sources)})"
             f"{' for the host' if host_only else ' for sm_100a'} ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    while True:
        try:
            output, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                _say(f"[tgo_b200]   still compiling {name} ({time.time() - t0:.0f} s)")
    text = output.decode(errors="replace")
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise KernelBuildError(f"the compiler failed on {name}:\n{' '.join(cmd)}\n{text}")
    os.replace(tmp, out)
    # older builds of the same library (other source hashes) are of no use any more
    prefix = f"libtgo_{name}_"
    for other in os.listdir(os.path.dirname(out)):
        if other.startswith(prefix) and other.endswith(".so") and \
                os.path.join(os.path.dirname(out), other) != out:
            try:
                os.unlink(os.path.join(os.path.dirname(out), other))
            except OSError:
                pass
    if verbose:
        _say(f"[tgo_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    if ptxas_info:
        print(text)
    return out


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library, compiled first if need be."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"{path} was built and does not load: {e}") from None
            _loaded[name] = lib
    return lib


def compile_together(names, verbose: bool = True) -> None:
    """Build several libraries at once, a compiler process each (a model's first step would
    otherwise build the ones it needs one after the other as it reaches them)."""
    from concurrent.futures import ThreadPoolExecutor
    todo = [n for n in dict.fromkeys(names) if n not in _loaded and not os.path.exists(library_path(n))]
    if len(todo) <= 1:
        for n in todo:
            compile_library(n, verbose=verbose)
        return
    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 2, 8)) as pool:
        for f in [pool.submit(compile_library, n, verbose) for n in todo]:
            f.result()


def build_all(verbose: bool = True) -> None:
    compile_together(sorted(LIBRARIES), verbose=verbose)
    for name in sorted(LIBRARIES):           # whatever was there already is checked to exist
        compile_library(name, verbose=verbose)
