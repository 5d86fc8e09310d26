"""Builds the CUDA sources of this folder for sm_100a and loads them with ctypes.

Each module is one shared library made by one ``nvcc`` call; a module is compiled the
first time something needs it (and ``build_all`` compiles every one), into ``_build/``
beside the sources when that folder can be written, else into a per-user folder under
the system's temporary folder. A library is rebuilt when its sources, the shared headers
or the flags change. While ``nvcc`` runs, a line is printed to stderr every few seconds.
There is no fallback: a missing compiler or a failed build raises ``KernelError``.
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

from ..errors import KernelError

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
HEADERS = ["common.cuh", "attention_common.cuh", "argmax_static.h"]
MODULES = {
    "rowwise": ["rowwise.cu"],
    "rope_kv": ["rope_kv.cu"],
    "attention_simt": ["attention_simt.cu"],
    "attention_mma": ["attention_mma.cu"],
    "attention_tc": ["attention_tc.cu"],
    "gemm_simt": ["gemm_simt.cu"],
    "sampling": ["sampling.cu", "decode_loop.cu"],
    "gemm_tc": ["gemm_tc.cu"],
    "random_fill": ["random_fill.cu"],
}
NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def find_nvcc() -> str:
    for cand in (os.environ.get("CAMELID_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelError("nvcc was not found (looked at $CAMELID_NVCC, PATH, $CUDA_HOME/bin and /usr/local/cuda/bin); "
                      "the CUDA kernels of camelid_b200 cannot be built and there is no other path")


_build_dir: str | None = None


def build_dir() -> str:
    global _build_dir
    if _build_dir is not None:
        return _build_dir
    in_tree = os.path.join(CSRC_DIR, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        fd, probe = tempfile.mkstemp(prefix=".w", dir=in_tree)
        os.close(fd)
        os.remove(probe)
        _build_dir = in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"camelid_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        _build_dir = d
    return _build_dir


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for fn in HEADERS + MODULES[name]:
        with open(os.path.join(CSRC_DIR, fn), "rb") as f:
            h.update(fn.encode())
            h.update(f.read())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    return os.path.join(build_dir(), f"libcamelid_{name}.so")


def is_current(name: str) -> bool:
    path = library_path(name)
    stamp = path + ".hash"
    if not (os.path.isfile(path) and os.path.isfile(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _digest(name)


def compile_module(name: str, verbose: bool = True) -> str:
    """Compile one module if it is stale; returns the library's path."""
    if name not in MODULES:
        raise KernelError(f"unknown kernel module {name!r}; known: {sorted(MODULES)}")
    path = library_path(name)
    if is_current(name):
        return path
    nvcc = find_nvcc()
    tmp = f"{path}.{os.getpid()}.tmp"
    cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC_DIR, "-o", tmp] + [os.path.join(CSRC_DIR, s) for s in MODULES[name]]
    t0 = time.time()
    if verbose:
        print(f"[camelid_b200] compiling CUDA module '{name}' for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=build_dir())
    while True:
        try:
            out, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[camelid_b200]   still compiling '{name}' ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelError(f"nvcc failed for module '{name}' (exit {proc.returncode}):\n{' '.join(cmd)}\n{out}")
    os.replace(tmp, path)
    with open(path + ".hash", "w") as f:
        f.write(_digest(name))
    if verbose:
        print(f"[camelid_b200] module '{name}' built in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return path


def build_all(verbose: bool = True, jobs: int | None = None) -> list[str]:
    """Compile every module (in parallel); used by the build check and before GPU runs."""
    from concurrent.futures import ThreadPoolExecutor
    names = list(MODULES)
    with ThreadPoolExecutor(max_workers=jobs or min(len(names), os.cpu_count() or 4)) as ex:
        return list(ex.map(lambda n: compile_module(n, verbose), names))


def load(name: str) -> ctypes.CDLL:
    """The module's library, compiled first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_module(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"could not load {path}: {e}") from None
            _loaded[name] = lib
        return lib
