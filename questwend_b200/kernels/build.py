"""Building and loading the hand-written CUDA libraries.

Each ``csrc/<module>.cu`` becomes one shared library ``_build/qwb_<module>.so``
with a C ABI, compiled for sm_100a by nvcc the first time the module is asked
for, and loaded with ctypes.  A stamp beside the library holds a hash of the
sources and flags; a library whose stamp does not match is rebuilt.  Only the
modules that a model uses are ever compiled.  There is no fallback: a module
that cannot be built or loaded raises ``KernelBuildError``.
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

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC"]
EXTRA_FLAGS: dict[str, list[str]] = {}
NVCC_FLAGS += os.environ.get("QWB200_NVCC_FLAGS", "").split()      # more flags (-D switches) for experiments; part of the stamp
MODULES = ("elementwise", "rope_kv", "attention", "attention_mma", "attention_tc", "gemm_small", "gemm_stream", "gemm_ring", "gemm_tc", "sampling")

_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[questwend_b200] {msg}", file=sys.stderr, flush=True)


def build_dir() -> str:
    """In-tree ``questwend_b200/_build`` when it can be written, else a per-user temporary folder."""
    d = os.path.join(os.path.dirname(_HERE), "_build")
    try:
        os.makedirs(d, exist_ok=True)
        if os.access(d, os.W_OK):
            return d
    except OSError:
        pass
    d = os.path.join(tempfile.gettempdir(), f"questwend_b200_build_{os.getuid()}")
    os.makedirs(d, exist_ok=True)
    return d


def _find_nvcc() -> str | None:
    for cand in (os.environ.get("QWB200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _sources(module: str) -> list[str]:
    src = os.path.join(CSRC, f"{module}.cu")
    if not os.path.exists(src):
        raise KernelBuildError(f"no kernel source for module '{module}' ({src})")
    headers = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    return [src] + headers


def _stamp(module: str) -> str:
    h = hashlib.sha256()
    for path in _sources(module):
        with open(path, "rb") as f:
            h.update(os.path.basename(path).encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + EXTRA_FLAGS.get(module, [])).encode())
    return h.hexdigest()


def library_path(module: str) -> str:
    return os.path.join(build_dir(), f"qwb_{module}.so")


def is_built(module: str) -> bool:
    lib = library_path(module)
    stamp_file = lib + ".stamp"
    if not (os.path.exists(lib) and os.path.exists(stamp_file)):
        return False
    with open(stamp_file) as f:
        return f.read().strip() == _stamp(module)


def compile_module(module: str, verbose: bool = True) -> str:
    """Compile one module if its library is missing or stale; returns the library's path."""
    lib = library_path(module)
    if is_built(module):
        return lib
    nvcc = _find_nvcc()
    if nvcc is None:
        raise KernelBuildError(f"kernel module '{module}' is not built and nvcc was not found "
                               f"(looked on PATH and in /usr/local/cuda/bin)")
    tmp = f"{lib}.{os.getpid()}.tmp"
    cmd = ([nvcc] + NVCC_FLAGS + [f'-DQWB_MODULE_NAME="{module}"', "-I", CSRC, "-o", tmp, os.path.join(CSRC, f"{module}.cu")]
           + EXTRA_FLAGS.get(module, []))
    if verbose:
        _log(f"compiling kernel module '{module}' for sm_100a (first use) ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    out_chunks: list[str] = []
    reader = threading.Thread(target=lambda: out_chunks.append(proc.stdout.read()), daemon=True)
    reader.start()
    last = t0
    while proc.poll() is None:
        time.sleep(0.2)
        if verbose and time.time() - last > 10:
            last = time.time()
            _log(f"  still compiling '{module}' ({int(last - t0)} s)")
    reader.join()
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for kernel module '{module}':\n{''.join(out_chunks)}")
    os.replace(tmp, lib)
    with open(lib + ".stamp", "w") as f:
        f.write(_stamp(module))
    if verbose:
        _log(f"  built {os.path.basename(lib)} in {time.time() - t0:.1f} s")
    return lib


def compile_modules(modules, verbose: bool = True) -> None:
    """Compile several modules side by side."""
    todo = [m for m in modules if not is_built(m)]
    if not todo:
        return
    errors: list[BaseException] = []

    def work(m):
        try:
            compile_module(m, verbose)
        except BaseException as e:      # noqa: BLE001 - reported below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(m,)) for m in todo]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]


def load_module(module: str) -> ctypes.CDLL:
    """The loaded library of a module, compiling it first if needed."""
    with _lock:
        lib = _loaded.get(module)
        if lib is not None:
            return lib
        path = compile_module(module)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelBuildError(f"cannot load kernel library {path}: {e}") from None
        lib.qwb_last_error.restype = ctypes.c_char_p
        _loaded[module] = lib
        return lib
