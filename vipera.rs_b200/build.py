"""Compiling the native parts at first use.

Two kinds of native code live under ``csrc/``: the host runtime (C++ with pybind11, no
CUDA) and the CUDA kernels, one shared library per ``.cu`` file, compiled for sm_100a
only and loaded with ctypes through their ``extern "C"`` launchers.  Nothing is built at
install time: a library is compiled the first time it is asked for, into ``_build/``
beside this file (or, where that folder cannot be written, into a per-user folder under
the system's temporary directory), and found again by the hash of its sources and flags.

While compiling, a line is printed to stderr at the start of each file and every few
seconds after, so that a first call that takes a minute does not look hung.
"""
from __future__ import annotations

import ctypes
import hashlib
import importlib.machinery
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional

from .errors import InternalError

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
KERNEL_DIR = os.path.join(CSRC, "kernels")
RUNTIME_DIR = os.path.join(CSRC, "runtime")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--expt-relaxed-constexpr",
    "-shared", "-Xcompiler", "-fPIC",
]
# Further compiler flags from the environment (for instance -D switches of a kernel file);
# they are part of a library's name, so builds with different flags live side by side.
NVCC_FLAGS += os.environ.get("VIPERA_NVCC_FLAGS", "").split()
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}
_runtime_module = None


def _say(message: str) -> None:
    print(f"[vipera build] {message}", file=sys.stderr, flush=True)


_build_dir = None


def build_dir() -> str:
    """Where built libraries go: in-tree when writable, else a per-user temporary folder."""
    global _build_dir
    with _lock:
        if _build_dir is None:
            _build_dir = _find_build_dir()
        return _build_dir


def _find_build_dir() -> str:
    override = os.environ.get("VIPERA_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(_HERE, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"vipera_rs_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".write_probe_{os.getpid()}_{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise InternalError("no writable folder for built libraries: tried " + ", ".join(candidates))


def find_nvcc() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and os.path.exists(os.path.join(root, "bin", "nvcc")):
            return os.path.join(root, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise InternalError("nvcc was not found (looked in CUDA_HOME, /usr/local/cuda and PATH); "
                        "the CUDA kernels cannot be compiled")


def _digest(paths: Iterable[str], flags: Iterable[str]) -> str:
    h = hashlib.sha256()
    for path in sorted(paths):
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as handle:
            h.update(handle.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _run(command: List[str], what: str) -> None:
    """Run a compiler, printing a line now and then while it works."""
    started = time.time()
    _say(f"compiling {what} ...")
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"still compiling {what} ({time.time() - started:.0f} s)")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    output, _ = process.communicate()
    done.set()
    if process.returncode != 0:
        raise InternalError(f"compiling {what} failed:\n{' '.join(command)}\n{output}")
    _say(f"compiled {what} in {time.time() - started:.1f} s")


def _kernel_headers() -> List[str]:
    return sorted(
        os.path.join(KERNEL_DIR, name) for name in os.listdir(KERNEL_DIR) if name.endswith((".cuh", ".h"))
    )


def kernel_library_path(name: str) -> str:
    """Compile ``csrc/kernels/<name>.cu`` if no up-to-date library exists; return its path."""
    source = os.path.join(KERNEL_DIR, name + ".cu")
    if not os.path.exists(source):
        raise InternalError(f"no kernel source {source}")
    digest = _digest([source] + _kernel_headers(), NVCC_FLAGS)
    out_dir = build_dir()
    target = os.path.join(out_dir, f"libvipera_{name}-{digest}.so")
    if os.path.exists(target):
        return target
    temporary = f"{target}.{os.getpid()}.{threading.get_ident()}.tmp"
    _run([find_nvcc(), *NVCC_FLAGS, "-I", KERNEL_DIR, source, "-o", temporary], f"{name}.cu for sm_100a")
    os.replace(temporary, target)
    return target


def load_kernel_library(name: str) -> ctypes.CDLL:
    """The shared library of one kernel family, compiled on first use."""
    with _lock:
        if name in _loaded:
            return _loaded[name]
    path = kernel_library_path(name)
    library = ctypes.CDLL(path)
    with _lock:
        _loaded.setdefault(name, library)
        return _loaded[name]


def build_kernels(names: Iterable[str]) -> None:
    """Compile several kernel families side by side (used when a model is built, so that
    the first step does not wait for one compiler run after another)."""
    names = [n for n in dict.fromkeys(names) if n not in _loaded]
    if not names:
        return
    with ThreadPoolExecutor(max_workers=min(len(names), os.cpu_count() or 1)) as pool:
        list(pool.map(kernel_library_path, names))


def all_kernel_names() -> List[str]:
    return sorted(name[:-3] for name in os.listdir(KERNEL_DIR) if name.endswith(".cu"))


def runtime_module():
    """The pybind11 module with the cache manager, scheduler and host sampler."""
    global _runtime_module
    with _lock:
        if _runtime_module is not None:
            return _runtime_module
    import pybind11

    sources = sorted(
        os.path.join(RUNTIME_DIR, name) for name in os.listdir(RUNTIME_DIR) if name.endswith(".cpp")
    )
    headers = sorted(
        os.path.join(RUNTIME_DIR, name) for name in os.listdir(RUNTIME_DIR) if name.endswith(".hpp")
    )
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    digest = _digest(sources + headers, CXX_FLAGS + [suffix])
    out_dir = os.path.join(build_dir(), f"runtime-{digest}")
    target = os.path.join(out_dir, "_vipera_runtime" + suffix)
    if not os.path.exists(target):
        os.makedirs(out_dir, exist_ok=True)
        compiler = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not compiler:
            raise InternalError("no C++ compiler (g++) was found for the host runtime")
        temporary = f"{target}.{os.getpid()}.tmp"
        command = [
            compiler, *CXX_FLAGS,
            "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", RUNTIME_DIR,
            *sources, "-o", temporary,
        ]
        _run(command, "the host runtime (C++)")
        os.replace(temporary, target)
    loader = importlib.machinery.ExtensionFileLoader("_vipera_runtime", target)
    spec = importlib.util.spec_from_file_location("_vipera_runtime", target, loader=loader)
    module = importlib.util.module_from_spec(spec)
    loader.exec_module(module)
    from . import errors

    module._set_error_types(errors.InfeasibleError, errors.InvalidArgumentError, errors.InternalError)
    with _lock:
        _runtime_module = module
    return module


def _drop_stale(keep: Iterable[str]) -> None:
    """Remove libraries in the build folder that no current source and flags lead to (every change
    of a source file leaves one behind).  A library another process has loaded stays usable: the
    file's name goes, not its contents."""
    keep = {os.path.abspath(path) for path in keep}
    out_dir = build_dir()
    for name in os.listdir(out_dir):
        path = os.path.abspath(os.path.join(out_dir, name))
        try:
            if name.startswith("libvipera_") and name.endswith(".so") and path not in keep:
                os.remove(path)
            elif name.startswith("runtime-") and os.path.isdir(path) and path not in keep:
                shutil.rmtree(path, ignore_errors=True)
        except OSError:
            pass


def build_all() -> None:
    """Compile everything: the host runtime and every kernel family; then clear the build folder
    of what earlier sources left behind."""
    module = runtime_module()
    names = all_kernel_names()
    build_kernels(names)
    _drop_stale([kernel_library_path(name) for name in names] + [os.path.dirname(module.__file__)])
