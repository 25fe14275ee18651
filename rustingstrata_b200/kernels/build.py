"""Compiles the CUDA sources under ``csrc/`` for sm_100a and loads them with ctypes.

The reference compiles its single kernel source at run time with NVRTC for the device
it finds and caches the cubin on disk (src/cuda/mod.rs:386-412, src/cuda/nvrtc.rs:98-127).
Here the sources are grouped into small libraries, each compiled with ``nvcc`` for
sm_100a only when first needed, so a run builds what its model and element type use
and nothing else.  Objects land in ``<package>/_build`` when that folder can be
written (a checkout), else in a per-user folder under the system's temporary
directory; a library is rebuilt when a source, a header or the flags change.  No home
directory and no network are needed.  A progress line is printed to stderr when a
compile starts and every few seconds while it runs.
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
from typing import Dict, List

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_PKG, "csrc")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# library name → sources (relative to csrc/) and extra link flags
LIBRARIES: Dict[str, Dict[str, List[str]]] = {
    "core": {"sources": ["elementwise.cu", "linear_simt.cu", "attention_simt.cu", "sampling.cu"], "link": []},
    # tensor-core paths of the bfloat16 engine; the 32-bit engine never loads this library
    # not loaded by the engine: one kernel whose wait is never satisfied, built with a 2 ms limit, so that a test can
    # see the bounded-wait path end in a status bit and leave the context usable
    "probe": {"sources": ["wait_probe.cu"], "link": [], "flags": ["-DRS_WAIT_LIMIT_NS_VALUE=2000000ull"]},
    "bf16": {"sources": ["gemm_tcgen05.cu", "skinny_gemm_tma.cu", "decode_chain.cu", "mid_gemm_tcgen05.cu", "attention_decode_mma.cu", "attention_prefill_mma.cu", "attention_prefill_tc.cu"], "link": []},
}


class KernelBuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    cands = [os.environ.get("CUDA_HOME", ""), os.environ.get("CUDA_PATH", ""), "/usr/local/cuda"]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "bin", "nvcc")):
            return os.path.join(c, "bin", "nvcc")
    w = shutil.which("nvcc")
    if w:
        return w
    raise KernelBuildError("nvcc not found (looked in $CUDA_HOME, /usr/local/cuda and PATH); the engine has no "
                           "fallback without its CUDA extension")


def build_dir() -> str:
    d = os.path.join(_PKG, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"rustingstrata_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(paths: List[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(os.path.basename(p).encode())     # not the folder: a built library travels with the tree
            h.update(f.read())
    return h.hexdigest()[:16]


def _say(msg: str) -> None:
    print(f"[rustingstrata_b200] {msg}", file=sys.stderr, flush=True)


def _run_with_heartbeat(cmd: List[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def beat():
        while not done.wait(10.0):
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")
    th = threading.Thread(target=beat, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise KernelBuildError(f"compiling {what} failed (exit {proc.returncode}):\n{' '.join(cmd)}\n{out}")


def compile_library(name: str, verbose: bool = True) -> str:
    """Builds ``name`` if it is stale and returns the path of its shared library."""
    if name not in LIBRARIES:
        raise KernelBuildError(f"unknown kernel library '{name}' (known: {', '.join(sorted(LIBRARIES))})")
    spec = LIBRARIES[name]
    srcs = [os.path.join(CSRC, s) for s in spec["sources"]]
    nvcc = find_nvcc()
    bdir = build_dir()
    flags = ARCH_FLAGS + NVCC_FLAGS + spec.get("flags", [])
    tag = _digest(srcs + _headers(), " ".join(flags + spec["link"]))
    lib = os.path.join(bdir, f"librs_{name}_{tag}.so")
    if os.path.isfile(lib):
        return lib
    if verbose:
        _say(f"compiling kernel library '{name}' for sm_100a ({len(srcs)} sources) into {bdir}")
    objs = []
    threads = []
    errors: List[BaseException] = []
    for s in srcs:
        obj = os.path.join(bdir, f"{name}_{os.path.basename(s)}_{tag}.o")
        objs.append(obj)

        def work(s=s, obj=obj):
            try:
                _run_with_heartbeat([nvcc] + flags + ["-I", CSRC, "-c", s, "-o", obj], os.path.basename(s))
            except BaseException as e:  # noqa: BLE001 - re-raised below
                errors.append(e)
        th = threading.Thread(target=work)
        th.start()
        threads.append(th)
    for th in threads:
        th.join()
    if errors:
        raise errors[0]
    tmp = lib + f".tmp{os.getpid()}"
    _run_with_heartbeat([nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp] + objs + ["-lcudart"] + spec["link"],
                        f"link {name}")
    os.replace(tmp, lib)
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    # drop stale builds of the same library
    for f in os.listdir(bdir):
        if f.startswith(f"librs_{name}_") and f.endswith(".so") and os.path.join(bdir, f) != lib:
            try:
                os.remove(os.path.join(bdir, f))
            except OSError:
                pass
    if verbose:
        _say(f"kernel library '{name}' ready")
    return lib


_LOADED: Dict[str, ctypes.CDLL] = {}
_LOCK = threading.Lock()


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library, compiled first if needed.  Fails loudly: there is no other path."""
    with _LOCK:
        lib = _LOADED.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load kernel library {path}: {e}") from None
            _LOADED[name] = lib
        return lib


def build_all(verbose: bool = True) -> List[str]:
    return [compile_library(n, verbose) for n in LIBRARIES]
