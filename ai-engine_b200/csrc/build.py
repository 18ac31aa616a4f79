"""Compiles the CUDA sources and the host runtime on first use.

Each `.cu` file becomes one shared library for sm_100a with `extern "C"`
launchers; the host runtime (cache manager, scheduler) becomes one pybind11
module.  A library is keyed by the hash of its source, the headers beside it
and the flags, so an unchanged file is compiled once.  Libraries are built in
`<package>/_build/` when that folder can be written, else in a per-user folder
under the system's temporary directory (or `AI_ENGINE_B200_BUILD_DIR`).
While a compiler runs, a line is printed every few seconds.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from typing import List, Optional

CSRC = os.path.dirname(os.path.abspath(__file__))
PACKAGE = os.path.dirname(CSRC)

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden"]

CUDA_SOURCES = ["elementwise.cu", "rope_kv.cu", "attention_plain.cu", "gemm_f32.cu",
                "sampling.cu", "attention_fast.cu", "attention_decode_noalloc.cu", "gemm_tc.cu", "attention_prefill_tc.cu"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[ai-engine_b200] {msg}", file=sys.stderr, flush=True)


def build_dir() -> str:
    env = os.environ.get("AI_ENGINE_B200_BUILD_DIR")
    cands = [env] if env else []
    cands.append(os.path.join(PACKAGE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"ai_engine_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def find_nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise BuildError("nvcc not found (set NVCC or put it on PATH): the CUDA kernels cannot be built")


def _hash(paths: List[str], flags: List[str]) -> str:
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _headers(folder: str) -> List[str]:
    return sorted(os.path.join(folder, f) for f in os.listdir(folder)
                  if f.endswith((".cuh", ".hpp", ".h")))


def _run(cmd: List[str], what: str) -> None:
    _say(f"compiling {what} (first use; cached afterwards)")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def tick():
        while not done.wait(10.0):
            _say(f"  still compiling {what} ... {time.time() - t0:.0f} s")

    th = threading.Thread(target=tick, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n{' '.join(cmd)}\n{out}")
    _say(f"  built {what} in {time.time() - t0:.1f} s")


def _build(target: str, cmd_prefix: List[str], sources: List[str], deps: List[str],
           flags: List[str], what: str) -> str:
    if os.path.exists(target):
        return target
    tmp = f"{target}.{os.getpid()}.tmp"
    _run(cmd_prefix + flags + sources + ["-o", tmp], what)
    os.replace(tmp, target)
    stem = os.path.basename(target).rsplit("-", 1)[0] + "-"      # older builds of the same source
    for f in os.listdir(os.path.dirname(target)):
        if f.startswith(stem) and f.endswith(".so") and f != os.path.basename(target):
            try:
                os.remove(os.path.join(os.path.dirname(target), f))
            except OSError:
                pass
    return target


def cuda_library(source: str, extra_flags: Optional[List[str]] = None) -> str:
    """Path of the shared library of csrc/<source>, compiled if need be.  An absolute path names a
    `.cu` file outside the package (a part defined elsewhere brings its own kernel); it may include
    the package's headers."""
    outside = os.path.isabs(source)
    src = source if outside else os.path.join(CSRC, source)
    flags = NVCC_FLAGS + (extra_flags or [])
    deps = [src] + _headers(CSRC) + (_headers(os.path.dirname(src)) if outside else [])
    key = _hash(deps, flags)
    stem = os.path.splitext(os.path.basename(source))[0]
    target = os.path.join(build_dir(), f"lib{stem}-{key}.so")
    if os.path.exists(target):
        return target
    return _build(target, [find_nvcc()], [src], deps, flags + ["-I", CSRC],
                  source if outside else f"csrc/{source}")


def host_module_path() -> str:
    """Path of the pybind11 module of csrc/host/ (cache manager and scheduler)."""
    import pybind11

    folder = os.path.join(CSRC, "host")
    srcs = [os.path.join(folder, "bindings.cpp")]
    deps = srcs + _headers(folder)
    flags = CXX_FLAGS + ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
                         "-I", folder]
    key = _hash(deps, [f for f in flags if not f.startswith('/')] + [sysconfig.get_config_var('SOABI') or sys.version])
    target = os.path.join(build_dir(), f"_aie_host-{key}.so")
    if os.path.exists(target):
        return target
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler found (g++): the host runtime cannot be built")
    return _build(target, [cxx], srcs, deps, flags, "csrc/host (cache manager, scheduler)")


def load_host_module():
    import importlib.util

    path = host_module_path()
    spec = importlib.util.spec_from_file_location("_aie_host", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def build_all() -> List[str]:
    """Compile everything (used by the build check); returns the library paths."""
    out = [host_module_path()]
    for s in CUDA_SOURCES:
        if os.path.exists(os.path.join(CSRC, s)):
            out.append(cuda_library(s))
    return out
