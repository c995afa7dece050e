"""Builds the engine's native code in the tree, at its first use.

Two kinds of library come out of `csrc/`:
  * the host library (`host/*.cc`, g++): cache manager and scheduler;
  * kernel libraries (`kernels/*.cu`, nvcc for sm_100a only): one for the kernels that take
    every size at run time, and one per specialisation (for instance the tensor-core
    attention of one head size), compiled when a model first needs it.
The output lies in `csrc/_build/`, named by a hash of the sources and flags, so a changed
source is rebuilt and an unchanged one is loaded as it is.  While compiling, a line is
printed to stderr every few seconds.  The reference compiles its one CUDA source at run time
as well, with NVRTC and a disk cache keyed the same way (crates/kernels/src/lib.rs:121-156).
There is no fallback: a missing compiler or a failed build raises `BackendError`."""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor

from ..errors import BackendError

CSRC = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(CSRC, "_build")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
GXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-fvisibility=hidden"]
# MRS_HOST_SANITIZE=1 builds the host library with the address and undefined-behaviour sanitizers (a library of
# its own name beside the ordinary one).  The process that loads it must have the sanitizer's runtime loaded first
# (LD_PRELOAD=$(gcc -print-file-name=libasan.so)); `sanitizer_environment()` gives that environment.  The device-side
# memory checker is a separate tool; this mode is for the cache manager, the scheduler and the batch layout, whose
# tests run without a GPU.
GXX_SANITIZE_FLAGS = ["-O1", "-g", "-std=c++17", "-fPIC", "-Wall", "-fvisibility=hidden", "-fno-omit-frame-pointer",
                      "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _say(text: str) -> None:
    print(f"[mini_rsglang_b200] {text}", file=sys.stderr, flush=True)


def _find(tool: str, extra: tuple[str, ...] = ()) -> str:
    path = shutil.which(tool)
    if path:
        return path
    for candidate in extra:
        if os.path.exists(candidate):
            return candidate
    raise BackendError(f"`{tool}` was not found; the engine's native code cannot be built "
                       f"(searched PATH and {list(extra)})")


def _hash(paths: list[str], flags: list[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _headers(folder: str) -> list[str]:
    return [os.path.join(folder, f) for f in sorted(os.listdir(folder)) if f.endswith((".h", ".cuh", ".hpp"))]


def _run(cmd: list[str], what: str) -> None:
    env = dict(os.environ)
    env.setdefault("TMPDIR", BUILD_DIR)
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if proc.returncode != 0:
        raise BackendError(f"building {what} failed (exit {proc.returncode}):\n$ {' '.join(cmd)}\n"
                           f"{proc.stdout}\n{proc.stderr}")


def _build(name: str, sources: list[str], compiler: list[str], flags: list[str], link_flags: list[str],
           header_dir: str) -> str:
    os.makedirs(BUILD_DIR, exist_ok=True)
    digest = _hash(sources + _headers(header_dir), flags + link_flags)
    target = os.path.join(BUILD_DIR, f"lib{name}_{digest}.so")
    if os.path.exists(target):
        return target
    with open(os.path.join(BUILD_DIR, f".{name}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if os.path.exists(target):           # another process built it meanwhile
            return target
        started = time.time()
        _say(f"compiling {name} ({len(sources)} source file(s)) ...")
        stop = threading.Event()

        def heartbeat():
            while not stop.wait(10.0):
                _say(f"still compiling {name} ({time.time() - started:.0f} s) ...")

        beat = threading.Thread(target=heartbeat, daemon=True)
        beat.start()
        try:
            objects = []
            jobs = []
            for src in sources:
                obj = os.path.join(BUILD_DIR, f"{name}_{digest}_{os.path.basename(src)}.o")
                objects.append(obj)
                jobs.append((compiler + flags + ["-c", src, "-o", obj], os.path.basename(src)))
            with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
                list(pool.map(lambda job: _run(*job), jobs))
            partial = target + f".tmp{os.getpid()}"
            _run(compiler + link_flags + ["-shared", "-o", partial] + objects, name)
            os.replace(partial, target)
            for obj in objects:
                os.remove(obj)
        finally:
            stop.set()
        _say(f"compiled {name} in {time.time() - started:.1f} s")
    return target


def _load(key: str, builder) -> ctypes.CDLL:
    with _lock:
        if key not in _loaded:
            path = builder()
            try:
                _loaded[key] = ctypes.CDLL(path)
            except OSError as e:
                raise BackendError(f"cannot load {path}: {e}") from None
        return _loaded[key]


def host_sanitized() -> bool:
    return os.environ.get("MRS_HOST_SANITIZE", "") not in ("", "0")


def sanitizer_environment(base: dict | None = None) -> dict:
    """The environment of a process that loads the sanitized host library: MRS_HOST_SANITIZE=1 and the sanitizer
    runtimes preloaded (Python itself is not built with them, so leak reports are off)."""
    env = dict(os.environ if base is None else base)
    gcc = _find("gcc")
    runtimes = []
    for name in ("libasan.so", "libubsan.so"):
        path = subprocess.run([gcc, f"-print-file-name={name}"], capture_output=True, text=True).stdout.strip()
        if not os.path.isabs(path) or not os.path.exists(path):
            raise BackendError(f"the sanitizer runtime {name} was not found beside {gcc}")
        runtimes.append(os.path.realpath(path))
    env["MRS_HOST_SANITIZE"] = "1"
    env["LD_PRELOAD"] = ":".join(runtimes + [p for p in env.get("LD_PRELOAD", "").split(":") if p])
    env["ASAN_OPTIONS"] = "detect_leaks=0:abort_on_error=1:" + env.get("ASAN_OPTIONS", "")
    env["UBSAN_OPTIONS"] = "print_stacktrace=1:halt_on_error=1:" + env.get("UBSAN_OPTIONS", "")
    return env


def host_library() -> ctypes.CDLL:
    """Cache manager and scheduler (C++, no CUDA)."""
    folder = os.path.join(CSRC, "host")
    sanitize = host_sanitized()

    def builder():
        sources = [os.path.join(folder, f) for f in sorted(os.listdir(folder)) if f.endswith(".cc")]
        if sanitize:
            return _build("mrs_host_sanitized", sources, [_find("g++")], GXX_SANITIZE_FLAGS, ["-fsanitize=address,undefined"], folder)
        return _build("mrs_host", sources, [_find("g++")], GXX_FLAGS, [], folder)

    return _load("host_sanitized" if sanitize else "host", builder)


GENERIC_KERNEL_SOURCES = ("elementwise.cu", "attention_simt.cu", "gemm_f32.cu", "sampling.cu")


def kernel_library() -> ctypes.CDLL:
    """The kernels that take every size at run time."""
    folder = os.path.join(CSRC, "kernels")

    def builder():
        sources = [os.path.join(folder, f) for f in GENERIC_KERNEL_SOURCES]
        nvcc = _find("nvcc", ("/usr/local/cuda/bin/nvcc",))
        return _build("mrs_kernels", sources, [nvcc], NVCC_FLAGS, [], folder)

    return _load("kernels", builder)


def specialised_kernel_library(source: str, defines: dict[str, int], extra_flags: tuple[str, ...] = ()) -> ctypes.CDLL:
    """One kernel source compiled for fixed sizes, e.g. attention for one head size."""
    folder = os.path.join(CSRC, "kernels")
    tag = "_".join(f"{k.lower()}{v}" for k, v in sorted(defines.items()))
    name = f"mrs_{os.path.splitext(source)[0]}_{tag}" if tag else f"mrs_{os.path.splitext(source)[0]}"

    def builder():
        flags = NVCC_FLAGS + [f"-D{k}={v}" for k, v in sorted(defines.items())] + list(extra_flags)
        nvcc = _find("nvcc", ("/usr/local/cuda/bin/nvcc",))
        link = ["-lcuda"] if "-lcuda" in extra_flags else []
        flags = [f for f in flags if f != "-lcuda"]
        return _build(name, [os.path.join(folder, source)], [nvcc], flags, link, folder)

    return _load(name, builder)


# Head sizes whose attention is compiled ahead of time by the build check; any other multiple of
# 16 up to 256 is compiled when a model first needs it.
PREBUILT_HEAD_DIMS = (16, 32, 48, 64, 128)
SPECIALISED_BUILDS = tuple((lambda d=d: specialised_kernel_library("attention_mma.cu", {"MRS_HEAD_DIM": d}))
                           for d in PREBUILT_HEAD_DIMS) + \
    tuple((lambda d=d: specialised_kernel_library("attention_decode_tma.cu", {"MRS_HEAD_DIM": d})) for d in (64, 128)) + \
    tuple((lambda d=d: specialised_kernel_library("attention_prefill_tc.cu", {"MRS_HEAD_DIM": d})) for d in (64, 128)) + \
    (lambda: specialised_kernel_library("gemm_tc.cu", {}), lambda: specialised_kernel_library("gemm_many_rows.cu", {}))
