"""Compiles the CUDA sources of this directory into shared libraries, on first use.

Each *module* is a list of ``.cu`` files linked into one ``libleone_<module>.so``
under ``csrc/_build`` (or under the temporary directory if the package
directory cannot be written).  A module is rebuilt when the contents of its
sources or headers, or the compiler flags, change.  Compilation needs only
``nvcc``; the CUDA runtime is linked statically, so the library depends on the driver only.  While nvcc
runs, a line is printed to stderr every few seconds.

The reference compiles its one translation unit at build time for sm_89
(crates/leone-cuda/build.rs:28-45); here the target is sm_100a only.
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
from typing import Dict, List

HERE = os.path.dirname(os.path.abspath(__file__))

MODULES: Dict[str, List[str]] = {
    # every run needs these: both dtypes, every size
    "core": ["elementwise.cu", "gemm_simt.cu", "attention_generic.cu", "sampling_pipeline.cu", "random_weights.cu"],
    # the bfloat16 serving path: tensor-core products and tiled attention
    "bf16": ["gemm_tc.cu", "gemm_pair.cu", "attention_tiled.cu", "attention_prefill_pingpong.cu"],
    # the entry point that allocates nothing (leone_static.h); it compiles attention_tiled.cu in
    "static": ["attention_decode_static.cu"],
    # the host side of the runtime (pages, block tables, step metadata, the scheduler's decisions,
    # seeded random weights for CPU tensors): plain C++, no device code
    "host": ["host_runtime.cpp", "random_weights_host.cpp"],
}
HOST_ONLY = {"host"}
HEADERS = ["common.cuh", "tc_common.cuh", "gemm_parts.cuh", "leone_static.h", "attention_tiled.cu", "random_draw.h"]

# -fno-gnu-unique: statics inside inline functions and templates (the once-per-kernel set-up
# flags, the launch mode switch) must belong to one library image each; with GNU unique
# binding the loader would share them between this package's libraries even though each is
# loaded with local scope.
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fno-gnu-unique", "--expt-relaxed-constexpr"]


# -ffp-contract=off: the seeded random weights must round as the device's do (random_draw.h)
HOST_FLAGS = ["-fPIC", "-ffp-contract=off", "-pthread"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("LEONE_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked in PATH, $CUDA_HOME/bin and /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be compiled")


def build_dir() -> str:
    local = os.path.join(HERE, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"leone_b200_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def _digest(module: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(HOST_FLAGS if module in HOST_ONLY else NVCC_FLAGS).encode())
    for name in MODULES[module] + HEADERS:
        path = os.path.join(HERE, name)
        if os.path.isfile(path):
            h.update(name.encode())
            with open(path, "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def library_path(module: str) -> str:
    return os.path.join(build_dir(), f"libleone_{module}.so")


def _run_with_heartbeat(cmd: List[str], what: str) -> None:
    started = time.time()
    done = threading.Event()

    def beat():
        while not done.wait(8.0):
            print(f"[leone_b200] still compiling {what} ({time.time() - started:.0f} s)",
                  file=sys.stderr, flush=True)

    t = threading.Thread(target=beat, daemon=True)
    t.start()
    try:
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    finally:
        done.set()
    if proc.returncode != 0:
        raise BuildError(f"the compiler failed on {what}:\n{' '.join(cmd)}\n{proc.stdout}")


def ensure_built(module: str, verbose: bool = True) -> str:
    """Return the path of the module's library, compiling it first if it is missing or stale."""
    if module not in MODULES:
        raise BuildError(f"unknown kernel module '{module}'")
    out_dir = build_dir()
    lib = os.path.join(out_dir, f"libleone_{module}.so")
    stamp = lib + ".stamp"
    digest = _digest(module)

    def fresh() -> bool:
        if not (os.path.isfile(lib) and os.path.isfile(stamp)):
            return False
        with open(stamp) as fh:
            return fh.read().strip() == digest

    if fresh():
        return lib
    missing = [s for s in MODULES[module] if not os.path.isfile(os.path.join(HERE, s))]
    if missing:
        raise BuildError(f"kernel module '{module}' lacks sources: {missing}")
    if module in HOST_ONLY:
        return _build_host(module, lib, stamp, digest, fresh, out_dir, verbose)
    nvcc = find_nvcc()
    lock_path = os.path.join(out_dir, f".{module}.lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():
                return lib
            if verbose:
                print(f"[leone_b200] compiling CUDA module '{module}' for sm_100a "
                      f"({len(MODULES[module])} files) into {out_dir}", file=sys.stderr, flush=True)
            t0 = time.time()
            objs = []

            def compile_one(src: str) -> str:
                obj = os.path.join(out_dir, f"{module}_{os.path.splitext(src)[0]}.o")
                _run_with_heartbeat([nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src),
                                     "-o", obj], src)
                return obj

            with ThreadPoolExecutor(max_workers=min(4, len(MODULES[module]))) as pool:
                objs = list(pool.map(compile_one, MODULES[module]))
            tmp_lib = lib + f".tmp{os.getpid()}"
            _run_with_heartbeat([nvcc, "-shared", "-o", tmp_lib, *objs], f"link {module}")
            os.replace(tmp_lib, lib)
            with open(stamp, "w") as fh:
                fh.write(digest)
            for obj in objs:
                try:
                    os.remove(obj)
                except OSError:
                    pass
            if verbose:
                print(f"[leone_b200] module '{module}' built in {time.time() - t0:.0f} s",
                      file=sys.stderr, flush=True)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    return find_nvcc()        # nvcc compiles plain C++ too


def _build_host(module, lib, stamp, digest, fresh, out_dir, verbose) -> str:
    """A module without device code: one call of the C++ compiler."""
    cxx = find_cxx()
    lock_path = os.path.join(out_dir, f".{module}.lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():
                return lib
            if verbose:
                print(f"[leone_b200] compiling C++ module '{module}' into {out_dir}", file=sys.stderr, flush=True)
            t0 = time.time()
            tmp_lib = lib + f".tmp{os.getpid()}"
            srcs = [os.path.join(HERE, s) for s in MODULES[module]]
            flags = ["-O2", "-std=c++17", "-shared", "-Xcompiler", ",".join(HOST_FLAGS)] \
                if os.path.basename(cxx).startswith("nvcc") \
                else ["-O2", "-std=c++17", "-shared", "-fno-gnu-unique", *HOST_FLAGS]
            _run_with_heartbeat([cxx, *flags, "-I", HERE, *srcs, "-o", tmp_lib], MODULES[module][0])
            os.replace(tmp_lib, lib)
            with open(stamp, "w") as fh:
                fh.write(digest)
            if verbose:
                print(f"[leone_b200] module '{module}' built in {time.time() - t0:.0f} s",
                      file=sys.stderr, flush=True)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


def build_all(verbose: bool = True) -> List[str]:
    return [ensure_built(m, verbose) for m in MODULES
            if all(os.path.isfile(os.path.join(HERE, s)) for s in MODULES[m])]
