"""Builds the CUDA sources of this folder into one shared library for sm_100a.

The library is compiled with nvcc at the first call that needs it (and again whenever a
source changes), into `_build/` beside the sources, or into a per-user temporary folder when
that place cannot be written.  nvcc cross-compiles without a GPU, so this also runs on a
machine that has none.  The reference compiles its kernels at run time too, through NVRTC
with a PTX cache (crates/kf-backend-cuda/src/registry.rs:154-195).
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libkungfu_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
if os.environ.get("KUNGFU_TUNING") == "1":          # a tuning build also exports the planners' measurement hooks
    NVCC_FLAGS.append("-DKF_TUNING")


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[kungfu_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("KUNGFU_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found (looked at $KUNGFU_NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                     "the CUDA kernels of kungfu_b200 cannot be built")


def sources() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers_hash() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(HERE)):
        if f.endswith((".cuh", ".h")):
            with open(os.path.join(HERE, f), "rb") as fh:
                h.update(f.encode() + b"\0" + fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _file_hash(path: str, salt: str) -> str:
    with open(path, "rb") as fh:
        return hashlib.sha256(salt.encode() + fh.read()).hexdigest()[:24]


def build_dir() -> str:
    """`_build/` beside the sources if it can be written, else a per-user temporary folder."""
    override = os.environ.get("KUNGFU_BUILD_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(HERE, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"kungfu_b200_build_{os.getuid()}"))
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


def build(verbose: bool = False, jobs: int | None = None) -> str:
    """Compile what is out of date and return the path of the shared library."""
    out = build_dir()
    lib = os.path.join(out, LIB_NAME)
    salt = _headers_hash()
    srcs = sources()
    wanted = {s: os.path.join(out, f"{s[:-3]}.{_file_hash(os.path.join(HERE, s), salt)}.o") for s in srcs}
    stamp = hashlib.sha256("\n".join(sorted(wanted.values())).encode()).hexdigest()
    stamp_path = os.path.join(out, "stamp")

    def fresh() -> bool:
        try:
            with open(stamp_path) as fh:
                return fh.read().strip() == stamp and os.path.exists(lib)
        except OSError:
            return False

    if fresh():
        return lib
    lock_path = os.path.join(out, ".lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():
                return lib
            nvcc = find_nvcc()
            todo = [s for s in srcs if not os.path.exists(wanted[s])]
            t0 = time.time()
            if todo:
                _say(f"compiling {len(todo)} CUDA source(s) for sm_100a with {nvcc} into {out}")

            def compile_one(s: str) -> str:
                t = time.time()
                tmp = wanted[s] + f".tmp{os.getpid()}"
                cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, s), "-o", tmp]
                if verbose:
                    cmd.insert(1, "-Xptxas=-v")
                r = subprocess.run(cmd, capture_output=True, text=True)
                if r.returncode != 0:
                    raise BuildError(f"nvcc failed on {s}:\n{r.stdout}\n{r.stderr}")
                os.replace(tmp, wanted[s])
                _say(f"  {s} done in {time.time() - t:.1f}s")
                if verbose and r.stderr:
                    print(r.stderr, file=sys.stderr)
                return s

            with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 2)) as pool:
                list(pool.map(compile_one, todo))
            tmp_lib = lib + f".tmp{os.getpid()}"
            cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_lib, *[wanted[s] for s in srcs], "-lcudart"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp_lib, lib)
            keep = set(wanted.values())
            for f in os.listdir(out):                      # objects of older sources
                p = os.path.join(out, f)
                if f.endswith(".o") and p not in keep:
                    os.remove(p)
            with open(stamp_path, "w") as fh:
                fh.write(stamp)
            _say(f"built {lib} in {time.time() - t0:.1f}s")
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


HOST_LIB_NAME = "libkungfu_b200_host.so"


def build_host() -> str:
    """Compile the host-side runtime (host_runtime.cpp: page pools, block tables, the step's integer block, the scheduler) with the
    C++ compiler; it needs neither nvcc nor a GPU.  Returns the path of the shared library."""
    out = build_dir()
    src = os.path.join(HERE, "host_runtime.cpp")
    tag = _file_hash(src, "host-v4")
    lib = os.path.join(out, HOST_LIB_NAME)
    stamp_path = os.path.join(out, "host_stamp")

    def fresh() -> bool:
        try:
            with open(stamp_path) as fh:
                return fh.read().strip() == tag and os.path.exists(lib)
        except OSError:
            return False

    if fresh():
        return lib
    with open(os.path.join(out, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if fresh():
                return lib
            cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++") or shutil.which("clang++")
            tmp = lib + f".tmp{os.getpid()}"
            if cxx:
                cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-static-libstdc++", "-static-libgcc",
                       src, "-o", tmp]
            else:
                cmd = [find_nvcc(), "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-x", "cu", src, "-o", tmp]
            _say(f"compiling the host runtime with {cmd[0]}")
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise BuildError(f"compiling host_runtime.cpp failed:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp, lib)
            with open(stamp_path, "w") as fh:
                fh.write(tag)
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    print(build_host())
    print(build(verbose="-v" in sys.argv))
