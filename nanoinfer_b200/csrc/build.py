"""Builds the kernel library (``libnanoinfer_b200.so``) from the ``.cu`` files of this folder with nvcc,
for sm_100a, into ``_build/`` beside them (or, when that is not writable, a per-user temp folder), and the
host runtime library (``libnanoinfer_b200_host.so``: the page allocator) from ``host/*.cpp`` with the host
compiler alone.

Nothing but the CUDA toolkit is needed: the sources include no framework header, so a cold build
takes well under a minute. It happens at the first call that needs a kernel, prints a line per
file meanwhile, and is skipped when sources and flags are unchanged.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libnanoinfer_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[nanoinfer_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                     "the engine has no path without its CUDA kernels")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sources() + headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def build_dir() -> str:
    env = os.environ.get("NANOINFER_B200_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"nanoinfer_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _compile_one(nvcc: str, src: str, obj: str) -> float:
    t0 = time.time()
    cmd = [nvcc] + NVCC_FLAGS + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{r.stdout}")
    return time.time() - t0


def build(force: bool = False, verbose: bool = True) -> str:
    """Returns the path of the built library, building it if sources or flags changed."""
    d = build_dir()
    lib = os.path.join(d, LIB_NAME)
    stamp = os.path.join(d, "build.json")
    digest = _digest()
    lock_path = os.path.join(d, ".lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and os.path.isfile(lib) and os.path.isfile(stamp):
                try:
                    with open(stamp) as f:
                        if json.load(f).get("digest") == digest:
                            return lib
                except (OSError, ValueError):
                    pass
            nvcc = find_nvcc()
            srcs = sources()
            if verbose:
                _say(f"building {LIB_NAME} for sm_100a from {len(srcs)} files in {d} ...")
            t0 = time.time()
            objs = [os.path.join(d, s[:-3] + ".o") for s in srcs]
            with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
                futs = {pool.submit(_compile_one, nvcc, s, o): s for s, o in zip(srcs, objs)}
                done = 0
                for fut in concurrent.futures.as_completed(futs):
                    secs = fut.result()
                    done += 1
                    if verbose:
                        _say(f"  compiled {futs[fut]} ({done}/{len(srcs)}, {secs:.0f} s)")
            tmp = lib + f".tmp{os.getpid()}"
            r = subprocess.run([nvcc, "-shared", "-o", tmp] + objs, stdout=subprocess.PIPE,
                               stderr=subprocess.STDOUT, text=True)
            if r.returncode != 0:
                raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}")
            os.replace(tmp, lib)
            with open(stamp, "w") as f:
                json.dump({"digest": digest, "flags": NVCC_FLAGS, "sources": srcs}, f)
            if verbose:
                _say(f"built {lib} in {time.time() - t0:.0f} s")
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


HOST_LIB_NAME = "libnanoinfer_b200_host.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        path = shutil.which(cand) if cand else None
        if path:
            return path
    raise BuildError("no C++ compiler was found (looked at $CXX, g++, c++, clang++); "
                     "the cache manager's page allocator is native code")


def host_sources() -> List[str]:
    d = os.path.join(HERE, "host")
    return sorted(os.path.join("host", f) for f in os.listdir(d) if f.endswith((".cpp", ".h")))


def build_host(force: bool = False, verbose: bool = True) -> str:
    """Returns the path of the host runtime library, building it (a second or two) if its sources changed."""
    d = build_dir()
    lib = os.path.join(d, HOST_LIB_NAME)
    stamp = os.path.join(d, "build_host.json")
    h = hashlib.sha256(" ".join(HOST_FLAGS).encode())
    srcs = host_sources()
    for f in srcs:
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    digest = h.hexdigest()
    with open(os.path.join(d, ".lock_host"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and os.path.isfile(lib) and os.path.isfile(stamp):
                try:
                    with open(stamp) as f:
                        if json.load(f).get("digest") == digest:
                            return lib
                except (OSError, ValueError):
                    pass
            cxx = find_cxx()
            if verbose:
                _say(f"building {HOST_LIB_NAME} in {d} ...")
            tmp = lib + f".tmp{os.getpid()}"
            cpp = [os.path.join(HERE, f) for f in srcs if f.endswith(".cpp")]
            r = subprocess.run([cxx] + HOST_FLAGS + ["-o", tmp] + cpp, stdout=subprocess.PIPE,
                               stderr=subprocess.STDOUT, text=True)
            if r.returncode != 0:
                raise BuildError(f"{cxx} failed on {HOST_LIB_NAME}:\n{r.stdout}")
            os.replace(tmp, lib)
            with open(stamp, "w") as f:
                json.dump({"digest": digest, "flags": HOST_FLAGS, "sources": srcs}, f)
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    print(build_host(force="--force" in sys.argv))
    print(build(force="--force" in sys.argv))
