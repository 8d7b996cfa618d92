"""Builds the CUDA sources of this folder into one shared library for sm_100a.

The library is built in-tree (``csrc/_build/``) with ``nvcc`` alone: no torch headers, every
entry point has a C signature and is called through ``ctypes``.  A build is reused while the
hash of the sources and flags is unchanged; otherwise the sources are compiled again, in
parallel, and a line is printed now and then so that a first call in a fresh checkout does
not look hung.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

CSRC = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libnanovllm_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-diag-suppress", "177",
]


class BuildError(RuntimeError):
    pass


def _sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the CUDA "
                     "extension cannot be built, and this engine has no other back end")


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in _sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _build_dir() -> str:
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        # a read-only checkout: build beside the temporary files of this user instead
        d = os.path.join(tempfile.gettempdir(), f"nanovllm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library; compiles it first if needed."""
    bdir = _build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "sources.sha256")
    digest = _digest()
    if os.path.exists(lib) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return lib
    if not build:
        raise BuildError(f"{lib} is missing or stale")
    _compile(bdir, lib, verbose)
    with open(stamp, "w") as f:
        f.write(digest)
    return lib


def _say(verbose: bool, msg: str) -> None:
    if verbose:
        print(f"[nano_vllm_cpp_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile(bdir: str, lib: str, verbose: bool) -> None:
    nvcc = _find_nvcc()
    srcs = _sources()
    t0 = time.time()
    _say(verbose, f"compiling {len(srcs)} source files (CUDA for sm_100a, host C++) with {nvcc}")
    procs = []
    objs = []
    for s in srcs:
        obj = os.path.join(bdir, os.path.splitext(s)[0] + ".o")
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, s), "-o", obj]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    pending = dict(procs)
    last = time.time()
    failures = []
    while pending:
        for s, p in list(pending.items()):
            if p.poll() is not None:
                out = p.stdout.read()
                if p.returncode != 0:
                    failures.append((s, out))
                else:
                    _say(verbose, f"  {s} done ({time.time() - t0:.0f} s)")
                del pending[s]
        if pending:
            time.sleep(0.2)
            if time.time() - last > 10:
                _say(verbose, f"  still compiling: {', '.join(sorted(pending))} ({time.time() - t0:.0f} s)")
                last = time.time()
    if failures:
        raise BuildError("nvcc failed:\n" + "\n".join(f"--- {s}\n{o}" for s, o in failures))
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp, *objs]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError("link failed:\n" + r.stdout)
    os.replace(tmp, lib)
    _say(verbose, f"built {lib} in {time.time() - t0:.0f} s")


if __name__ == "__main__":
    print(library_path())
