"""Builds the engine's native code in-tree, at first use.

Two libraries come out of ``axon_b200/csrc``:

* ``libaxon_cuda.so`` from ``cuda/*.cu``: the sm_100a kernels behind plain
  ``extern "C"`` launchers (loaded with ctypes; no PyTorch headers, so a file
  compiles in seconds);
* ``axon_host`` (a CPython module, pybind11) from ``host/*.cpp``: the page
  allocator, the cache manager, the scheduler and the sampler's host half.

Objects and libraries go to ``axon_b200/_build``; a library is rebuilt when the
hash of its sources and flags changes.  Progress is printed to stderr, a line
per file and a line every few seconds while compilers run, because the first
call of a fresh checkout spends a minute or so here.
"""

from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import threading
import time
from typing import List, Sequence

CSRC = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(os.path.dirname(CSRC), "_build")

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[axon_b200 build] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("AXON_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels cannot be built")


def _sources(sub: str, exts: Sequence[str]) -> List[str]:
    d = os.path.join(CSRC, sub)
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(tuple(exts)))


def _digest(files: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _run(cmd: Sequence[str], what: str) -> None:
    p = subprocess.run(list(cmd), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       env={**os.environ, "TMPDIR": os.environ.get("TMPDIR", "/tmp")})
    if p.returncode != 0:
        raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{p.stdout}")


class _Heartbeat:
    """Prints a line every few seconds while a build step runs."""

    def __init__(self, what: str, every: float = 10.0):
        self.what, self.every = what, every
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._loop, daemon=True)

    def _loop(self) -> None:
        t0 = time.time()
        while not self._stop.wait(self.every):
            _say(f"{self.what}: still compiling ({time.time() - t0:.0f} s)")

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()


def _locked(path: str):
    os.makedirs(BUILD_DIR, exist_ok=True)
    f = open(path, "w")
    fcntl.flock(f, fcntl.LOCK_EX)
    return f


def _build(name: str, out: str, sources: List[str], headers: List[str], compile_one, link) -> str:
    """Compile ``sources`` to objects (in parallel) and link ``out`` unless up to date."""
    stamp = out + ".sha256"
    want = _digest(sources + headers, CUDA_FLAGS + HOST_FLAGS + [sys.version])
    if os.path.exists(out) and os.path.exists(stamp) and open(stamp).read().strip() == want:
        return out
    lock = _locked(os.path.join(BUILD_DIR, name + ".lock"))
    try:
        if os.path.exists(out) and os.path.exists(stamp) and open(stamp).read().strip() == want:
            return out
        t0 = time.time()
        what = "for sm_100a " if any(x.endswith(".cu") for x in sources) else ""
        _say(f"{name}: compiling {len(sources)} source files {what}(first use of this checkout, or its sources changed)")
        objs = []
        with _Heartbeat(name), concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            futs = {}
            for s in sources:
                o = os.path.join(BUILD_DIR, name + "_" + os.path.basename(s) + ".o")
                objs.append(o)
                futs[ex.submit(compile_one, s, o)] = s
            for fu in concurrent.futures.as_completed(futs):
                fu.result()
                _say(f"{name}: compiled {os.path.basename(futs[fu])}")
        tmp = out + f".tmp{os.getpid()}"
        link(objs, tmp)
        os.replace(tmp, out)
        with open(stamp, "w") as f:
            f.write(want)
        _say(f"{name}: built in {time.time() - t0:.0f} s")
        return out
    finally:
        lock.close()


def build_cuda() -> str:
    """Build (if needed) and return the path of ``libaxon_cuda.so``."""
    nvcc = _nvcc()
    out = os.path.join(BUILD_DIR, "libaxon_cuda.so")
    srcs = _sources("cuda", (".cu",))
    hdrs = _sources("cuda", (".cuh", ".h"))

    def compile_one(s: str, o: str) -> None:
        _run([nvcc, *CUDA_FLAGS, "-I", os.path.join(CSRC, "cuda"), "-c", s, "-o", o], f"nvcc {os.path.basename(s)}")

    def link(objs: List[str], dst: str) -> None:
        _run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", dst, *objs],
             "linking libaxon_cuda.so")

    return _build("axon_cuda", out, srcs, hdrs, compile_one, link)


def build_host() -> str:
    """Build (if needed) and return the path of the ``axon_host`` extension module."""
    import pybind11

    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler was found (g++): the host library cannot be built")
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    out = os.path.join(BUILD_DIR, "axon_host" + suffix)
    srcs = _sources("host", (".cpp",))
    hdrs = _sources("host", (".h", ".hpp"))
    incs = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", os.path.join(CSRC, "host")]

    def compile_one(s: str, o: str) -> None:
        _run([cxx, *HOST_FLAGS, *incs, "-c", s, "-o", o], f"{cxx} {os.path.basename(s)}")

    def link(objs: List[str], dst: str) -> None:
        _run([cxx, "-shared", "-o", dst, *objs], "linking axon_host")

    return _build("axon_host", out, srcs, hdrs, compile_one, link)


def build_all() -> None:
    build_host()
    build_cuda()


if __name__ == "__main__":
    build_all()
