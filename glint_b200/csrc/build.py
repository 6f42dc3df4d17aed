"""Builds the CUDA kernels for sm_100a with nvcc, and the host-side C++ with the C++ compiler, and
loads them through ctypes.

Sources are grouped into libraries so that a process compiles only what its model and
dtype need: ``core`` (plain kernels and the step runtime, both dtypes), ``tensor`` (tcgen05/TMA
kernels, bfloat16 only) and ``host`` (the cache manager's bookkeeping: no CUDA, so it builds and
runs where there is no GPU and no nvcc).  A library is rebuilt when the hash of its sources and flags changes.  It is
built inside the package (``csrc/_build``) when that folder can be written, else under the
system's temporary folder; nothing depends on HOME.  While nvcc runs, a line is printed to
stderr every few seconds.
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

from ..errors import KernelError

CSRC = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
# extra flags for a debugging build (for instance -DGLINT_WAIT_LIMIT_LOG2=16); they are part of the hash
NVCC_FLAGS += os.environ.get("GLINT_NVCC_EXTRA", "").split()

LIBRARIES = {
    "core": ["elementwise.cu", "gemm_plain.cu", "attention_plain.cu", "sampling.cu", "sample_noalloc.cu", "runtime.cu"],
    "tensor": ["gemm_tcgen05.cu", "gemm_skinny.cu", "attention_decode.cu", "attention_prefill.cu", "attention_tcgen05.cu"],
    "host": ["host/cache_core.cpp"],
}
HEADERS = ["common.cuh", "tcgen05.cuh", "noalloc.h", "runtime.h"]
HOST_LIBRARIES = {"host"}                 # plain C++: compiled without nvcc
HOST_HEADERS = ["host/cache_core.h"]
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall"]

_loaded = {}
_lock = threading.Lock()


def _say(msg):
    print(f"[glint_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc():
    for cand in (os.environ.get("GLINT_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelError("nvcc not found (looked at $GLINT_NVCC, PATH and /usr/local/cuda/bin): "
                      "the CUDA kernels cannot be built and there is no fallback")


def find_cxx():
    for cand in (os.environ.get("GLINT_CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelError("no C++ compiler found (looked at $GLINT_CXX, g++, c++, clang++): the host-side library "
                      "cannot be built")


def _sources(name):
    return [os.path.join(CSRC, s) for s in LIBRARIES[name] if os.path.isfile(os.path.join(CSRC, s))]


def _digest(name):
    h = hashlib.sha256()
    host = name in HOST_LIBRARIES
    h.update(" ".join(HOST_FLAGS if host else NVCC_FLAGS).encode())
    for path in _sources(name) + [os.path.join(CSRC, x) for x in (HOST_HEADERS if host else HEADERS)]:
        if os.path.isfile(path):
            h.update(os.path.basename(path).encode())
            with open(path, "rb") as f:
                h.update(f.read())
    return h.hexdigest()[:16]


def _build_dirs():
    dirs = [os.path.join(CSRC, "_build")]
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(os.path.join(tempfile.gettempdir(), f"glint_b200_build_{uid}"))
    return dirs


def _writable_dir():
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe_{os.getpid()}")
            with open(probe, "w") as f:
                f.write("x")
            os.remove(probe)
            return d
        except OSError:
            continue
    raise KernelError(f"no writable folder to build the CUDA kernels in (tried {', '.join(_build_dirs())})")


def library_path(name):
    """Path of an up-to-date built library, or ``None``."""
    tag = _digest(name)
    for d in _build_dirs():
        p = os.path.join(d, f"libglint_{name}_{tag}.so")
        if os.path.isfile(p):
            return p
    return None


def _run_with_heartbeat(cmds, what):
    """Run the commands in parallel, printing a line every few seconds until all are done."""
    compiler = os.path.basename(cmds[0][0]) if cmds else "compiler"
    t0 = time.time()
    procs = [(c, subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)) for c in cmds]
    outputs = [None] * len(procs)
    done = [False] * len(procs)

    def wait(i):
        outputs[i] = procs[i][1].communicate()[0]
        done[i] = True

    threads = [threading.Thread(target=wait, args=(i,), daemon=True) for i in range(len(procs))]
    for t in threads:
        t.start()
    last = t0
    while not all(done):
        time.sleep(0.2)
        if time.time() - last >= 5.0:
            last = time.time()
            _say(f"still compiling {what} ({sum(done)}/{len(done)} files done, {last - t0:.0f} s)")
    for t in threads:
        t.join()
    for (cmd, p), out in zip(procs, outputs):
        if p.returncode != 0:
            raise KernelError(f"{compiler} failed ({p.returncode}): {' '.join(cmd)}\n{out}")


def build_library(name, verbose=True):
    """Compile library ``name`` if no up-to-date build exists; return its path."""
    if name not in LIBRARIES:
        raise KernelError(f"unknown kernel library '{name}'")
    with _lock:
        path = library_path(name)
        if path:
            return path
        srcs = _sources(name)
        if not srcs:
            raise KernelError(f"kernel library '{name}' has no sources in {CSRC}")
        host = name in HOST_LIBRARIES
        nvcc = None if host else find_nvcc()
        out_dir = _writable_dir()
        tag = _digest(name)
        final = os.path.join(out_dir, f"libglint_{name}_{tag}.so")
        work = tempfile.mkdtemp(prefix=f"{name}_{tag}_", dir=out_dir)
        try:
            t0 = time.time()
            tmp_so = os.path.join(work, "lib.so")
            if host:
                if verbose:
                    _say(f"compiling host library '{name}' ({len(srcs)} files) into {out_dir}")
                _run_with_heartbeat([[find_cxx()] + HOST_FLAGS + ["-I", CSRC, "-shared", "-o", tmp_so] + srcs],
                                    f"'{name}'")
            else:
                if verbose:
                    _say(f"compiling kernel library '{name}' for sm_100a ({len(srcs)} files) into {out_dir}")
                objs, cmds = [], []
                for s in srcs:
                    o = os.path.join(work, os.path.basename(s) + ".o")
                    objs.append(o)
                    cmds.append([nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", s, "-o", o])
                _run_with_heartbeat(cmds, f"'{name}'")
                _run_with_heartbeat([[nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp_so] + objs],
                                    f"'{name}' (link)")
            os.replace(tmp_so, final)  # atomic: concurrent builders never see a partial file
            for old in os.listdir(out_dir):  # drop builds of earlier source versions
                if old.startswith(f"libglint_{name}_") and old.endswith(".so") and old != os.path.basename(final):
                    try:
                        os.remove(os.path.join(out_dir, old))
                    except OSError:
                        pass
            if verbose:
                _say(f"built {os.path.basename(final)} in {time.time() - t0:.1f} s")
        finally:
            shutil.rmtree(work, ignore_errors=True)
        return final


def load_library(name):
    """Build if needed, then ``ctypes.CDLL`` the library (once per process)."""
    lib = _loaded.get(name)
    if lib is None:
        path = build_library(name)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from None
        _loaded[name] = lib
    return lib


def build_all(verbose=True):
    return {name: build_library(name, verbose) for name in LIBRARIES if _sources(name)}


if __name__ == "__main__":
    for k, v in build_all().items():
        print(k, v)
