"""Compiles the CUDA sources of this folder for sm_100a into one shared library.

The library is built at first use (and again when a source changes) with nvcc,
one object per ``.cu`` file in parallel, then linked.  It is kept in
``csrc/_build/`` inside the package when that folder can be written, otherwise
in a per-user folder under the system's temporary directory; nothing is read
from or written to the home directory.  The sources use no PyTorch headers:
the Python side passes raw device pointers and the stream through ctypes.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libmini_llm_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# -dlcm=cg: plain global loads go to L2, not through L1.  With programmatic dependent launch a kernel is already
# resident while the kernel before it writes its inputs, and an L1 line left by an earlier kernel on the same SM
# can then still be read just after the dependency wait returns (seen as a stale query row in decode attention).
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xptxas", "-dlcm=cg", "-Xcompiler", "-fPIC", "-Xcompiler",
              "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[mini_llm_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("MINI_LLM_B200_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 os.path.join(os.environ.get("CUDA_PATH", ""), "bin", "nvcc") if os.environ.get("CUDA_PATH") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found: set CUDA_HOME or put nvcc on PATH (the kernels are compiled at first use)")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _digest(paths: List[str], extra: str = "") -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    for p in paths:
        h.update(p.encode())
        with open(os.path.join(CSRC_DIR, p), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def build_dir() -> str:
    override = os.environ.get("MINI_LLM_B200_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    in_tree = os.path.join(CSRC_DIR, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"mini_llm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path() -> str:
    return os.path.join(build_dir(), LIB_NAME)


def _run(cmd: List[str], what: str) -> None:
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    p = subprocess.run(cmd, cwd=CSRC_DIR, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"{what} failed (exit {p.returncode}):\n$ {' '.join(cmd)}\n{p.stdout}")


class _Lock:
    """A file lock so that two processes do not build into the same folder at once."""

    def __init__(self, path):
        self.path = path

    def __enter__(self):
        import fcntl
        self.f = open(self.path, "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *a):
        import fcntl
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def ensure_built(verbose: Optional[bool] = None, force: bool = False) -> str:
    """Return the path of an up-to-date library, compiling what is stale."""
    bdir = build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    srcs = sources()
    hdr_digest = _digest(_headers(), " ".join(ARCH_FLAGS + NVCC_FLAGS))
    with _Lock(os.path.join(bdir, ".lock")):
        objs, todo = [], []
        for s in srcs:
            d = _digest([s], hdr_digest)
            obj = os.path.join(bdir, f"{s[:-3]}.{d}.o")
            objs.append(obj)
            if force or not os.path.isfile(obj):
                todo.append((s, obj))
        stamp = os.path.join(bdir, "lib.stamp")
        lib_digest = hashlib.sha256(" ".join(os.path.basename(o) for o in objs).encode()).hexdigest()[:16]
        have = open(stamp).read().strip() if os.path.isfile(stamp) else ""
        if not todo and os.path.isfile(lib) and have == lib_digest:
            return lib
        nvcc = find_nvcc()
        t0 = time.time()
        _say(f"compiling {len(todo)} of {len(srcs)} CUDA sources for sm_100a with {nvcc} into {bdir} "
             f"(first use only)")
        done = [0]
        stop = threading.Event()

        def ticker():
            while not stop.wait(10.0):
                _say(f"... still compiling: {done[0]}/{len(todo)} done, {time.time() - t0:.0f} s")

        th = threading.Thread(target=ticker, daemon=True)
        th.start()
        try:
            def one(job):
                s, obj = job
                tmp = obj + f".{os.getpid()}.tmp"
                _run([nvcc, "-c", *NVCC_FLAGS, *ARCH_FLAGS, s, "-o", tmp], f"compiling {s}")
                os.replace(tmp, obj)
                done[0] += 1
                _say(f"compiled {s} ({done[0]}/{len(todo)})")

            workers = max(1, min(len(todo), os.cpu_count() or 2, 8))
            with ThreadPoolExecutor(max_workers=workers) as ex:
                list(ex.map(one, todo))
            tmp = lib + f".{os.getpid()}.tmp"
            _run([nvcc, "-shared", *ARCH_FLAGS, "-o", tmp, *objs], "linking")
            os.replace(tmp, lib)
            with open(stamp, "w") as f:
                f.write(lib_digest)
        finally:
            stop.set()
        # drop objects of older source versions
        keep = set(objs)
        for f in os.listdir(bdir):
            p = os.path.join(bdir, f)
            if f.endswith(".o") and p not in keep:
                try:
                    os.remove(p)
                except OSError:
                    pass
        _say(f"built {lib} in {time.time() - t0:.1f} s")
        return lib


if __name__ == "__main__":
    print(ensure_built(force="--force" in sys.argv))
