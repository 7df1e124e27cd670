"""Builds the CUDA library of the package for sm_100a, in-tree, with nvcc.

Every ``*.cu`` under ``arle_b200/csrc`` is compiled to an object file (in
parallel) and linked into ``arle_b200/csrc/_build/libarle_b200.so``.  The
launchers are plain ``extern "C"`` functions over raw pointers, so no Python or
torch headers are involved and a full build takes well under a minute.  A hash of
the sources is kept beside the library; the build is repeated only when it
changes.  When the package folder is not writable the build goes to a per-user
folder under the system's temporary directory.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libarle_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[arle_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("CUDACXX"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $CUDACXX, $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                     "the CUDA kernels of arle_b200 cannot be built")


def sources() -> list:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def source_hash() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def build_dir() -> str:
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"arle_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build_if_needed: bool = True) -> str:
    """Path of an up-to-date library; builds it first when it is missing or stale."""
    want = source_hash()
    for d in (os.path.join(CSRC, "_build"), os.path.join(tempfile.gettempdir(), f"arle_b200_build_{os.getuid()}")):
        lib, tag = os.path.join(d, LIB_NAME), os.path.join(d, "source.sha256")
        if os.path.isfile(lib) and os.path.isfile(tag):
            with open(tag) as f:
                if f.read().strip() == want:
                    return lib
    if not build_if_needed:
        raise BuildError("the CUDA library of arle_b200 is not built")
    return build()


def build(verbose: bool = True) -> str:
    nvcc = find_nvcc()
    out_dir = build_dir()
    srcs = sources()
    if not srcs:
        raise BuildError(f"no .cu sources under {CSRC}")
    t0 = time.time()
    if verbose:
        _say(f"building {LIB_NAME} for sm_100a: {len(srcs)} files with {nvcc} into {out_dir}")
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"still compiling ... {time.time() - t0:.0f}s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        hb.start()

    def compile_one(src: str):
        obj = os.path.join(out_dir, src[:-3] + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return src, obj

    objs = []
    try:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            for n, (src, obj) in enumerate(pool.map(compile_one, srcs), 1):
                objs.append(obj)
                if verbose:
                    _say(f"compiled {src} ({n}/{len(srcs)})")
        lib = os.path.join(out_dir, LIB_NAME)
        tmp = lib + f".tmp{os.getpid()}"
        r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs], capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
        with open(os.path.join(out_dir, "source.sha256"), "w") as f:
            f.write(source_hash())
    finally:
        done.set()
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.1f}s")
    return lib
