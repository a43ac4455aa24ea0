"""Compiles the CUDA sources of this folder for sm_100a into one shared
library and finds it again.  Plain nvcc, no torch headers: a file compiles in
seconds.  The library lies in `<this folder>/build/` (or, if that cannot be
written, in $ULLM_B200_BUILD_DIR or a per-user temporary folder) next to a
stamp of the sources' hash; it is rebuilt when a source or a flag changes.
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

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libullm_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def sources() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH): the CUDA kernels cannot be compiled")


def _writable_dir() -> str:
    cands = [os.environ.get("ULLM_B200_BUILD_DIR"), os.path.join(HERE, "build")]
    try:
        uid = os.getuid()
    except AttributeError:
        uid = 0
    cands.append(os.path.join(tempfile.gettempdir(), f"ullm_b200_build_{uid}"))
    for d in cands:
        if not d:
            continue
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise RuntimeError("no writable folder for the compiled kernels (set ULLM_B200_BUILD_DIR)")


def find_built() -> str | None:
    want = source_hash()
    cands = [os.environ.get("ULLM_B200_BUILD_DIR"), os.path.join(HERE, "build")]
    try:
        cands.append(os.path.join(tempfile.gettempdir(), f"ullm_b200_build_{os.getuid()}"))
    except AttributeError:
        pass
    for d in cands:
        if not d:
            continue
        lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "stamp")
        if os.path.isfile(lib) and os.path.isfile(stamp):
            with open(stamp) as f:
                if f.read().strip() == want:
                    return lib
    return None


def build(verbose: bool = True, force: bool = False) -> str:
    """Returns the path of an up-to-date library, compiling if needed.  Prints
    a line per file and a heartbeat every few seconds while nvcc runs."""
    if not force:
        lib = find_built()
        if lib:
            return lib
    out_dir = _writable_dir()
    nvcc = _nvcc()
    srcs = sources()
    log = (lambda m: print(f"[ullm_b200 build] {m}", file=sys.stderr, flush=True)) if verbose else (lambda m: None)
    log(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir}")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(8.0):
            log(f"... still compiling ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()

    def compile_one(src: str) -> str:
        obj = os.path.join(out_dir, src[:-3] + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        log(f"compiled {src} ({time.time() - t0:.0f} s)")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as ex:
            objs = list(ex.map(compile_one, srcs))
        lib_tmp = os.path.join(out_dir, f".{LIB_NAME}.{os.getpid()}")
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", lib_tmp, *objs, "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
        lib = os.path.join(out_dir, LIB_NAME)
        os.replace(lib_tmp, lib)
        with open(os.path.join(out_dir, "stamp"), "w") as f:
            f.write(source_hash())
    finally:
        done.set()
    log(f"built {lib} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
