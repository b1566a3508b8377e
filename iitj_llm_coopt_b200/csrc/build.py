"""Compiles the CUDA sources of this folder into one shared library for sm_100a.

`library_path()` returns the path of an up-to-date `libllm_kernels.so`, building it first if
the sources changed since the last build (a hash of sources, headers and flags is kept
beside the library).  The build runs `nvcc` once per source file, in parallel, then links;
it needs no GPU.  While it runs it prints a progress line every few seconds to stderr.

The library is built in-tree under `csrc/_build/`; if that folder cannot be written, under
the system's temporary folder.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import glob
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libllm_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr", "-diag-suppress", "177"]
NVCC_FLAGS += os.environ.get("IITJ_NVCC_FLAGS", "").split()      # extra flags, e.g. -D switches for measurements


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and $CUDA_HOME/bin); "
                     "the CUDA kernels of this engine cannot be built")


def sources() -> list:
    return sorted(glob.glob(os.path.join(HERE, "*.cu")))


def _fingerprint() -> str:
    h = hashlib.sha256()
    headers = sorted(glob.glob(os.path.join(HERE, "*.cuh")) + glob.glob(os.path.join(HERE, "*.h")))
    for path in sources() + headers:
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _build_dir() -> str:
    first = os.path.join(HERE, "_build")
    try:
        os.makedirs(first, exist_ok=True)
        probe = os.path.join(first, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return first
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"iitj_llm_coopt_b200-build-{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def _up_to_date(bdir: str, fp: str) -> bool:
    stamp, lib = os.path.join(bdir, "stamp.json"), os.path.join(bdir, LIB_NAME)
    if not (os.path.isfile(stamp) and os.path.isfile(lib)):
        return False
    try:
        with open(stamp) as f:
            return json.load(f).get("fingerprint") == fp
    except (OSError, ValueError):
        return False


def _run(cmd: list) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError("command failed: " + " ".join(cmd) + "\n" + p.stdout)


def build(verbose: bool = True, force: bool = False) -> str:
    fp = _fingerprint()
    bdir = _build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    with open(os.path.join(bdir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)  # one builder at a time; the others then find it built
        if not force and _up_to_date(bdir, fp):
            return lib
        nvcc = _nvcc()
        srcs = sources()
        t0 = time.time()
        done = threading.Event()

        def progress():
            while not done.wait(8.0):
                print(f"[iitj_llm_coopt_b200] compiling CUDA kernels for sm_100a ... {time.time() - t0:.0f}s",
                      file=sys.stderr, flush=True)

        if verbose:
            print(f"[iitj_llm_coopt_b200] building {LIB_NAME} from {len(srcs)} CUDA sources "
                  f"(first use, or sources changed)", file=sys.stderr, flush=True)
            threading.Thread(target=progress, daemon=True).start()
        try:
            objs = [os.path.join(bdir, os.path.basename(s)[:-3] + ".o") for s in srcs]
            with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
                jobs = [ex.submit(_run, [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", HERE, "-c", s, "-o", o])
                        for s, o in zip(srcs, objs)]
                for j in jobs:
                    j.result()
            tmp = lib + f".tmp{os.getpid()}"
            _run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs])
            os.replace(tmp, lib)
            with open(os.path.join(bdir, "stamp.json"), "w") as f:
                json.dump({"fingerprint": fp, "sources": [os.path.basename(s) for s in srcs]}, f)
        finally:
            done.set()
        if verbose:
            print(f"[iitj_llm_coopt_b200] built {lib} in {time.time() - t0:.0f}s", file=sys.stderr, flush=True)
    return lib


def library_path(verbose: bool = True) -> str:
    return build(verbose=verbose)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
