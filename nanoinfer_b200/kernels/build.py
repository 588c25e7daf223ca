"""Compiles the CUDA sources under ``csrc/`` into one shared library for sm_100a.

The library is built with ``nvcc`` alone (no torch headers), one object file per
source in parallel, and is kept in ``nanoinfer_b200/_build`` next to the package
(or in ``$NANOINFER_B200_BUILD_DIR``, or a per-user temporary folder when the
package folder cannot be written).  A stamp of the sources' contents decides
whether anything has to be rebuilt; while compiling, a line is printed now and
then so that a first call does not look hung.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List, Optional

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
LIB_NAME = "libnib_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (
        os.environ.get("NVCC"),
        os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (set NVCC or CUDA_HOME); the CUDA kernels cannot be built")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _stamp() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC_DIR)):
        if name.endswith((".cu", ".cuh", ".h")):
            h.update(name.encode())
            with open(os.path.join(CSRC_DIR, name), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build_dir() -> str:
    env = os.environ.get("NANOINFER_B200_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    in_tree = os.path.join(PKG_DIR, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"nanoinfer_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of the up-to-date library, building it first if needed."""
    d = build_dir()
    lib = os.path.join(d, LIB_NAME)
    stamp_file = os.path.join(d, "stamp.txt")
    stamp = _stamp()
    if os.path.isfile(lib) and os.path.isfile(stamp_file):
        with open(stamp_file) as fh:
            if fh.read().strip() == stamp:
                return lib
    if not build:
        raise BuildError(f"{lib} is missing or out of date")
    _compile_all(d, lib, verbose)
    with open(stamp_file, "w") as fh:
        fh.write(stamp)
    return lib


def _run(cmd: List[str]) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError("command failed: " + " ".join(cmd) + "\n" + p.stdout)
    if p.stdout.strip() and os.environ.get("NANOINFER_B200_BUILD_VERBOSE"):
        print(p.stdout, file=sys.stderr)


def _compile_all(d: str, lib: str, verbose: bool, extra: Optional[List[str]] = None) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()

    def say(msg: str) -> None:
        if verbose:
            print(f"[nanoinfer_b200] {msg}", file=sys.stderr, flush=True)

    say(f"compiling {len(srcs)} CUDA sources for sm_100a into {d} (first call only)")
    objs = [os.path.join(d, s[:-3] + ".o") for s in srcs]
    jobs = {}
    workers = max(1, min(len(srcs), os.cpu_count() or 1))
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
        for s, o in zip(srcs, objs):
            cmd = [nvcc, *NVCC_FLAGS, *(extra or []), "-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, s), "-o", o]
            jobs[pool.submit(_run, cmd)] = s
        pending = set(jobs)
        while pending:
            done, pending = concurrent.futures.wait(pending, timeout=10.0)
            for f in done:
                f.result()  # raises BuildError with the compiler's output
                say(f"  compiled {jobs[f]} ({time.time() - t0:.0f} s)")
            if pending:
                say(f"  still compiling {', '.join(sorted(jobs[f] for f in pending))} ({time.time() - t0:.0f} s)")
    tmp = lib + f".tmp{os.getpid()}"
    _run([nvcc, "-shared", "-o", tmp, *objs])
    os.replace(tmp, lib)
    say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")


def ptxas_report() -> str:
    """Registers, spills and shared memory of every kernel (``-Xptxas -v``), as text."""
    nvcc = find_nvcc()
    out = []
    with tempfile.TemporaryDirectory() as tmp:
        for s in sources():
            cmd = [nvcc, *NVCC_FLAGS, "-Xptxas", "-v", "-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, s),
                   "-o", os.path.join(tmp, s + ".o")]
            p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            out.append(f"== {s}\n{p.stdout}")
    return "\n".join(out)


if __name__ == "__main__":
    print(library_path())
