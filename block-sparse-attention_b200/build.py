"""Builds libbsa_b200.so (hand-written sm_100a kernels + C ABI) in-tree with nvcc.

Usage: ``python build.py [--force] [--verbose] [--phase-timers] [--csrc DIR --out LIB]``.  The library
lands next to the Python package (``block_sparse_attention/libbsa_b200.so``); object files go to
``build/``.  nvcc cross-compiles for sm_100a, so no GPU is needed to build.

``--phase-timers`` builds a second, instrumented library (``libbsa_b200_timers.so``, compiled with
``-DBSA_PHASE_TIMERS``): every warp role of the tcgen05 kernels accumulates clock deltas per phase, and
``phase_timers.py`` prints them as a table.  ``--csrc`` / ``--out`` compile another copy of the sources
into another file (A/B builds); ``BSA_B200_LIB`` selects the library the Python package loads.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "block_sparse_attention", "libbsa_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libbsa_b200.so cannot be built")
    return nvcc


def _newest_header_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return max(os.path.getmtime(p) for p in paths)


def _compile(src: str, force: bool, verbose: bool, csrc: str = CSRC, build_dir: str = BUILD, defines=()) -> str:
    obj = os.path.join(build_dir, src[:-3] + ".o")
    src_path = os.path.join(csrc, src)
    stamp = max(os.path.getmtime(src_path), _newest_header_mtime())
    if csrc != CSRC:
        stamp = max([stamp] + [os.path.getmtime(os.path.join(csrc, f)) for f in os.listdir(csrc)])
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= stamp:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-I", INCLUDE, "-c", src_path, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = os.path.join(build_dir, src[:-3] + ".ptxas.txt")
    with open(log, "w") as f:
        f.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return obj


TIMERS_LIB = os.path.join(HERE, "block_sparse_attention", "libbsa_b200_timers.so")


def build(force: bool = False, verbose: bool = False, phase_timers: bool = False, csrc: str = CSRC,
          out: str = "") -> str:
    """Compiles every .cu file under `csrc` and links them into `out` (default: the in-tree library, or the
    instrumented one with phase_timers)."""
    lib = out or (TIMERS_LIB if phase_timers else LIB)
    build_dir = BUILD
    if phase_timers:
        build_dir = os.path.join(BUILD, "timers")
    if out:
        build_dir = os.path.join(BUILD, "variant_" + os.path.splitext(os.path.basename(out))[0])
    os.makedirs(build_dir, exist_ok=True)
    defines = ("BSA_PHASE_TIMERS",) if phase_timers else ()
    srcs = sorted(f for f in os.listdir(csrc) if f.endswith(".cu"))
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose, csrc, build_dir, defines), srcs))
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(lib) or os.path.getmtime(lib) < newest:
        cmd = [_nvcc(), "-shared", "-o", lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--phase-timers", action="store_true", help="also build the instrumented library")
    ap.add_argument("--csrc", default=CSRC, help="directory holding the .cu / .cuh sources")
    ap.add_argument("--out", default="", help="output library (default: the in-tree one)")
    a = ap.parse_args()
    print(build(a.force, a.verbose, False, a.csrc, a.out))
    if a.phase_timers:
        print(build(a.force, a.verbose, True, a.csrc, ""))
