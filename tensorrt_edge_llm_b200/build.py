"""In-tree build of the native libraries (no torch headers, seconds per file).

``libtelb_kernels.so``  every ``csrc/kernels/*.cu`` compiled for sm_100a with an ``extern "C"`` API
                        (loaded through ctypes by ``ops/cuda.py``).
``_telb_runtime*.so``   the C++ runtime (scheduler, page table, sampler glue, tokenizer …) as a
                        pybind11 module.

Run ``python -m tensorrt_edge_llm_b200.build`` (add ``--force`` to rebuild everything, ``-v`` for
ptxas resource usage).  Objects are cached under ``build/`` keyed by source mtime.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import sysconfig
from typing import List

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
LIBDIR = os.path.join(ROOT, "_lib")
BUILD = os.path.join(os.path.dirname(ROOT), "build", "telb")

NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "--expt-relaxed-constexpr",
              "-diag-suppress", "177", "-diag-suppress", "550"]
# sources listed here are compiled without --use_fast_math (none at present: the RoPE table is built by torch ops)
NO_FAST_MATH: set = set()


def _newer(src: str, dst: str, deps: List[str]) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(p) > t for p in [src] + deps)


def _run(cmd: List[str]) -> str:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build_kernels(force=False, verbose=False) -> str:
    kdir = os.path.join(CSRC, "kernels")
    os.makedirs(BUILD, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    headers = [os.path.join(kdir, f) for f in os.listdir(kdir) if f.endswith((".h", ".cuh", ".inc"))]
    srcs = sorted(f for f in os.listdir(kdir) if f.endswith(".cu"))
    objs, jobs = [], []
    for f in srcs:
        src, obj = os.path.join(kdir, f), os.path.join(BUILD, f[:-3] + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            flags = [x for x in NVCC_FLAGS if not (f in NO_FAST_MATH and x == "--use_fast_math")]
            if verbose:
                flags = flags + ["-Xptxas", "-v"]
            jobs.append([NVCC] + flags + ["-c", src, "-o", obj])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(_run, jobs):
                if verbose and out.strip():
                    print(out)
    lib = os.path.join(LIBDIR, "libtelb_kernels.so")
    if jobs or not os.path.exists(lib):
        # link beside the target and rename: a process (or a snapshot of the tree) never sees a half-written library
        _run([NVCC, "-shared", "-o", lib + ".tmp"] + objs + ["-lcudart_static", "-lpthread", "-ldl", "-lrt"])
        os.replace(lib + ".tmp", lib)
    return lib


def build_runtime(force=False, verbose=False) -> str:
    rdir = os.path.join(CSRC, "runtime")
    if not os.path.isdir(rdir):
        return ""
    srcs = sorted(f for f in os.listdir(rdir) if f.endswith(".cpp"))
    if not srcs:
        return ""
    import pybind11
    os.makedirs(BUILD, exist_ok=True)
    headers = [os.path.join(rdir, f) for f in os.listdir(rdir) if f.endswith((".h", ".hpp", ".inc"))]
    inc = ["-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], "-I" + rdir]
    cxx = shutil.which("g++") or "g++"
    flags = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter", "-fvisibility=hidden", "-pthread"]
    objs, jobs = [], []
    for f in srcs:
        src, obj = os.path.join(rdir, f), os.path.join(BUILD, "rt_" + f[:-4] + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            jobs.append([cxx] + flags + inc + ["-c", src, "-o", obj])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    ext = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    lib = os.path.join(LIBDIR, "_telb_runtime" + ext)
    if jobs or not os.path.exists(lib):
        _run([cxx, "-shared", "-o", lib + ".tmp"] + objs + ["-pthread"])
        os.replace(lib + ".tmp", lib)
    return lib


def build_race_check(sanitizer: str = "thread") -> str:
    """The native runtime's concurrency check (``csrc/runtime/checks/race_check.cpp``) linked with the runtime sources under a
    sanitizer (``thread``, ``address`` or ``undefined``); returns the executable's path.  It runs on the host, no GPU."""
    if sanitizer not in ("thread", "address", "undefined"):
        raise ValueError("sanitizer must be thread, address or undefined")
    rdir = os.path.join(CSRC, "runtime")
    srcs = [os.path.join(rdir, f) for f in sorted(os.listdir(rdir)) if f.endswith(".cpp") and f != "bindings.cpp"]
    srcs.append(os.path.join(rdir, "checks", "race_check.cpp"))
    os.makedirs(BUILD, exist_ok=True)
    exe = os.path.join(BUILD, f"race_check_{sanitizer}")
    cxx = shutil.which("g++") or "g++"
    _run([cxx, "-O1", "-g", "-std=c++17", "-fno-omit-frame-pointer", f"-fsanitize={sanitizer}", "-pthread", "-I" + rdir] + srcs + ["-o", exe])
    return exe


def build_all(force=False, verbose=False):
    return build_kernels(force, verbose), build_runtime(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--sanitize", choices=["thread", "address", "undefined"], default=None,
                    help="build (only) the native runtime's concurrency check under this sanitizer and print its path")
    a = ap.parse_args()
    if a.sanitize:
        print(build_race_check(a.sanitize))
    else:
        print(build_all(a.force, a.verbose))
