"""Build the sm_100a kernel library in-tree with nvcc.

``python -m ollama_b200.kernels.build`` compiles every ``.cu`` of this directory for
``compute_100a / sm_100a`` and links ``libb200ops.so`` next to the sources (and the C++ host
helpers of ``ollama_b200/native`` into ``libb200host.so``).  Objects are rebuilt only when their
source (or a header) is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
NATIVE = os.path.join(os.path.dirname(HERE), "native")
LIB = os.path.join(HERE, "libb200ops.so")
HOSTLIB = os.path.join(NATIVE, "libb200host.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC,-fvisibility=hidden"]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    nvcc = _nvcc()
    srcs = sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))
    hdrs = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))]
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    for s in srcs:
        src, obj = os.path.join(HERE, s), os.path.join(objdir, s[:-3] + ".o")
        if force or _stale(obj, [src] + hdrs):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj] + (["-Xptxas", "-v"] if verbose else [])
            jobs.append((s, cmd))

    def run(job):
        name, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return name, r.returncode, r.stdout + r.stderr

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for name, rc, out in ex.map(run, jobs):
                if verbose or rc:
                    sys.stderr.write(f"--- {name}\n{out}\n")
                if rc:
                    raise RuntimeError(f"nvcc failed on {name}")
    objs = [os.path.join(objdir, s[:-3] + ".o") for s in srcs]
    if force or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-lcuda"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    build_host(verbose, force)
    return LIB


def build_host(verbose: bool = False, force: bool = False) -> str | None:
    """C++ host-side helpers (no CUDA needed): device query, BPE merge loop, GGUF block codecs."""
    if not os.path.isdir(NATIVE):
        return None
    srcs = sorted(os.path.join(NATIVE, f) for f in os.listdir(NATIVE) if f.endswith(".cpp"))
    if not srcs:
        return None
    if force or _stale(HOSTLIB, srcs):
        cmd = ["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-shared", "-fPIC", "-fvisibility=hidden", "-o", HOSTLIB, *srcs, "-ldl", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("host library build failed")
    probe_src, probe_bin = os.path.join(NATIVE, "devquery.cpp"), os.path.join(NATIVE, "devquery")
    if os.path.exists(probe_src) and (force or _stale(probe_bin, [probe_src])):      # the device probe also exists as a stand-alone child program
        r = subprocess.run(["g++", "-O2", "-std=c++17", "-DB2_DEVQUERY_MAIN", probe_src, "-ldl", "-o", probe_bin], capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("device probe build failed")
    return HOSTLIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
