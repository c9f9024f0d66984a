"""Build the in-tree CUDA library for sm_100a.

Every ``.cu`` file in this directory is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` to an object and the
objects are linked into ``libb200_kernels.so`` next to the sources.  nvcc
cross-compiles without a GPU, so the build also runs on CPU-only machines.
Objects are rebuilt only when their source (or a header) is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libb200_kernels.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
          "-Xcompiler", "-fvisibility=default"]


def lib_path() -> str:
    return os.path.join(HERE, LIB_NAME)


def _sources() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cu", ".cpp")))


def _headers_mtime() -> float:
    hs = [os.path.getmtime(os.path.join(HERE, f)) for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))]
    return max(hs) if hs else 0.0


def build(verbose: bool = False, force: bool = False, extra_flags: tuple = ()) -> str:
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    hdr = _headers_mtime()
    jobs = []
    objs = []
    for src in _sources():
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        sp = os.path.join(HERE, src)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(sp), hdr):
            cmd = [NVCC, *ARCH, *COMMON, *extra_flags, "-c", sp, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr + "\n")
            failed |= r.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    out = lib_path()
    if jobs or not os.path.exists(out):
        cmd = [NVCC, *ARCH, "-shared", "-o", out, *objs, "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return out


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
