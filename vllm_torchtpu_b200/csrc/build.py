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


CHECKED_LIB_NAME = "libb200_attention_checked.so"
CHECKED_SOURCES = ("attention.cu", "attention_tc.cu", "attention_mla.cu")


def lib_path() -> str:
    return os.path.join(HERE, LIB_NAME)


def checked_lib_path() -> str:
    return os.path.join(HERE, CHECKED_LIB_NAME)


def build_checked(force: bool = False) -> str:
    """The attention kernels once more with ``-DB200_BOUNDS_CHECK`` (block ids and page indices that fall
    outside their tables are counted) as a second library.  It leaves the helpers it shares with the main
    library undefined; load the main library first (``ops.cuda.lib`` does)."""
    objdir = os.path.join(HERE, "build_checked")
    os.makedirs(objdir, exist_ok=True)
    hdr = _headers_mtime()
    objs, jobs = [], []
    for src in CHECKED_SOURCES:
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        sp = os.path.join(HERE, src)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(sp), hdr):
            jobs.append([NVCC, *ARCH, *COMMON, "-DB200_BOUNDS_CHECK", "-c", sp, "-o", obj])
    with ThreadPoolExecutor(max_workers=max(1, len(jobs))) as ex:
        for r, cmd in zip(ex.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs), jobs):
            if r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr + "\n")
                raise RuntimeError("nvcc failed (bounds-checked build)")
    out = checked_lib_path()
    if jobs or not os.path.exists(out):
        r = subprocess.run([NVCC, *ARCH, "-shared", "-o", out, *objs, "-lcudart_static", "-lpthread", "-ldl",
                            "-lrt"], capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed (bounds-checked build)")
    return out


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
    print(build_checked(force="-f" in sys.argv))
