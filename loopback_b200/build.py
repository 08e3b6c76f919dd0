"""Builds libloopback_b200.so (the CUDA kernels and their C ABI) in-tree with nvcc for sm_100a.

Each source of csrc/ is compiled to an object file under csrc/build/ (in parallel, and only when it or a header
changed), then the objects are linked into one shared library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libloopback_b200.so")
SOURCES = ("lb_api.cu", "lb_write.cu", "lb_write_mma.cu", "lb_read_fwd.cu", "lb_read_bwd.cu", "lb_read_bwd_f32.cu", "lb_step.cu",
           "lb_noalloc.cu", "lb_peer.cu")
HEADERS = ("lb_common.cuh", "lb_kernels.h", "lb_read_bwd_impl.cuh", os.path.join("..", "..", "include", "loopback_b200.h"))
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-ccbin", "g++",
         "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA kernels of loopback_b200 cannot be built")


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _headers_mtime() -> float:
    return max(os.path.getmtime(os.path.join(CSRC, h)) for h in HEADERS if os.path.exists(os.path.join(CSRC, h)))


def _obj_of(src: str) -> str:
    return os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")


def _stale(src: str, hdr_t: float) -> bool:
    o = _obj_of(src)
    return not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(src), hdr_t)


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + [os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.exists(f) and os.path.getmtime(f) > t for f in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu of csrc/ for sm_100a and link them into one shared library. Returns its path."""
    if not force and not needs_build():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc, hdr_t = _nvcc(), _headers_mtime()
    todo = [s for s in sources() if force or _stale(s, hdr_t)]

    def compile_one(src):
        cmd = [nvcc, *ARCH, *FLAGS, "-c", src, "-o", _obj_of(src)]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        return src, subprocess.run(cmd, capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as pool:
        for src, proc in pool.map(compile_one, todo):
            if proc.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n" + proc.stdout + proc.stderr)
            if verbose:
                print(proc.stderr)
    link = [nvcc, *ARCH, "-shared", "-Xcompiler", "-fPIC", "-ccbin", "g++", "-cudart", "static", "-o", LIB,
            *[_obj_of(s) for s in sources()]]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc link failed:\n" + proc.stdout + proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="-f" in sys.argv or "-v" in sys.argv, verbose="-v" in sys.argv))
