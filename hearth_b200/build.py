"""Builds hearth_b200/libhearth_b200.so in-tree with nvcc for sm_100a.

Run as `python -m hearth_b200.build` (add --force to rebuild everything, -v to
print register / shared-memory usage from ptxas).  Translation units compile
in parallel and are re-built only when their source or a header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libhearth_b200.so")

SOURCES = ["abi.cu", "quantize.cu", "producers.cu", "repack.cu", "gemv_dp4a.cu", "kquant.cu", "noalloc.cu", "gemm_tc.cu", "gemm_tc_rows.cu", "tc_peak.cu", "argmax.cu", "gguf.cu", "f32act.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(os.path.dirname(HERE), "include", "hb200.h"))
    return hs


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


# The bounds-checked debug build: the translation units whose kernels carry index checks (and the host layer, which
# reports them) are compiled again with -DHB200_BOUNDS; the others are shared with the normal build.
BOUNDS_LIB = os.path.join(HERE, "libhearth_b200_bounds.so")
BOUNDS_SOURCES = ["abi.cu", "quantize.cu", "producers.cu", "gemv_dp4a.cu", "kquant.cu", "noalloc.cu"]


def build_bounds(force: bool = False) -> str:
    """libhearth_b200_bounds.so: the same library with -DHB200_BOUNDS (load it with HB200_LIB=<path>)."""
    build(force=force)
    obj_b = os.path.join(HERE, "build_bounds")
    os.makedirs(obj_b, exist_ok=True)
    nvcc = _nvcc()
    headers = _headers()
    jobs = []
    for src in BOUNDS_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(obj_b, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + headers):
            jobs.append((src, [nvcc] + NVCC_FLAGS + ["-DHB200_BOUNDS", "-c", s, "-o", o]))

    def run(job):
        src, cmd = job
        p = subprocess.run(cmd, capture_output=True, text=True)
        return src, p.returncode, p.stdout + p.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for src, rc, out in ex.map(run, jobs):
                if rc:
                    sys.stderr.write(f"--- {src} (bounds)\n{out}\n")
                    raise RuntimeError(f"nvcc failed on {src} (bounds-checked build)")
    objs = [os.path.join(obj_b if s in BOUNDS_SOURCES else OBJ, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or _stale(BOUNDS_LIB, objs):
        cmd = [nvcc, "-shared", "-o", BOUNDS_LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link failed (bounds-checked build)")
    return BOUNDS_LIB


def build(force: bool = False, verbose: bool = False) -> str:
    """HB200_NVCC_EXTRA in the environment adds nvcc flags (a -D switch for a measurement build, -Xptxas options); a
    build with extra flags always recompiles everything."""
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    extra = os.environ.get("HB200_NVCC_EXTRA", "").split()
    force = force or bool(extra)
    headers = _headers()
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + headers):
            cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        p = subprocess.run(cmd, capture_output=True, text=True)
        return src, p.returncode, p.stdout + p.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for src, rc, out in ex.map(run, jobs):
                if verbose or rc:
                    sys.stderr.write(f"--- {src}\n{out}\n")
                if rc:
                    raise RuntimeError(f"nvcc failed on {src}")
    objs = [os.path.join(OBJ, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    if "--bounds" in sys.argv:
        print(build_bounds(force="--force" in sys.argv))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
