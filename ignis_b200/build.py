"""Builds the CUDA library in-tree: ignis_b200/libignis_b200.so (sm_100a only).

    python -m ignis_b200.build [--force] [--verbose] [--trace]

Every .cu and .cpp under csrc/ is compiled with nvcc to an object (in parallel) and linked into one
shared library with the CUDA runtime linked statically, so the file loads beside any PyTorch
build. nvcc cross-compiles without a GPU.

--trace builds a second library beside it, ignis_b200/libignis_b200_trace.so: the same objects except
the NVFP4 decode kernel compiled with -DB200Q_GEMV_TRACE (phase time stamps per CTA, read by
`bench.py --workload timeline`). The shipped library never carries the stamps.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libignis_b200.so")
TRACE_LIB = os.path.join(HERE, "libignis_b200_trace.so")
TRACE_SOURCES = ("nvfp4_gemv.cu",)   # the files B200Q_GEMV_TRACE changes
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _deps() -> list[str]:
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    headers += glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h"))
    return headers


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _compile(src: str, verbose: bool, trace: bool = False) -> str:
    obj = os.path.join(OBJ, os.path.splitext(os.path.basename(src))[0] + (".trace.o" if trace else ".o"))
    if _stale(obj, [src] + _deps()):
        cmd = [NVCC, *FLAGS, "-c", src, "-o", obj] + (["-Xptxas", "-v"] if verbose else []) + (["-DB200Q_GEMV_TRACE"] if trace else [])
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    if force:
        for f in glob.glob(os.path.join(OBJ, "*.o")):
            os.remove(f)
    sources = _sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), sources))
    if force or _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
               "-Xlinker", "--exclude-libs=ALL"]
        subprocess.run(cmd, check=True)
    return LIB


def build_trace(verbose: bool = False) -> str:
    """The library with the decode kernel's phase stamps compiled in (see the module text)."""
    build(verbose=verbose)
    objs = []
    for src in _sources():
        traced = os.path.basename(src) in TRACE_SOURCES
        objs.append(_compile(src, verbose, trace=True) if traced else os.path.join(OBJ, os.path.splitext(os.path.basename(src))[0] + ".o"))
    if _stale(TRACE_LIB, objs):
        subprocess.run([NVCC, "-shared", "-o", TRACE_LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
                        "-Xlinker", "--exclude-libs=ALL"], check=True)
    return TRACE_LIB


if __name__ == "__main__":
    if "--trace" in sys.argv:
        print(build_trace(verbose="--verbose" in sys.argv))
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
