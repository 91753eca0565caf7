"""Builds the CPU oracle (test infrastructure, never part of the shipped library).

    python oracle/build.py            # oracle/liboracle.so, and oracle/_ref/libref.so when the
                                      # reference checkout is present

`liboracle.so` is the plain-C restatement (b200q_oracle.c). `_ref/libref.so` is the reference's
own host-side oracle code compiled from its headers in place (ref_driver.cpp includes them by
path; no reference source is copied). The second build is skipped, keeping any prebuilt file,
when the reference checkout is absent.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: B200Q_REFERENCE_ROOT, else a directory `reference` beside this repository
REFERENCE = os.environ.get("B200Q_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")

ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libref.so")


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_oracle(force: bool = False) -> str:
    src = [os.path.join(HERE, "b200q_oracle.c"), os.path.join(HERE, "b200q_oracle.h")]
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-pthread", "-std=c11", "-o", ORACLE_SO, src[0], "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def build_ref(force: bool = False) -> str | None:
    """Compiles the reference's host oracle in place; None when it cannot be built here."""
    kernel = os.path.join(REFERENCE, "kernel")
    if not os.path.isdir(kernel):
        return REF_SO if os.path.exists(REF_SO) else None
    src = os.path.join(HERE, "ref_driver.cpp")
    if not force and _newer(REF_SO, [src]):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = [
        "g++", "-O2", "-std=c++20", "-fPIC", "-shared", "-o", REF_SO, src,
        "-I", os.path.join(kernel, "vendor", "tests"),
        "-I", os.path.join(kernel, "vendor", "src"),
        "-I", os.path.join(kernel, "vendor", "include"),
        "-I", os.path.join(kernel, "tests"),
        "-I", os.path.join(kernel, "include"),
        "-I", os.path.join(CUDA_HOME, "include"),
        "-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart",
        "-Wl,-rpath," + os.path.join(CUDA_HOME, "lib64"),
    ]
    subprocess.run(cmd, check=True)
    return REF_SO


def main() -> None:
    force = "--force" in sys.argv
    print("oracle:", build_oracle(force))
    print("reference oracle:", build_ref(force) or "not built (reference checkout absent)")


if __name__ == "__main__":
    main()
