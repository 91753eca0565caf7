"""The boundary seen from compiled code: a C99 program over include/*.h alone and a C++ program over
the ops shim (include/b200q_ninfer_ops.hpp), both built here with gcc / g++ against the in-tree
library. Host mode needs no device; GPU mode (marked) runs real products on device 0."""
from __future__ import annotations

import os
import shutil
import struct
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "include")
LIBDIR = os.path.join(ROOT, "ignis_b200")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build(tmp_path, source: str, with_cuda: bool) -> str:
    from ignis_b200 import _lib

    _lib.load()   # the library must exist: there is nothing to link against otherwise
    cxx = source.endswith(".cpp")
    compiler = shutil.which("g++" if cxx else "gcc")
    if compiler is None:
        pytest.skip("no host compiler")
    exe = str(tmp_path / (os.path.basename(source).split(".")[0] + ("_gpu" if with_cuda else "_host")))
    cmd = [compiler, "-std=c++17" if cxx else "-std=c99", "-O1", "-Wall", "-Wextra", "-Werror", "-pedantic", f"-I{INCLUDE}",
           os.path.join(ROOT, "tests", "c", source), "-o", exe, f"-L{LIBDIR}", "-l:libignis_b200.so", f"-Wl,-rpath,{LIBDIR}"]
    if with_cuda:
        cmd += ["-DWITH_CUDA", "-isystem", f"{CUDA}/include", f"-L{CUDA}/lib64", "-lcudart", f"-Wl,-rpath,{CUDA}/lib64"]
    if not cxx:
        cmd += ["-lm"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def _run(args: list[str]) -> str:
    res = subprocess.run(args, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.strip().endswith("ok")
    return res.stdout


def _container(tmp_path) -> str:
    from ignis_b200 import artifact as art

    g = art.blockscale_geometry([128, 64])
    blob = np.zeros(g["encoded_bytes"], np.uint8)
    blob[g["weight_divisor_offset"]:] = np.frombuffer(struct.pack("<f", 448.0), np.uint8)
    path = str(tmp_path / "c.ninfer")
    art.write_container(path, "m", "w", [
        {"name": "text/layers/0/mlp/down", "format": "NVFP4", "layout": "blockscale-k16-m128x4-v1", "shape": [128, 64], "data": blob},
        {"name": "text/layers/0/mlp/down_projection/input_scale_divisor", "format": "FP32", "layout": "contiguous-le-v1", "shape": [],
         "data": np.array([2.0], np.float32).view(np.uint8)},
        {"name": "frontend/tokenizer.json", "encoding": "raw-bytes-v1", "data": b"{}"}])
    return path


def test_c99_driver_host(tmp_path):
    out = _run([_build(tmp_path, "abi_driver.c", False), "host", _container(tmp_path)])
    assert "object text/layers/0/mlp/down: 4612 bytes" in out


def test_cpp_ops_shim_host(tmp_path):
    _run([_build(tmp_path, "ops_shim_driver.cpp", False), "host"])


@pytest.mark.gpu
def test_c99_driver_gpu(tmp_path):
    _run([_build(tmp_path, "abi_driver.c", True), "gpu"])


@pytest.mark.gpu
def test_cpp_ops_shim_gpu(tmp_path):
    _run([_build(tmp_path, "ops_shim_driver.cpp", True), "gpu"])
