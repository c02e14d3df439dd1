"""The C++ host side (namespace llm, the reference's own signatures): builds the assert-style test
programs under tests/cpp/ — written like the reference's tests — and runs them."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")
BIN = os.path.join(CPP, "bin")


def _build(name):
    from cuda_llm_b200 import build
    import oracle
    shim = build.build_shim()
    assert shim, "C++ shim sources missing"
    oracle.build(ref=False)
    os.makedirs(BIN, exist_ok=True)
    exe, src = os.path.join(BIN, name), os.path.join(CPP, name + ".cpp")
    deps = [src, shim, os.path.join(ROOT, "oracle", "liboracle.so")]
    if os.path.exists(exe) and all(os.path.getmtime(d) <= os.path.getmtime(exe) for d in deps):
        return exe
    lib_dir, orc_dir = os.path.dirname(shim), os.path.join(ROOT, "oracle")
    cmd = [os.environ.get("NVCC", "nvcc"), "-std=c++17", "-O1", "--default-stream", "per-thread",
           "-I", os.path.join(ROOT, "include"), src, "-o", exe, "-L", lib_dir, "-lb2llm", "-lb2ops", "-L", orc_dir, "-loracle",
           "-Xlinker", f"-rpath,{lib_dir}", "-Xlinker", f"-rpath,{orc_dir}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    return exe


def _run(exe):
    proc = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    return proc.stdout


def test_tensor_host_program():
    assert "test_tensor_host passed" in _run(_build("test_tensor_host"))


@pytest.mark.gpu
def test_ops_cuda_program():
    out = _run(_build("test_ops_cuda_b200"))
    assert "test_ops_cuda_b200 passed" in out and "bit-exact" in out


@pytest.mark.gpu
def test_sampling_program():
    assert "test_sampling_b200 passed" in _run(_build("test_sampling_b200"))
