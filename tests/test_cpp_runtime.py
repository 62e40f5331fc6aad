"""Builds and runs the C++ runtime tests (tests/cpp/test_runtime.cu) with nvcc."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.gpu
def test_cpp_runtime_suite(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = tmp_path / "test_runtime"
    build = subprocess.run(
        [nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(ROOT / "nanotitan_b200/csrc/runtime"),
         str(ROOT / "tests/cpp/test_runtime.cu"), "-o", str(exe)], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and "ALL PASSED" in run.stdout, run.stdout + run.stderr
