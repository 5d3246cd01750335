"""Runs the C++ host-layer tests (tests/cpp/kernel_tests.cpp): the reference's
Rust kernel tests restated against whetstone_b200/host/whetstone_host.hpp."""

import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "tests" / "cpp" / "bin" / "kernel_tests"


def test_cpp_host_layer_compiles():
    subprocess.run(["make", "-C", str(ROOT / "tests" / "cpp")], check=True, capture_output=True)
    assert BIN.exists()


def test_cpp_paged_kv_manager_tests_pass():
    """tests/cpp/paged_kv_tests.cpp: the page manager and scheduler used from C++ (no GPU)."""
    subprocess.run(["make", "-C", str(ROOT / "tests" / "cpp")], check=True, capture_output=True)
    proc = subprocess.run([str(BIN.parent / "paged_kv_tests")], capture_output=True, text=True,
                          timeout=60)
    assert proc.returncode == 0 and "0 failed" in proc.stdout, proc.stdout + proc.stderr


@pytest.mark.gpu
def test_cpp_kernel_tests_pass():
    if not BIN.exists():
        subprocess.run(["make", "-C", str(ROOT / "tests" / "cpp")], check=True, capture_output=True)
    proc = subprocess.run([str(BIN)], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "0 failed" in proc.stdout and proc.stdout.count("ok ") == 14, proc.stdout
