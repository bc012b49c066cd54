"""Builds tests/cpp/reference_tests.cpp -- the reference's integration tests written against the
C++ mirror of its host API (include/sile.hpp) -- and runs it."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def binary(tmp_path_factory):
    import sile_b200
    lib = sile_b200.build()
    out = str(tmp_path_factory.mktemp("cpp") / "reference_tests")
    lib_dir = os.path.dirname(lib)
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "reference_tests.cpp"), "-o", out,
                    "-L", lib_dir, "-lsile_cuda", f"-Wl,-rpath,{lib_dir}"], check=True)
    return out


def test_host_only_cases(binary):
    """Device selection, error kinds and messages: no device is touched."""
    r = subprocess.run([binary, "--host"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "3 cases, 0 failures" in r.stdout


@pytest.mark.gpu
def test_reference_tests_on_the_cuda_device(binary):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    r = subprocess.run([binary], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "10 cases, 0 failures" in r.stdout
