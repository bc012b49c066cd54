"""Builds and runs the C++ test programs under tests/cpp:
reference_tests.cpp   the reference's integration tests written against the C++ mirror of its
                      host API (include/sile.hpp);
recogniser_tests.cpp  kernel descriptions (the mirror of sile_hir::Kernel, include/sile_hir.hpp)
                      through sile::recognise, then on the device."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path_factory, name):
    import sile_b200
    lib = sile_b200.build()
    out = str(tmp_path_factory.mktemp("cpp") / name)
    lib_dir = os.path.dirname(lib)
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", name + ".cpp"), "-o", out,
                    "-L", lib_dir, "-lsile_cuda", f"-Wl,-rpath,{lib_dir}"], check=True)
    return out


@pytest.fixture(scope="module")
def binary(tmp_path_factory):
    return _build(tmp_path_factory, "reference_tests")


@pytest.fixture(scope="module")
def recogniser_binary(tmp_path_factory):
    return _build(tmp_path_factory, "recogniser_tests")


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


def test_recogniser_host_cases(recogniser_binary):
    """Structural recognition of the reference's example kernels and refusal of near misses."""
    r = subprocess.run([recogniser_binary, "--host"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "3 cases, 0 failures" in r.stdout


@pytest.mark.gpu
def test_recognised_kernels_on_the_cuda_device(recogniser_binary):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    r = subprocess.run([recogniser_binary], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "7 cases, 0 failures" in r.stdout
