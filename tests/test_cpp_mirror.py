"""The C++ host mirror (include/rg_b200.hpp): compiles on CPU, runs on the GPU."""
import os
import subprocess

import pytest

from rustygradients_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "host_mirror_test")


def _compile():
    lib = build.build()
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp"),
           "-o", EXE, "-L", os.path.dirname(lib), "-lrg_b200", "-Wl,-rpath," + os.path.dirname(lib)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return EXE


def test_cpp_mirror_compiles_and_links():
    assert os.path.exists(_compile())


@pytest.mark.gpu
def test_cpp_mirror_runs():
    exe = _compile()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout + r.stderr
