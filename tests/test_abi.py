"""CPU tests of the boundary: the library builds, loads and exports exactly the
entry points the header declares (no compute calls: no GPU here)."""
import os
import re
import subprocess

import pytest

import rustygradients_b200 as rg
from rustygradients_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "rg_b200.h")


def _declared():
    src = open(HEADER).read()
    return sorted(set(re.findall(r"RG_API[^;()]*?\b(rg_\w+)\s*\(", src)))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    assert os.path.exists(path)
    out = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True, check=True).stdout
    exported = sorted(set(re.findall(r" T (rg_\w+)", out)))
    declared = _declared()
    assert len(declared) >= 45
    assert exported == declared


def test_python_binding_covers_the_header():
    assert sorted(_lib.SIGNATURES) == _declared()
    lib = _lib.load()
    assert lib.rg_version().startswith(b"rg_b200")
    assert lib.rg_last_error() is not None


def test_header_cites_the_reference_for_every_entry_point():
    src = open(HEADER).read()
    assert "src/backend/mod.rs" in src and "src/models/gpt.rs" in src and "wasm_api.rs:97-163" in src


def test_header_compiles_as_c():
    r = subprocess.run(["gcc", "-std=c99", "-fsyntax-only", "-x", "c", HEADER], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_no_gpu_is_an_error_not_a_fallback():
    if rg.B200Backend.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(rg.BackendError):
        rg.B200Backend(0)
