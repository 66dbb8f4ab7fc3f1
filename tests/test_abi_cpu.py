"""CPU-side checks of the C ABI: the library loads, exports every declared symbol, and refuses to run
without a GPU (there is no fallback path).  No compute call is made here."""
import ctypes
import os
import re

import pytest

import loom_b200
from loom_b200 import build as lb_build
from loom_b200 import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    return lb_build.build()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "loom_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(loom_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built):
    L = ctypes.CDLL(built)
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), "missing export " + n


def test_binding_table_matches_header(built):
    assert sorted(cabi.SIGNATURES) == declared_symbols()


def test_api_version(built):
    assert cabi.lib().loom_b200_api_version() == 1


def test_no_gpu_means_error_not_fallback(built):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert cabi.lib().loom_b200_device_count() == 0
    with pytest.raises(loom_b200.LoomB200Error) as ei:
        loom_b200.Context(0)
    assert ei.value.code == -4
    assert "no CPU fallback" in str(ei.value)


def test_null_context_calls_return_errors(built):
    L = cabi.lib()
    assert L.loom_b200_sync(None) == -1
    assert L.loom_b200_quantize_activation(None, 1, 16, None, None, None) == -1
    assert L.loom_b200_ternary_linear(None, None, 1, None, None, None, None, -1, None, None) == -1
    assert b"NULL" in L.loom_b200_last_error(None)


def build_c_harness(tmp_path, lib):
    """tests/abi_harness.c compiled by gcc against include/loom_b200.h and linked with the library: the view a cgo or
    FFI host has of it."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    exe = str(tmp_path / "abi_harness")
    libdir = os.path.dirname(lib)
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I" + os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "abi_harness.c"),
                    "-L" + libdir, "-lloom_b200", "-Wl,-rpath," + libdir, "-lm", "-o", exe], check=True)
    return exe


def test_plain_c_caller_links_and_gets_an_error_without_a_gpu(built, tmp_path):
    import subprocess
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the compute run of the harness is a gpu test")
    r = subprocess.run([build_c_harness(tmp_path, built)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "no device" in r.stdout and "no CPU fallback" in r.stdout


@pytest.mark.gpu
def test_plain_c_caller_computes_a_dense_layer(built, tmp_path):
    import subprocess
    r = subprocess.run([build_c_harness(tmp_path, built)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 of 96 outputs differ" in r.stdout
