"""CPU tests of the C-ABI boundary: the library builds, loads, exports every symbol the header
declares, the ctypes table matches the header, and argument checks reject bad calls before any
CUDA work (no compute call is made here)."""
import ctypes as C
import os
import re

import pytest

from aether_ml_b200 import _lib
from aether_ml_b200.build import build_library

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "aether_b200.h")


@pytest.fixture(scope="module")
def lib():
    build_library()
    return _lib.lib()


def header_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aether_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    names = header_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), "library does not export %s" % n
        assert n in _lib.SIGNATURES, "no ctypes signature for %s" % n
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_counters(lib):
    assert lib.aether_version() >= 100
    assert lib.aether_launch_count() >= 0
    assert lib.aether_device_status() == 0


def test_conv_argument_checks(lib):
    assert lib.aether_conv2d_fwd(None, None, None, None, None, None, 0, None) == -1
    assert b"null descriptor" in lib.aether_last_error()
    d = _lib.AetherConvDesc(2, 8, 8, 64, 64, 3, 3, 1, 1, 1, 1, 0)
    assert lib.aether_conv2d_fwd(C.byref(d), None, None, None, None, None, 0, None) == -1
    bad = _lib.AetherConvDesc(2, 8, 8, 64, 64, 3, 3, 0, 1, 1, 1, 0)          # stride 0
    assert lib.aether_conv2d_fwd(C.byref(bad), 16, 16, None, 16, None, 0, None) == -1
    big = _lib.AetherConvDesc(1, 2, 2, 4, 4, 5, 5, 1, 1, 0, 0, 2)            # filter larger than input
    assert lib.aether_conv2d_bwd(C.byref(big), 16, 16, 16, None, 16, 16, None, 0, 0, None) == -1
    mis = _lib.AetherConvDesc(2, 8, 8, 64, 64, 3, 3, 1, 1, 1, 1, 0)
    assert lib.aether_conv2d_fwd(C.byref(mis), 8, 16, None, 16, None, 0, None) == -1   # misaligned x
    assert b"aligned" in lib.aether_last_error()
    mode = _lib.AetherConvDesc(2, 8, 8, 64, 64, 3, 3, 1, 1, 1, 1, 7)
    assert lib.aether_conv2d_workspace_bytes(C.byref(mode)) == 0


def test_workspace_query_is_pure(lib):
    for mode in (0, 1, 2):
        d = _lib.AetherConvDesc(256, 56, 56, 64, 128, 3, 3, 1, 1, 1, 1, mode)
        n = lib.aether_conv2d_workspace_bytes(C.byref(d))
        assert n > 0 and n % 1024 == 0
    d = _lib.AetherConvDesc(128, 32, 32, 3, 32, 3, 3, 1, 1, 1, 1, 0)          # first layer: CUDA-core path
    assert lib.aether_conv2d_workspace_bytes(C.byref(d)) > 0
    assert lib.aether_bn_workspace_bytes(128 * 32 * 32, 32) > 0


def test_layer_argument_checks(lib):
    assert lib.aether_bn_fwd_train(*([None] * 8), 10, 4, 1e-5, 0.9, None, 0, None) == -1
    assert lib.aether_pool_fwd(None, None, None, 1, 4, 4, 4, 2, 2, 2, 2, 0, None) == -1
    assert lib.aether_pool_fwd(16, 16, 16, 1, 1, 4, 4, 2, 2, 2, 2, 0, None) == -1     # window larger than input
    assert lib.aether_adam_step(None, None, None, None, 4, 1e-3, .9, .999, 1e-7, .1, .001, 1.0, None) == -1
    assert lib.aether_adam_step(16, 16, 16, 16, 4, 1e-3, .9, .999, 1e-7, 0.0, .001, 1.0, None) == -1
    assert lib.aether_softmax_cce(None, None, None, None, None, None, 4, 10, 0.0, 0.0, 0, None) == -1
    assert lib.aether_leaky_relu_fwd(8, 16, 4, 0.0, None) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.AetherError):
        _lib.lib()
