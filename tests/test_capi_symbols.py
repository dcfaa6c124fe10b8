"""The C-ABI library loads and exports every symbol include/atlas_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

from atlasinfer_b200 import _capi, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()  # no-op when the library is newer than its sources
    return _capi.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "atlas_b200.h")).read()
    return sorted(set(re.findall(r"ATLAS_API[^;(]*?\b(atlas_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(_capi.EXPORTS)


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_version_and_status_strings(lib):
    assert lib.atlas_version() >= 100
    assert lib.atlas_status_string(0) == b"ok"
    assert b"unsupported" in lib.atlas_status_string(_capi.ERR_UNSUPPORTED)


def test_argument_validation_needs_no_gpu(lib):
    # rejected before any CUDA call: no kernel is launched here
    counts = (ctypes.c_int64 * 4)()
    st = lib.atlas_quantize(None, 128, 100, 3.0, None, None, None, 0, None, counts, None, 0, None)
    assert st == _capi.ERR_UNSUPPORTED and b"block_size" in lib.atlas_last_error()
    st = lib.atlas_quantize(None, -1, 128, 3.0, None, None, None, 0, None, counts, None, 0, None)
    assert st == _capi.ERR_BAD_ARGUMENT
    st = lib.atlas_repack(None, 0, None, None, 0, None, 4, 100, 128, None, None, None, None, None, None, None)
    assert st == _capi.ERR_UNSUPPORTED
    st = lib.atlas_dequantize(None, 5, None, None, 0, None, 128, 128, None, None)
    assert st == _capi.ERR_BAD_ARGUMENT  # 5 codes + 0 outliers do not cover 128 elements
    assert lib.atlas_tiles_bytes(200, 256) == 256 * 256
    assert lib.atlas_quantize_workspace_bytes(8192 * 3 + 1, 128) == 16 + 8 * 4


def test_unsupported_maps_to_not_implemented(lib):
    with pytest.raises(NotImplementedError):
        _capi.check(_capi.ERR_UNSUPPORTED, "x")
    with pytest.raises(_capi.AtlasError):
        _capi.check(_capi.ERR_LAUNCH, "x")
