"""The C-ABI library builds, loads and exports every symbol the header declares (no GPU)."""
import ctypes
import re

from ishizuki_b200 import _lib, build


def test_library_builds_and_loads():
    assert build.build().exists()
    _lib.load()


def test_every_declared_symbol_is_exported(tmp_path):
    header = (build.PKG.parent / "include" / "ishizuki_cuda.h").read_text()
    declared = set(re.findall(r"\b(ishi_[a-z0-9_]+)\s*\(", header))
    declared -= {"ishi_status"}
    lib = ctypes.CDLL(str(build.LIB))
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, f"declared but not exported: {missing}"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_constants_that_need_no_device():
    lib = _lib.load()
    # GGUFTests.blockGeometry (Tests/IshizukiKitTests/GGUFTests.swift:17-35)
    assert [lib.ishi_ggml_type_size(t) for t in (12, 14, 17)] == [144, 210, 74]
    assert [lib.ishi_ggml_type_size(t) for t in (10, 16, 18, 19, 21, 22, 23, 29)] == [84, 66, 98, 50, 110, 82, 136, 56]
    assert [lib.ishi_ggml_block_size(t) for t in (12, 14, 17, 11)] == [256, 256, 256, 0]
    # VerifyMatmulTests.rowFloor
    assert lib.ishi_reference_minimum_rows(248_320 * 5120 * 2 // 8) == 2
    assert lib.ishi_reference_minimum_rows(17_408 * 5120 * 2 // 8) == 3
    assert lib.ishi_reference_minimum_rows(6144 * 5120 * 2 // 8) == 4
    assert lib.ishi_reference_minimum_rows(1024 * 5120 * 2 // 8) == 6
    assert lib.ishi_status_string(2).decode().startswith("shape")


def test_no_device_is_an_error_not_a_fallback():
    lib = _lib.load()
    import torch

    if torch.cuda.is_available():
        return
    handle = ctypes.c_void_p()
    assert lib.ishi_ctx_create(0, ctypes.byref(handle)) != _lib.OK
    assert not handle
