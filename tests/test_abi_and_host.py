"""CPU-side checks of the boundary: the library loads, exports every symbol the public
header declares, and the no-GPU error paths behave; plus the host mirror's pure logic."""
import ctypes
import os
import re

import numpy as np
import pytest

import skainet_b200 as skn
from skainet_b200 import _ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "skainet_cuda.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(skn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = ctypes.CDLL(_ffi.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 16
    for n in names:
        assert hasattr(L, n), f"{n} is declared in skainet_cuda.h but not exported"


def test_python_binding_covers_the_header():
    assert sorted(_ffi.SIGNATURES) == declared_symbols()


def test_version_and_geometry():
    L = _ffi.lib()
    assert L.skn_version() == 100
    e, b = ctypes.c_int32(), ctypes.c_int32()
    for t, (ee, bb) in skn.GGML_QUANT_SIZES.items():
        assert L.skn_quant_geometry(int(t), ctypes.byref(e), ctypes.byref(b)) == 0
        assert (e.value, b.value) == (ee, bb)
    assert L.skn_quant_geometry(16, ctypes.byref(e), ctypes.byref(b)) == 2  # SKN_ERR_TYPE (IQ2_XXS not built)
    rb = ctypes.c_int64()
    assert L.skn_quant_row_bytes(12, 4096, ctypes.byref(rb)) == 0 and rb.value == 2304
    assert L.skn_quant_row_bytes(12, 4000, ctypes.byref(rb)) == 1           # SKN_ERR_SHAPE
    assert b"not a multiple" in L.skn_last_error(None)


def test_bad_handles_are_rejected_without_a_gpu():
    L = _ffi.lib()
    assert L.skn_ctx_destroy(None) == 7
    assert L.skn_tensor_destroy(None) == 7
    assert L.skn_sync(None) == 7
    out = ctypes.c_void_p()
    assert L.skn_tensor_upload_quant(None, 12, 1, 256, None, 144, ctypes.byref(out)) == 7
    assert L.skn_kv_create_typed(None, 1, 1, 64, 8, 1, ctypes.byref(out)) == 7
    assert L.skn_matmul_async(None, None, None, 1, 256, None, None) == 7
    dt = ctypes.c_int32()
    assert L.skn_kv_dtype(None, ctypes.byref(dt)) == 7


def test_quant_shape_to_byte_shape():
    # Quants.kt:10-20
    assert skn.quant_shape_to_byte_shape((4096, 4096), skn.GGMLQuantizationType.Q4_K) == (4096, 2304)
    assert skn.quant_shape_to_byte_shape((14336,), skn.GGMLQuantizationType.Q6_K) == (11760,)
    with pytest.raises(ValueError, match="not a multiple of Q4_0 block size"):
        skn.quant_shape_to_byte_shape((3, 33), skn.GGMLQuantizationType.Q4_0)


def test_shape_mirror():
    # ShapeTest.kt:10-43
    s = skn.Shape(2, 3, 4)
    assert s.volume == 24 and s.rank == 3
    assert skn.Shape(2, 3) == skn.Shape(2, 3) and skn.Shape(2, 3) != skn.Shape(3, 2)
    assert skn.Shape().volume == 1 and skn.Shape().rank == 0
    assert "2 x 3 x 4" in repr(s)
