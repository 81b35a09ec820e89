"""Host-side mirror of the reference's GGUF reader API over the native, memory-mapped reader:

  GGUFFile(path).fields   name -> value      GGUFReader.fields   (GGUFReader.kt:60, :285-318)
  GGUFFile(path).tensors  [ReaderTensor]     GGUFReader.tensors  (GGUFReader.kt:61, :332-401)
  ReaderTensor            name, tensor_type, shape, n_elements, n_bytes, data_offset, data
                                             (GGUFReader.kt:35-44)

`data` of a quantized tensor is the raw blocks, unchanged (a zero-copy uint8 view of the mapping);
F32 / F16 / integer tensors come back as typed numpy views.  `upload(ctx, tensor)` puts a quantized
tensor in HBM without an intermediate copy.
"""
from __future__ import annotations

import ctypes
import struct
from dataclasses import dataclass
from typing import Any, Dict, List

import numpy as np

from . import _ffi
from .tensor import Context, QuantTensor, Shape, SknError, _check, _raise, SKN_OK

# GGUFValueType ids (gguf/src/commonMain/kotlin/sk/ai/net/gguf/Constants.kt)
_SCALAR = {0: ("<B", 1), 1: ("<b", 1), 2: ("<H", 2), 3: ("<h", 2), 4: ("<I", 4), 5: ("<i", 4), 6: ("<f", 4),
           7: ("<?", 1), 10: ("<Q", 8), 11: ("<q", 8), 12: ("<d", 8)}
_NP = {0: np.uint8, 1: np.int8, 2: np.uint16, 3: np.int16, 4: np.uint32, 5: np.int32, 6: np.float32, 7: np.bool_,
       10: np.uint64, 11: np.int64, 12: np.float64}
_TENSOR_NP = {0: np.float32, 1: np.float16, 24: np.int8, 25: np.int16, 26: np.int32, 27: np.int64, 28: np.float64}


@dataclass
class ReaderTensor:
    name: str
    tensor_type: int
    shape: tuple          # file order: shape[0] is the contiguous dimension
    n_elements: int
    n_bytes: int
    data_offset: int
    data: np.ndarray
    index: int


class GGUFFile:
    def __init__(self, path: str):
        self._h = ctypes.c_void_p()
        L = _ffi.lib()
        rc = L.skn_gguf_open(str(path).encode(), ctypes.byref(self._h))
        if rc != SKN_OK:
            self._h = ctypes.c_void_p()
            _raise(None, rc)
        v, nt, nk, al, do = ctypes.c_int32(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        _check(None, L.skn_gguf_counts(self._h, ctypes.byref(v), ctypes.byref(nt), ctypes.byref(nk), ctypes.byref(al),
                                       ctypes.byref(do)))
        self.version, self.alignment, self.data_offset = v.value, al.value, do.value
        self.fields: Dict[str, Any] = {}
        for i in range(nk.value):
            k, val = self._kv(i)
            self.fields[k] = val
        self.tensors: List[ReaderTensor] = [self._tensor(i) for i in range(nt.value)]

    def _kv(self, i: int):
        L = _ffi.lib()
        key, vt, et = ctypes.c_char_p(), ctypes.c_int32(), ctypes.c_int32()
        ptr, cnt = ctypes.c_void_p(), ctypes.c_int64()
        _check(None, L.skn_gguf_kv(self._h, i, ctypes.byref(key), ctypes.byref(vt), ctypes.byref(et), ctypes.byref(ptr),
                                   ctypes.byref(cnt)))
        k = key.value.decode("utf-8", "replace")
        t, n = vt.value, cnt.value
        if t in _SCALAR:
            fmt, size = _SCALAR[t]
            return k, struct.unpack(fmt, ctypes.string_at(ptr.value, size))[0]
        if t == 8:
            return k, ctypes.string_at(ptr.value, n).decode("utf-8", "replace") if n else ""
        e = et.value
        if e == 8:
            out, p = [], ptr.value
            for _ in range(n):
                ln = struct.unpack("<Q", ctypes.string_at(p, 8))[0]
                out.append(ctypes.string_at(p + 8, ln).decode("utf-8", "replace"))
                p += 8 + ln
            return k, out
        dt = np.dtype(_NP[e])
        if n == 0:
            return k, np.empty(0, dtype=dt)
        buf = (ctypes.c_uint8 * (n * dt.itemsize)).from_address(ptr.value)
        return k, np.frombuffer(buf, dtype=dt).copy()

    def _tensor(self, i: int) -> ReaderTensor:
        L = _ffi.lib()
        name, nd, tt = ctypes.c_char_p(), ctypes.c_int32(), ctypes.c_int32()
        dims = (ctypes.c_int64 * 4)()
        off, nb, ptr = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_void_p()
        _check(None, L.skn_gguf_tensor(self._h, i, ctypes.byref(name), ctypes.byref(nd), dims, ctypes.byref(tt),
                                       ctypes.byref(off), ctypes.byref(nb), ctypes.byref(ptr)))
        shape = tuple(int(dims[d]) for d in range(nd.value))
        n_el = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if nb.value:
            raw = np.frombuffer((ctypes.c_uint8 * nb.value).from_address(ptr.value), dtype=np.uint8)
        else:
            raw = np.empty(0, dtype=np.uint8)
        raw.flags.writeable = False
        if tt.value in _TENSOR_NP:
            data = raw.view(_TENSOR_NP[tt.value]).reshape(shape[::-1])
        else:
            data = raw
        return ReaderTensor(name.value.decode("utf-8", "replace"), tt.value, shape, n_el, nb.value, off.value, data, i)

    def upload(self, ctx: Context, tensor: ReaderTensor) -> QuantTensor:
        """Quantized tensor -> HBM, straight from the mapping."""
        h = ctypes.c_void_p()
        rc = _ffi.lib().skn_gguf_upload(ctx.handle, self._h, tensor.index, ctypes.byref(h))
        if rc != SKN_OK:
            _raise(ctx.handle, rc)
        t = QuantTensor.__new__(QuantTensor)
        t.ctx, t.quant_type, t._h = ctx, tensor.tensor_type, h
        rows = tensor.shape[1] if len(tensor.shape) > 1 else 1
        t.shape = Shape(rows, tensor.shape[0])
        return t

    def close(self):
        # views handed out earlier point into the mapping: drop them before closing
        if self._h:
            self.tensors = []
            _ffi.lib().skn_gguf_close(self._h)
            self._h = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
