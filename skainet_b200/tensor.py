"""Host-side mirror of the reference's op / backend interface for the quantized path,
written over the C ABI (ctypes).  Names, argument meaning and error behaviour follow the
Kotlin originals so that tests read like the reference's own:

  Shape            core/src/commonMain/kotlin/sk/ai/net/Shape.kt
  QuantTensor      a Tensor (core/src/commonMain/kotlin/sk/ai/net/Tensor.kt:6-92) whose
                   elements are raw GGUF blocks resident in HBM
  (QuantLinear, Module and the parameter classes live in nn.py)
  GGMLQuantizationType / GGML_QUANT_SIZES / quant_shape_to_byte_shape
                   gguf/src/commonMain/kotlin/sk/ai/net/gguf/Constants.kt:14-90, Quants.kt:10-20

Where the reference throws IllegalArgumentException this raises ValueError with the same
message ("Shapes do not align.").  Other failures raise SknError carrying the status code.
"""
from __future__ import annotations

import ctypes
import enum
from typing import Optional, Sequence

import numpy as np

from . import _ffi

SKN_OK, SKN_ERR_SHAPE, SKN_ERR_TYPE, SKN_ERR_ALIGN, SKN_ERR_OOM = 0, 1, 2, 3, 4
SKN_ERR_CUDA, SKN_ERR_TIMEOUT, SKN_ERR_BAD_HANDLE, SKN_ERR_ARG, SKN_ERR_COMM, SKN_ERR_BUSY = 5, 6, 7, 8, 9, 10


class GGMLQuantizationType(enum.IntEnum):
    """Constants.kt:14-52 (the block types this backend runs: the four of the hot path with their
    own kernels, and Q4_1 / Q5_0 / Q5_1 / Q5_K / Q2_K / Q3_K / IQ4_NL / IQ4_XS on the dequantiser and
    the generic dequant-dot)."""
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    IQ4_NL = 20
    IQ4_XS = 23


QK_K = 256  # Constants.kt:55
GGML_QUANT_SIZES = {  # Constants.kt:58-90
    GGMLQuantizationType.Q4_0: (32, 2 + 16),
    GGMLQuantizationType.Q8_0: (32, 2 + 32),
    GGMLQuantizationType.Q4_K: (256, 2 + 2 + QK_K // 2 + 12),
    GGMLQuantizationType.Q6_K: (256, 2 + QK_K // 2 + QK_K // 4 + QK_K // 16),
    GGMLQuantizationType.Q4_1: (32, 2 + 2 + 16),
    GGMLQuantizationType.Q5_0: (32, 2 + 4 + 16),
    GGMLQuantizationType.Q5_1: (32, 2 + 2 + 4 + 16),
    GGMLQuantizationType.Q5_K: (256, 2 + 2 + 12 + QK_K // 8 + QK_K // 2),
    GGMLQuantizationType.Q2_K: (256, 2 + 2 + QK_K // 16 + QK_K // 4),
    GGMLQuantizationType.Q3_K: (256, 2 + QK_K // 4 + QK_K // 8 + 12),
    GGMLQuantizationType.IQ4_NL: (32, 2 + 16),
    GGMLQuantizationType.IQ4_XS: (256, 2 + 2 + QK_K // 2 + QK_K // 64),
}


def quant_shape_to_byte_shape(shape: Sequence[int], quant_type: GGMLQuantizationType) -> tuple:
    """Quants.kt:10-20."""
    block_size, type_size = GGML_QUANT_SIZES[GGMLQuantizationType(quant_type)]
    if shape[-1] % block_size != 0:
        raise ValueError(
            f"Quantized tensor row size ({shape[-1]}) is not a multiple of "
            f"{GGMLQuantizationType(quant_type).name} block size ({block_size})")
    return tuple(shape[:-1]) + (shape[-1] // block_size * type_size,)


class SknError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


class Shape:
    """Shape.kt: dimensions, volume, rank."""

    def __init__(self, *dimensions: int):
        self.dimensions = tuple(int(d) for d in dimensions)

    @property
    def volume(self) -> int:
        v = 1
        for d in self.dimensions:
            v *= d
        return v

    @property
    def rank(self) -> int:
        return len(self.dimensions)

    def __eq__(self, other):
        return isinstance(other, Shape) and other.dimensions == self.dimensions

    def __hash__(self):
        return hash(self.dimensions)

    def __repr__(self):
        return "Shape: Dimensions = [" + " x ".join(str(d) for d in self.dimensions) + f"], Size (Volume) = {self.volume}"


def _raise(ctx_handle, code: int):
    # a refused (busy) call leaves its message with the refused thread, not in the context
    msg = _ffi.lib().skn_last_error(None if code == SKN_ERR_BUSY else ctx_handle).decode("utf-8", "replace")
    if code == SKN_ERR_SHAPE:
        raise ValueError(msg)
    raise SknError(code, msg)


def _check(ctx_handle, code: int):
    if code != SKN_OK:
        _raise(ctx_handle, code)


def _ptr(a) -> Optional[int]:
    """Raw address of a numpy array (host) or a torch tensor (host or device)."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    if hasattr(a, "data_ptr"):
        return a.data_ptr()
    if isinstance(a, int):
        return a
    raise TypeError(f"cannot take the address of {type(a)}")


class Context:
    """One CUDA device + stream (skn_ctx).  Use as a context manager or call close()."""

    def __init__(self, device: int = 0):
        self._h = ctypes.c_void_p()
        L = _ffi.lib()
        rc = L.skn_ctx_create(int(device), ctypes.byref(self._h))
        if rc != SKN_OK:
            self._h = ctypes.c_void_p()
            _raise(None, rc)
        self.device = int(device)

    @property
    def handle(self):
        return self._h

    def set_stream(self, cuda_stream: Optional[int]):
        _check(self._h, _ffi.lib().skn_ctx_set_stream(self._h, cuda_stream))

    def set_relaxed_order(self, on: bool):
        """Declare consecutive device-pointer launches independent (they may overlap)."""
        _check(self._h, _ffi.lib().skn_ctx_set_option(self._h, 1, 1 if on else 0))

    def set_prefill_min_m(self, m: int):
        """Batch size from which matmuls use the tensor cores (bf16 operands); 0 = never."""
        _check(self._h, _ffi.lib().skn_ctx_set_option(self._h, 2, int(m)))

    def set_fused_exchange(self, on):
        """Tensor-parallel decode steps of one or two rows: push partial products from the matvec
        epilogue and sum them in the next projection's preparation of x (SKN_OPT_FUSED_EXCHANGE).
        True / False, or None for the automatic choice (on from four ranks)."""
        _check(self._h, _ffi.lib().skn_ctx_set_option(self._h, 3, -1 if on is None else (1 if on else 0)))

    def set_kv_f16(self, on: bool):
        """Decoders created afterwards keep their KV caches in fp16 (SKN_OPT_KV_F16)."""
        _check(self._h, _ffi.lib().skn_ctx_set_option(self._h, 4, 1 if on else 0))

    def set_kv_dtype(self, dtype: str):
        """Element type of the KV caches of decoders created afterwards: "f32", "f16" or "q8_0" (SKN_OPT_KV_DTYPE)."""
        _check(self._h, _ffi.lib().skn_ctx_set_option(self._h, 6, KVCache.DTYPES[dtype]))

    def set_wait_limit_ms(self, ms: int):
        """How long a kernel of the inter-GPU exchange waits for its peers before it reports
        SKN_ERR_TIMEOUT (SKN_OPT_WAIT_LIMIT_MS; 0 restores the default of two seconds)."""
        _check(self._h, _ffi.lib().skn_ctx_set_option(self._h, 5, int(ms)))

    def sync(self):
        _check(self._h, _ffi.lib().skn_sync(self._h))

    def close(self):
        if self._h:
            _ffi.lib().skn_ctx_destroy(self._h)
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

    # TensorFactory-style entry (TensorFactory.kt:7-9 takes a DoubleArray and cannot carry
    # raw blocks; this is the added factory function for quantized data)
    def create_quantized(self, shape: Shape, quant_type, blocks) -> "QuantTensor":
        return QuantTensor(self, shape, quant_type, blocks)


class QuantTensor:
    """A [out, in] weight stored as raw GGUF blocks in HBM."""

    def __init__(self, ctx: Context, shape: Shape, quant_type, blocks, *, shard=None):
        if isinstance(shape, (tuple, list)):
            shape = Shape(*shape)
        if shape.rank != 2:
            raise ValueError("a quantized weight is a rank-2 tensor [out, in]")
        self.ctx = ctx
        self.quant_type = int(quant_type)
        raw = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        self._h = ctypes.c_void_p()
        n_rows, n_cols = shape.dimensions
        L = _ffi.lib()
        if shard is None:
            rc = L.skn_tensor_upload_quant(ctx.handle, self.quant_type, n_rows, n_cols, raw.ctypes.data, raw.size,
                                           ctypes.byref(self._h))
            self.shape = shape
        else:
            r0, rc_, c0, cc = shard
            rc = L.skn_tensor_upload_quant_shard(ctx.handle, self.quant_type, n_rows, n_cols, raw.ctypes.data, raw.size,
                                                 r0, rc_, c0, cc, ctypes.byref(self._h))
            self.shape = Shape(rc_, cc)
        if rc != SKN_OK:
            self._h = ctypes.c_void_p()
            _raise(ctx.handle, rc)

    @property
    def handle(self):
        return self._h

    @property
    def rank(self) -> int:
        return self.shape.rank

    @property
    def size(self) -> int:
        return self.shape.volume

    def info(self) -> dict:
        t, r, c = ctypes.c_int32(), ctypes.c_int64(), ctypes.c_int64()
        rb, pitch, dev = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_void_p()
        _check(self.ctx.handle, _ffi.lib().skn_tensor_info(self._h, ctypes.byref(t), ctypes.byref(r), ctypes.byref(c),
                                                          ctypes.byref(rb), ctypes.byref(pitch), ctypes.byref(dev)))
        return {"type": t.value, "n_rows": r.value, "n_cols": c.value, "row_bytes": rb.value,
                "row_pitch_bytes": pitch.value, "device_blocks": dev.value}

    def dequantize(self) -> np.ndarray:
        out = np.empty(self.shape.dimensions, dtype=np.float32)
        _check(self.ctx.handle, _ffi.lib().skn_dequantize(self.ctx.handle, self._h, out.ctypes.data))
        return out

    def matmul_t(self, x: np.ndarray, bias: Optional[np.ndarray] = None) -> np.ndarray:
        """x . W^T (+ bias): x is [K] or [M, K] fp32 on the host; result [N] or [M, N]."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim == 1:
            m, k, vec = 1, x.shape[0], True
        elif x.ndim == 2:
            m, k, vec = x.shape[0], x.shape[1], False
        else:
            raise ValueError("Shapes do not align.")
        n = self.shape.dimensions[0]
        y = np.empty((m, n), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        if b is not None and b.shape != (n,):
            raise ValueError("Shapes do not align.")
        _check(self.ctx.handle, _ffi.lib().skn_matmul(self.ctx.handle, self._h, x.ctypes.data, m, k, _ptr(b),
                                                     y.ctypes.data))
        return y[0] if vec else y

    def matmul_t_async(self, x: np.ndarray, out: np.ndarray, bias: Optional[np.ndarray] = None):
        """Host-pointer form that only enqueues (skn_matmul_async): x [K] or [M, K] and out [N] or [M, N] are
        C-contiguous fp32 host arrays that the caller keeps alive and untouched until Context.sync() returns
        (page-locked arrays keep the call free of staged copies)."""
        for a in (x, out) + (() if bias is None else (bias,)):
            if a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"]:
                raise ValueError("fp32 C-contiguous host arrays are required")
        m = 1 if x.ndim == 1 else x.shape[0]
        n = self.shape.dimensions[0]
        if x.ndim not in (1, 2) or out.size != m * n or (bias is not None and bias.shape != (n,)):
            raise ValueError("Shapes do not align.")
        _check(self.ctx.handle, _ffi.lib().skn_matmul_async(self.ctx.handle, self._h, x.ctypes.data, m, x.shape[-1],
                                                           _ptr(bias), out.ctypes.data))

    def matmul_t_dev(self, x_dev, m: int, y_dev, bias_dev=None, k: Optional[int] = None):
        """Device-pointer form: enqueue only (x_dev, y_dev: torch CUDA tensors or addresses)."""
        kk = self.shape.dimensions[1] if k is None else k
        _check(self.ctx.handle, _ffi.lib().skn_matmul_dev(self.ctx.handle, self._h, _ptr(x_dev), m, kk, _ptr(bias_dev),
                                                         _ptr(y_dev)))

    def close(self):
        if self._h:
            _ffi.lib().skn_tensor_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def ffn_swiglu(ctx: Context, wg: QuantTensor, wu: QuantTensor, wd: QuantTensor, x: np.ndarray) -> np.ndarray:
    """(silu(x Wg^T) * (x Wu^T)) Wd^T for x [M, K] (or [K]) on the host."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    vec = x.ndim == 1
    x2 = x.reshape(1, -1) if vec else x
    if x2.ndim != 2 or x2.shape[1] != wg.shape.dimensions[1]:
        raise ValueError("Shapes do not align.")
    y = np.empty((x2.shape[0], wd.shape.dimensions[0]), dtype=np.float32)
    _check(ctx.handle, _ffi.lib().skn_ffn_swiglu(ctx.handle, wg.handle, wu.handle, wd.handle, x2.ctypes.data,
                                                 x2.shape[0], y.ctypes.data))
    return y[0] if vec else y


class KVCache:
    """Device-resident KV cache (head-major ring) with decode attention.  `dtype` is "f32" (default), "f16" or
    "q8_0" (int8 with one fp16 scale per 32 head dims): the element type K and V are kept in; every method
    takes and returns fp32 either way."""

    DTYPES = {"f32": 0, "f16": 1, "q8_0": 2}

    def __init__(self, ctx: Context, batch: int, n_kv_heads: int, head_dim: int, capacity: int, dtype: str = "f32"):
        if dtype not in self.DTYPES:
            raise ValueError("dtype must be 'f32', 'f16' or 'q8_0'")
        self.ctx = ctx
        self.batch, self.n_kv_heads, self.head_dim, self.capacity = batch, n_kv_heads, head_dim, capacity
        self.dtype = dtype
        self._h = ctypes.c_void_p()
        rc = _ffi.lib().skn_kv_create_typed(ctx.handle, batch, n_kv_heads, head_dim, capacity, self.DTYPES[dtype],
                                            ctypes.byref(self._h))
        if rc != SKN_OK:
            self._h = ctypes.c_void_p()
            _raise(ctx.handle, rc)

    @property
    def handle(self):
        return self._h

    def reset(self):
        _check(self.ctx.handle, _ffi.lib().skn_kv_reset(self._h))

    def load(self, k: np.ndarray, v: np.ndarray, lens):
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        lens = np.ascontiguousarray(lens, dtype=np.int32)
        if k.shape != v.shape or k.ndim != 4 or k.shape[0] != self.batch or k.shape[1] != self.n_kv_heads \
                or k.shape[3] != self.head_dim or lens.shape != (self.batch,):
            raise ValueError("Shapes do not align.")
        _check(self.ctx.handle, _ffi.lib().skn_kv_load(self._h, k.ctypes.data, v.ctypes.data, k.shape[2],
                                                      lens.ctypes.data))

    def lengths(self):
        lens = np.empty(self.batch, dtype=np.int32)
        start = np.empty(self.batch, dtype=np.int32)
        _check(self.ctx.handle, _ffi.lib().skn_kv_lengths(self._h, lens.ctypes.data, start.ctypes.data))
        return lens, start

    def append(self, k_new: np.ndarray, v_new: np.ndarray):
        k_new = np.ascontiguousarray(k_new, dtype=np.float32)
        v_new = np.ascontiguousarray(v_new, dtype=np.float32)
        if k_new.shape != (self.batch, self.n_kv_heads, self.head_dim) or v_new.shape != k_new.shape:
            raise ValueError("Shapes do not align.")
        _check(self.ctx.handle, _ffi.lib().skn_kv_append(self._h, k_new.ctypes.data, v_new.ctypes.data))

    def append_dev(self, k_new_dev, v_new_dev):
        _check(self.ctx.handle, _ffi.lib().skn_kv_append_dev(self._h, _ptr(k_new_dev), _ptr(v_new_dev)))

    def gather(self, b: int, pos_begin: int, count: int):
        k = np.empty((self.n_kv_heads, count, self.head_dim), dtype=np.float32)
        v = np.empty_like(k)
        _check(self.ctx.handle, _ffi.lib().skn_kv_gather(self._h, b, pos_begin, count, k.ctypes.data, v.ctypes.data))
        return k, v

    def attend(self, q: np.ndarray, scale: Optional[float] = None) -> np.ndarray:
        """q [batch, n_q_heads, head_dim] on the host -> attention output of the same shape."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        if q.ndim != 3 or q.shape[0] != self.batch or q.shape[2] != self.head_dim:
            raise ValueError("Shapes do not align.")
        if scale is None:
            scale = 1.0 / float(np.sqrt(self.head_dim))
        out = np.empty_like(q)
        _check(self.ctx.handle, _ffi.lib().skn_attn_decode(self._h, q.ctypes.data, q.shape[1], scale, out.ctypes.data))
        return out

    def attend_dev(self, q_dev, n_q_heads: int, out_dev, scale: Optional[float] = None, scratch_dev=None):
        if scale is None:
            scale = 1.0 / float(np.sqrt(self.head_dim))
        _check(self.ctx.handle, _ffi.lib().skn_attn_decode_dev(self._h, _ptr(q_dev), n_q_heads, scale, _ptr(out_dev),
                                                              _ptr(scratch_dev)))

    def scratch_bytes(self, n_q_heads: int) -> int:
        return int(_ffi.lib().skn_attn_scratch_bytes(self._h, n_q_heads))

    def close(self):
        if self._h:
            _ffi.lib().skn_kv_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
