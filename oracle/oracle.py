"""CPU oracle, Python side.  TEST INFRASTRUCTURE ONLY.

Two independent restatements of the GGUF block arithmetic live here:

* ``liboracle.so`` (``skn_oracle.c``, loaded through ctypes) -- the C restatement that
  also provides the fp64 matmul in the reference's loop order, the fp64 attention /
  SwiGLU / RMSNorm / RoPE definitions and the timed CPU baseline;
* the vectorised numpy functions ``np_dequant_*`` below -- used to cross-check the C
  code without any compiled artefact.

Parity status: unpinned by the reference (sk-ai-net/skainet v0.0.7 has no quantized
arithmetic and no golden vector for it; gguf/.../Quants.kt:8 is a TODO).  Both
restatements are pinned against gguf-py 0.19.0 through ``tests/golden/``.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may
import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

Q4_0, Q8_0, Q4_K, Q6_K = 2, 8, 12, 14  # Constants.kt:14-52
Q4_1, Q5_0, Q5_1, Q5_K = 3, 6, 7, 13
Q2_K, Q3_K, IQ4_NL, IQ4_XS = 10, 11, 20, 23
GEOMETRY = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210),
            Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q5_K: (256, 176),
            Q2_K: (256, 84), Q3_K: (256, 110), IQ4_NL: (32, 18), IQ4_XS: (256, 136)}  # Constants.kt:58-90

_lib = None


def build(force: bool = False) -> str:
    """Compile liboracle.so next to its source (gcc, a second or two)."""
    src = os.path.join(_HERE, "skn_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        c_i64, c_int, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.skn_oracle_row_bytes.restype = c_i64
        L.skn_oracle_row_bytes.argtypes = [c_int, c_i64]
        L.skn_oracle_dequant.argtypes = [c_int, vp, c_i64, vp]
        L.skn_oracle_dequant_f64.argtypes = [c_int, vp, c_i64, c_i64, vp]
        L.skn_oracle_linear_ref.argtypes = [vp, c_i64, c_i64, vp, c_i64, vp, vp]
        L.skn_oracle_matmul.argtypes = [c_int, vp, c_i64, c_i64, c_i64, vp, c_i64, vp, vp, c_int]
        L.skn_oracle_ffn_swiglu.argtypes = [c_int, vp, vp, c_int, vp, c_i64, c_i64, c_i64, vp, c_i64,
                                            vp, vp, c_int]
        L.skn_oracle_attn_decode.argtypes = [vp, vp, vp, vp, vp, c_i64, c_i64, c_i64, c_i64, c_i64,
                                             ctypes.c_double, vp]
        L.skn_oracle_rmsnorm.argtypes = [vp, vp, c_i64, c_i64, ctypes.c_double, vp]
        L.skn_oracle_rope.argtypes = [vp, vp, c_i64, c_i64, c_i64, ctypes.c_double, vp]
        _lib = L
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def row_bytes(qtype: int, n_cols: int) -> int:
    """Quants.kt:10-20; raises ValueError where the reference throws."""
    r = lib().skn_oracle_row_bytes(qtype, n_cols)
    if r < 0:
        raise ValueError(f"row size {n_cols} is not a multiple of the block size of type {qtype}")
    return int(r)


def dequant(qtype: int, blocks: np.ndarray) -> np.ndarray:
    """uint8 blocks (any shape whose byte count is a whole number of blocks) -> flat fp32."""
    e, b = GEOMETRY[qtype]
    raw = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    assert raw.size % b == 0
    n = raw.size // b
    out = np.empty(n * e, dtype=np.float32)
    assert lib().skn_oracle_dequant(qtype, _p(raw), n, _p(out)) == 0
    return out


def matmul(qtype: int, blocks: np.ndarray, N: int, K: int, X: np.ndarray, threads: int = 0,
           row_pitch: int | None = None):
    """fp64 X[M,K] . W[N,K]^T, k-ascending accumulation.  Returns (Y[M,N], absdot[M,N])."""
    raw = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    X = np.ascontiguousarray(X, dtype=np.float32).reshape(-1, K)
    M = X.shape[0]
    pitch = row_bytes(qtype, K) if row_pitch is None else row_pitch
    assert raw.size >= N * pitch
    Y = np.empty((M, N), dtype=np.float64)
    A = np.empty((M, N), dtype=np.float64)
    rc = lib().skn_oracle_matmul(qtype, _p(raw), pitch, N, K, _p(X), M, _p(Y), _p(A), threads)
    assert rc == 0, rc
    return Y, A


def linear_ref(qtype: int, blocks: np.ndarray, N: int, K: int, X: np.ndarray, bias=None,
               W64: np.ndarray | None = None) -> np.ndarray:
    """Reference-faithful Linear.forward (transposed copy + reference loop order), 1 thread."""
    X = np.ascontiguousarray(X, dtype=np.float32).reshape(-1, K)
    M = X.shape[0]
    if W64 is None:
        W64 = dequant_f64(qtype, blocks, N, K)
    Y = np.empty((M, N), dtype=np.float64)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    assert lib().skn_oracle_linear_ref(_p(W64), N, K, _p(X), M, _p(b), _p(Y)) == 0
    return Y


def dequant_f64(qtype: int, blocks: np.ndarray, N: int, K: int) -> np.ndarray:
    raw = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    W = np.empty((N, K), dtype=np.float64)
    assert lib().skn_oracle_dequant_f64(qtype, _p(raw), N, K, _p(W)) == 0
    return W


def ffn_swiglu(type_gu, wg, wu, type_d, wd, F, K, N, X, threads: int = 0, want_h: bool = False):
    X = np.ascontiguousarray(X, dtype=np.float32).reshape(-1, K)
    M = X.shape[0]
    Y = np.empty((M, N), dtype=np.float64)
    H = np.empty((M, F), dtype=np.float64) if want_h else None
    wg = np.ascontiguousarray(wg, dtype=np.uint8).reshape(-1)
    wu = np.ascontiguousarray(wu, dtype=np.uint8).reshape(-1)
    wd = np.ascontiguousarray(wd, dtype=np.uint8).reshape(-1)
    rc = lib().skn_oracle_ffn_swiglu(type_gu, _p(wg), _p(wu), type_d, _p(wd), F, K, N, _p(X), M,
                                     _p(Y), _p(H), threads)
    assert rc == 0, rc
    return (Y, H) if want_h else Y


def attn_decode(q, kc, vc, lens, start=None, scale: float | None = None) -> np.ndarray:
    """q [B,Hq,D], caches [B,Hkv,cap,D] fp32, lens [B] int32 -> fp64 [B,Hq,D]."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    kc = np.ascontiguousarray(kc, dtype=np.float32)
    vc = np.ascontiguousarray(vc, dtype=np.float32)
    lens = np.ascontiguousarray(lens, dtype=np.int32)
    st = None if start is None else np.ascontiguousarray(start, dtype=np.int32)
    B, Hq, D = q.shape
    _, Hkv, cap, _ = kc.shape
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    out = np.empty((B, Hq, D), dtype=np.float64)
    rc = lib().skn_oracle_attn_decode(_p(q), _p(kc), _p(vc), _p(lens), _p(st), B, Hq, Hkv, D, cap,
                                      float(scale), _p(out))
    assert rc == 0, rc
    return out


def rmsnorm(x, gain, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    x2 = x.reshape(-1, x.shape[-1])
    g = np.ascontiguousarray(gain, dtype=np.float32)
    y = np.empty(x2.shape, dtype=np.float64)
    assert lib().skn_oracle_rmsnorm(_p(x2), _p(g), x2.shape[0], x2.shape[1], float(eps), _p(y)) == 0
    return y.reshape(x.shape)


def rope(x, pos, theta: float) -> np.ndarray:
    """x [M,H,D] fp32, pos [M] int32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    M, H, D = x.shape
    y = np.empty(x.shape, dtype=np.float64)
    assert lib().skn_oracle_rope(_p(x), _p(pos), M, H, D, float(theta), _p(y)) == 0
    return y


# --------------------------------------------------------------------------------------
# Independent numpy restatement of the four block layouts (fp32 arithmetic throughout).
# --------------------------------------------------------------------------------------

def _f16(bytes2: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(bytes2).view(np.float16).astype(np.float32).reshape(-1)


def np_dequant_q4_0(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 18)
    d = _f16(b[:, 0:2])[:, None]
    qs = b[:, 2:18]
    lo = (qs & 15).astype(np.int8) - np.int8(8)
    hi = (qs >> 4).astype(np.int8) - np.int8(8)
    q = np.concatenate([lo, hi], axis=1).astype(np.float32)
    return (q * d).reshape(-1)


def np_dequant_q8_0(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 34)
    d = _f16(b[:, 0:2])[:, None]
    q = b[:, 2:34].view(np.int8).astype(np.float32)
    return (q * d).reshape(-1)


def np_quantize_q8_0(x: np.ndarray):
    """Q8_0 quantisation of fp32 values in blocks of 32 along the last axis, as the KV cache of type SKN_KV_Q8_0
    stores them.  The reference has no quantiser (its gguf module only reads: gguf/src/commonMain/kotlin/sk/ai/net/
    gguf/Quants.kt); this restates gguf-py 0.19.0 `quants.py`, Q8_0.quantize_blocks (itself bit-exact with ggml's
    quantize_row_q8_0_ref): d = max|x| / 127 in fp32, id = 1 / d (0 for an all-zero block), q = x * id rounded
    half away from zero, d kept as fp16.  Returns (q int8 [..., n], d float16 [..., n / 32])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.shape[-1] % 32 == 0
    blocks = x.reshape(-1, 32)
    d = (np.abs(blocks).max(axis=1, keepdims=True) / np.float32(127)).astype(np.float32)
    with np.errstate(all="ignore"):         # (a subnormal scale has an infinite inverse, as in the original)
        inv = np.where(d == 0, np.float32(0), np.float32(1) / d).astype(np.float32)
        t = (blocks * inv).astype(np.float32)
        q = (np.sign(t) * np.floor(np.abs(t) + np.float32(0.5))).astype(np.int8)      # roundf: half away from zero
        dh = d.astype(np.float16)
    return q.reshape(x.shape), dh.reshape(x.shape[:-1] + (x.shape[-1] // 32,))


def np_q8_0_roundtrip(x: np.ndarray) -> np.ndarray:
    """What a Q8_0 cache hands back for x: q * fp16(d), in fp32 (gguf-py Q8_0.dequantize_blocks)."""
    q, dh = np_quantize_q8_0(x)
    return (q.reshape(-1, 32).astype(np.float32) * dh.reshape(-1, 1).astype(np.float32)).reshape(q.shape)


def np_q4k_scales(s: np.ndarray):
    """s: [n,12] uint8 -> (sc[n,8], mn[n,8]) uint8."""
    sc = np.empty((s.shape[0], 8), dtype=np.uint8)
    mn = np.empty((s.shape[0], 8), dtype=np.uint8)
    sc[:, 0:4] = s[:, 0:4] & 63
    mn[:, 0:4] = s[:, 4:8] & 63
    sc[:, 4:8] = (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:8] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc, mn


def np_dequant_q4_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 144)
    n = b.shape[0]
    d = _f16(b[:, 0:2])[:, None]
    dmin = _f16(b[:, 2:4])[:, None]
    sc, mn = np_q4k_scales(b[:, 4:16])
    dl = (d * sc.astype(np.float32))[:, :, None]
    ml = (dmin * mn.astype(np.float32))[:, :, None]
    qs = b[:, 16:144].reshape(n, 4, 32)
    q = np.stack([qs & 15, qs >> 4], axis=2).reshape(n, 8, 32).astype(np.float32)
    return (dl * q - ml).reshape(-1)


def np_dequant_q6_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 210)
    n = b.shape[0]
    ql = b[:, 0:128].reshape(n, 2, 2, 32)       # [half, g&1, l]
    qh = b[:, 128:192].reshape(n, 2, 1, 32)     # [half, 1, l]
    sc = b[:, 192:208].view(np.int8).reshape(n, 2, 4, 2)  # [half, g, l/16]
    d = _f16(b[:, 208:210])[:, None, None, None]
    out = np.empty((n, 2, 4, 32), dtype=np.float32)
    for g in range(4):
        nib = (ql[:, :, g & 1, :] & 15) if g < 2 else (ql[:, :, g & 1, :] >> 4)
        hi = (qh[:, :, 0, :] >> (2 * g)) & 3
        q = (nib | (hi << 4)).astype(np.int8) - np.int8(32)
        dl = d[:, :, 0, :] * np.repeat(sc[:, :, g, :].astype(np.float32), 16, axis=2)
        out[:, :, g, :] = dl * q.astype(np.float32)
    return out.reshape(-1)


def _nib32(qs: np.ndarray) -> np.ndarray:
    """16 bytes per block -> 32 nibbles (low nibbles first), uint8."""
    return np.concatenate([qs & 15, qs >> 4], axis=1)


def _bits32(qh4: np.ndarray) -> np.ndarray:
    """4 little-endian bytes per block -> 32 bits (bit i = weight i), uint8."""
    w = np.ascontiguousarray(qh4).view(np.uint32).reshape(-1, 1)
    return ((w >> np.arange(32, dtype=np.uint32)[None, :]) & 1).astype(np.uint8)


def np_dequant_q4_1(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 20)
    d, m = _f16(b[:, 0:2])[:, None], _f16(b[:, 2:4])[:, None]
    return (d * _nib32(b[:, 4:20]).astype(np.float32) + m).reshape(-1)


def np_dequant_q5_0(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 22)
    d = _f16(b[:, 0:2])[:, None]
    q = (_nib32(b[:, 6:22]) | (_bits32(b[:, 2:6]) << 4)).astype(np.int8) - np.int8(16)
    return (d * q.astype(np.float32)).reshape(-1)


def np_dequant_q5_1(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 24)
    d, m = _f16(b[:, 0:2])[:, None], _f16(b[:, 2:4])[:, None]
    q = (_nib32(b[:, 8:24]) | (_bits32(b[:, 4:8]) << 4)).astype(np.float32)
    return (d * q + m).reshape(-1)


def np_dequant_q5_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 176)
    n = b.shape[0]
    d = _f16(b[:, 0:2])[:, None]
    dmin = _f16(b[:, 2:4])[:, None]
    sc, mn = np_q4k_scales(b[:, 4:16])
    dl = (d * sc.astype(np.float32))[:, :, None]
    ml = (dmin * mn.astype(np.float32))[:, :, None]
    qs = b[:, 48:176].reshape(n, 4, 32)
    nib = np.stack([qs & 15, qs >> 4], axis=2).reshape(n, 8, 32)
    hi = (b[:, 16:48][:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1
    q = (nib | (hi << 4)).astype(np.float32)
    return (dl * q - ml).reshape(-1)


def _crumbs256(qs: np.ndarray) -> np.ndarray:
    """64 bytes per block -> 256 two-bit fields: weight 128h + 32s + l = (qs[32h + l] >> 2s) & 3."""
    n = qs.shape[0]
    q = qs.reshape(n, 2, 1, 32) >> (2 * np.arange(4, dtype=np.uint8))[None, None, :, None]
    return (q & 3).reshape(n, 256)


def np_dequant_q2_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 84)
    n = b.shape[0]
    d, dmin = _f16(b[:, 80:82])[:, None], _f16(b[:, 82:84])[:, None]
    dl = (d * (b[:, 0:16] & 15).astype(np.float32))[:, :, None]
    ml = (dmin * (b[:, 0:16] >> 4).astype(np.float32))[:, :, None]
    q = _crumbs256(b[:, 16:80]).reshape(n, 16, 16).astype(np.float32)
    return (dl * q - ml).reshape(-1)


def np_dequant_q3_k(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 110)
    n = b.shape[0]
    d = _f16(b[:, 108:110])[:, None]
    sp = b[:, 96:108]
    i = np.arange(16)
    lo = np.where(i < 8, sp[:, i & 7] & 15, sp[:, i & 7] >> 4)
    hi = (sp[:, 8 + (i & 3)] >> (2 * (i >> 2)).astype(np.uint8)) & 3
    sc = (lo | (hi << 4)).astype(np.int8) - np.int8(32)
    dl = (d * sc.astype(np.float32))[:, :, None]
    clear = ((b[:, None, 0:32] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1) ^ 1   # [n, g, l]
    q = _crumbs256(b[:, 32:96]).astype(np.int8) - (clear.reshape(n, 256) << 2).astype(np.int8)
    return (dl * q.reshape(n, 16, 16).astype(np.float32)).reshape(-1)


# the 16-entry non-linear codebook of the IQ4 formats (part of the published format)
IQ4_CODEBOOK = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.int8)


def np_dequant_iq4_nl(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 18)
    d = _f16(b[:, 0:2])[:, None]
    return (d * IQ4_CODEBOOK[_nib32(b[:, 2:18])].astype(np.float32)).reshape(-1)


def np_dequant_iq4_xs(raw: np.ndarray) -> np.ndarray:
    b = raw.reshape(-1, 136)
    n = b.shape[0]
    d = _f16(b[:, 0:2])[:, None]
    sh = np.ascontiguousarray(b[:, 2:4]).view(np.uint16).reshape(n, 1)
    i = np.arange(8)
    lo = (b[:, 4:8][:, i >> 1] >> (4 * (i & 1)).astype(np.uint8)) & 15
    hi = ((sh >> (2 * i).astype(np.uint16)) & 3).astype(np.uint8)
    sc = (lo | (hi << 4)).astype(np.int8) - np.int8(32)
    dl = (d * sc.astype(np.float32))[:, :, None]
    qs = b[:, 8:136].reshape(n, 8, 16)
    idx = np.concatenate([qs & 15, qs >> 4], axis=2)
    return (dl * IQ4_CODEBOOK[idx].astype(np.float32)).reshape(-1)


NP_DEQUANT = {Q2_K: np_dequant_q2_k, Q3_K: np_dequant_q3_k, IQ4_NL: np_dequant_iq4_nl, IQ4_XS: np_dequant_iq4_xs,
              Q4_0: np_dequant_q4_0, Q8_0: np_dequant_q8_0, Q4_K: np_dequant_q4_k, Q6_K: np_dequant_q6_k,
              Q4_1: np_dequant_q4_1, Q5_0: np_dequant_q5_0, Q5_1: np_dequant_q5_1, Q5_K: np_dequant_q5_k}


def np_dequant(qtype: int, blocks: np.ndarray) -> np.ndarray:
    return NP_DEQUANT[qtype](np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1))
