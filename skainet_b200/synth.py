"""Seeded synthetic GGUF blocks and activations with the value distributions of the
benchmark configurations (no model file or dataset is involved anywhere).

Draw order per tensor is fixed: d -> dmin (if the type has one) -> scale bytes ->
quant bytes; activations are drawn after the weights from the same generator.
Block geometry follows gguf/src/commonMain/kotlin/sk/ai/net/gguf/Constants.kt:58-90.
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0, Q4_K, Q6_K = 2, 8, 12, 14
Q4_1, Q5_0, Q5_1, Q5_K = 3, 6, 7, 13
Q2_K, Q3_K, IQ4_NL, IQ4_XS = 10, 11, 20, 23
GEOMETRY = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210),
            Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q5_K: (256, 176),
            Q2_K: (256, 84), Q3_K: (256, 110), IQ4_NL: (32, 18), IQ4_XS: (256, 136)}
# the four types of the benchmark configurations (streaming / tensor-core kernels) ...
TYPE_NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q6_K: "Q6_K"}
# ... and the further block types served by the dequantiser and the generic dequant-dot
EXTRA_TYPE_NAMES = {Q4_1: "Q4_1", Q5_0: "Q5_0", Q5_1: "Q5_1", Q5_K: "Q5_K",
                    Q2_K: "Q2_K", Q3_K: "Q3_K", IQ4_NL: "IQ4_NL", IQ4_XS: "IQ4_XS"}
ALL_TYPE_NAMES = {**TYPE_NAMES, **EXTRA_TYPE_NAMES}


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def _half_abs_normal(g: np.random.Generator, n: int, sigma: float) -> np.ndarray:
    return np.abs(g.normal(0.0, sigma, size=n)).astype(np.float16).view(np.uint8).reshape(n, 2)


def make_blocks(g: np.random.Generator, qtype: int, n_blocks: int) -> np.ndarray:
    """n_blocks raw blocks as uint8 [n_blocks, block_bytes]."""
    _, bb = GEOMETRY[qtype]
    out = np.empty((n_blocks, bb), dtype=np.uint8)
    if qtype == Q4_0:
        out[:, 0:2] = _half_abs_normal(g, n_blocks, 0.01)
        out[:, 2:18] = g.integers(0, 256, size=(n_blocks, 16), dtype=np.uint8)
    elif qtype == Q8_0:
        out[:, 0:2] = _half_abs_normal(g, n_blocks, 0.01)
        out[:, 2:34] = g.integers(-127, 128, size=(n_blocks, 32), dtype=np.int8).view(np.uint8)
    elif qtype == Q4_K:
        out[:, 0:2] = _half_abs_normal(g, n_blocks, 0.01)
        out[:, 2:4] = _half_abs_normal(g, n_blocks, 0.005)
        # uniform bytes make every unpacked 6-bit scale / min uniform on 0..63
        out[:, 4:16] = g.integers(0, 256, size=(n_blocks, 12), dtype=np.uint8)
        out[:, 16:144] = g.integers(0, 256, size=(n_blocks, 128), dtype=np.uint8)
    elif qtype == Q6_K:
        d = _half_abs_normal(g, n_blocks, 0.01)
        sc = g.integers(-32, 32, size=(n_blocks, 16), dtype=np.int8).view(np.uint8)
        out[:, 0:192] = g.integers(0, 256, size=(n_blocks, 192), dtype=np.uint8)
        out[:, 192:208] = sc
        out[:, 208:210] = d
    elif qtype in (Q4_1, Q5_0, Q5_1):
        # fp16 scale (and min) as for Q4_0, every other byte uniform
        out[:, :] = g.integers(0, 256, size=(n_blocks, bb), dtype=np.uint8)
        out[:, 0:2] = _half_abs_normal(g, n_blocks, 0.01)
        if qtype != Q5_0:
            out[:, 2:4] = _half_abs_normal(g, n_blocks, 0.005)
    elif qtype == Q5_K:
        out[:, 0:2] = _half_abs_normal(g, n_blocks, 0.01)
        out[:, 2:4] = _half_abs_normal(g, n_blocks, 0.005)
        out[:, 4:176] = g.integers(0, 256, size=(n_blocks, 172), dtype=np.uint8)
    elif qtype in (Q2_K, Q3_K, IQ4_NL, IQ4_XS):
        # fp16 super-block scale(s) where the format keeps them, every other byte uniform
        out[:, :] = g.integers(0, 256, size=(n_blocks, bb), dtype=np.uint8)
        if qtype == Q2_K:
            out[:, 80:82] = _half_abs_normal(g, n_blocks, 0.01)
            out[:, 82:84] = _half_abs_normal(g, n_blocks, 0.005)
        elif qtype == Q3_K:
            out[:, 108:110] = _half_abs_normal(g, n_blocks, 0.01)
        else:
            out[:, 0:2] = _half_abs_normal(g, n_blocks, 0.0003 if qtype == IQ4_XS else 0.001)
    else:
        raise ValueError(f"unsupported type {qtype}")
    return out


def make_weight(g: np.random.Generator, qtype: int, n_rows: int, n_cols: int) -> np.ndarray:
    """Raw blocks of a [n_rows, n_cols] weight, uint8 [n_rows, row_bytes]."""
    e, bb = GEOMETRY[qtype]
    if n_cols % e:
        raise ValueError("n_cols must be a multiple of the block size")
    nb = n_cols // e
    return make_blocks(g, qtype, n_rows * nb).reshape(n_rows, nb * bb)


def make_activations(g: np.random.Generator, m: int, k: int) -> np.ndarray:
    return g.standard_normal(size=(m, k), dtype=np.float32)


def cfg1(seed: int = 0):
    """Q4_K 4096x4096 weight and a length-4096 fp32 vector."""
    g = rng(seed)
    w = make_weight(g, Q4_K, 4096, 4096)
    x = make_activations(g, 1, 4096)
    return w, x
