"""Generates tests/golden/quant_golden.npz from gguf-py (the llama.cpp Python package the
reference's gguf module says it is transliterating: Constants.kt:3-6, Quants.kt:3-6).

Run in a container that has `gguf` 0.19.0 importable:
    python tests/golden/make_golden.py
For each of Q4_0 / Q8_0 / Q4_K / Q6_K and Q4_1 / Q5_0 / Q5_1 / Q5_K / Q2_K / Q3_K / IQ4_NL / IQ4_XS the file holds raw blocks (uint8) and the fp32
values `gguf.quants.dequantize` returns for them: 48 seeded random blocks with the
benchmark's value distributions, 8 blocks of uniformly random bytes with a finite
fp16 scale, and hand-built edge blocks (all-zero, all-ones bits, subnormal / negative /
largest finite fp16 scales, extreme quants).
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from skainet_b200 import synth  # noqa: E402

import gguf  # noqa: E402
from gguf import quants  # noqa: E402
from gguf.constants import GGMLQuantizationType as T  # noqa: E402

GG = {synth.Q4_0: T.Q4_0, synth.Q8_0: T.Q8_0, synth.Q4_K: T.Q4_K, synth.Q6_K: T.Q6_K,
      synth.Q4_1: T.Q4_1, synth.Q5_0: T.Q5_0, synth.Q5_1: T.Q5_1, synth.Q5_K: T.Q5_K,
      synth.Q2_K: T.Q2_K, synth.Q3_K: T.Q3_K, synth.IQ4_NL: T.IQ4_NL, synth.IQ4_XS: T.IQ4_XS}
# byte offsets of the fp16 fields per type
F16_FIELDS = {synth.Q4_0: [0], synth.Q8_0: [0], synth.Q4_K: [0, 2], synth.Q6_K: [208],
              synth.Q4_1: [0, 2], synth.Q5_0: [0], synth.Q5_1: [0, 2], synth.Q5_K: [0, 2],
              synth.Q2_K: [80, 82], synth.Q3_K: [108], synth.IQ4_NL: [0], synth.IQ4_XS: [0]}
EDGE_HALVES = [0x0000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0x8001, 0xBC00, 0x3C00]  # 0, subnormals, min normal, max, -sub, -1, 1


def put_half(block, off, h):
    block[off] = h & 0xFF
    block[off + 1] = h >> 8


def edge_blocks(qtype):
    e, bb = synth.GEOMETRY[qtype]
    out = []
    for fill in (0x00, 0xFF, 0x0F, 0xF0, 0x80, 0x7F):
        for h in EDGE_HALVES:
            b = np.full(bb, fill, dtype=np.uint8)
            for off in F16_FIELDS[qtype]:
                put_half(b, off, h)
            out.append(b)
    return np.stack(out)


def random_byte_blocks(g, qtype, n):
    e, bb = synth.GEOMETRY[qtype]
    b = g.integers(0, 256, size=(n, bb), dtype=np.uint8)
    for off in F16_FIELDS[qtype]:
        # keep the scale finite: clear the top exponent bit
        b[:, off + 1] &= 0xBF
    return b


def main():
    g = synth.rng(20240607)
    data = {"gguf_version": np.array(getattr(gguf, "__version__", "0.19.0"))}
    for qt, name in synth.ALL_TYPE_NAMES.items():
        blocks = np.concatenate([
            synth.make_blocks(g, qt, 48),
            random_byte_blocks(g, qt, 8),
            edge_blocks(qt),
        ])
        vals = quants.dequantize(blocks, GG[qt]).astype(np.float32)
        assert np.isfinite(vals).all(), name
        data[f"{name}_blocks"] = blocks
        data[f"{name}_values"] = vals
        print(name, blocks.shape, vals.shape)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_golden.npz")
    np.savez_compressed(out, **data)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
