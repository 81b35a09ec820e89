"""Generates tests/golden/q8_0_quant_golden.npz from gguf-py: fp32 rows and the Q8_0 blocks
`gguf.quants.quantize` makes of them, which pins oracle.np_quantize_q8_0 (the rule the Q8_0-style
KV cache follows).

Run in a container that has `gguf` 0.19.0 importable:
    python tests/golden/make_q8_quant_golden.py
Rows: seeded normal values at several magnitudes, rows with ties (values whose quotient by the
block scale ends in .5), an all-zero block, a block with one huge value, subnormal values, and
values whose scale overflows fp16.
"""
import os

import numpy as np
from gguf import quants
from gguf.constants import GGMLQuantizationType as T

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    g = np.random.default_rng(20240607)
    rows = [g.standard_normal(128).astype(np.float32) * np.float32(s) for s in (1.0, 1e-3, 37.5, 1e4)]
    ties = np.zeros(128, dtype=np.float32)
    ties[:32] = np.arange(32, dtype=np.float32) * 0.5            # max 15.5: d = 15.5 / 127
    ties[32:64] = -np.arange(32, dtype=np.float32) * 0.5
    ties[64:96] = 127.0 * np.linspace(-1, 1, 32, dtype=np.float32)
    ties[96:] = (np.arange(32) - 16.5).astype(np.float32) * 63.5 / 15.5
    rows.append(ties)
    edge = np.zeros(128, dtype=np.float32)                        # first block all zero
    edge[32:64] = 1e-3
    edge[40] = 1e6                                                # one value towers over its block
    edge[64:96] = np.float32(1e-41)                               # subnormal fp32 values
    edge[96:] = g.standard_normal(32).astype(np.float32) * np.float32(3e7)   # d overflows fp16 -> inf
    rows.append(edge)
    x = np.stack(rows)
    with np.errstate(all="ignore"):
        blocks = quants.quantize(x, T.Q8_0)                       # [rows, 4 * 34] uint8
    np.savez_compressed(os.path.join(HERE, "q8_0_quant_golden.npz"), x=x, blocks=blocks)
    print("wrote", x.shape, blocks.shape)


if __name__ == "__main__":
    main()
