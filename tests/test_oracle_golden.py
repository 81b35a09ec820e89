"""The oracle against the committed golden vectors (gguf-py 0.19.0 outputs) -- CPU only."""
import numpy as np
import pytest

from oracle import oracle
from skainet_b200 import synth

TYPES = list(synth.ALL_TYPE_NAMES.items())


@pytest.mark.parametrize("qt,name", TYPES)
def test_c_oracle_matches_golden_bit_exact(golden, qt, name):
    blocks, vals = golden[f"{name}_blocks"], golden[f"{name}_values"].reshape(-1)
    got = oracle.dequant(qt, blocks)
    assert np.array_equal(got.view(np.uint32), vals.view(np.uint32))


@pytest.mark.parametrize("qt,name", TYPES)
def test_numpy_oracle_matches_golden_bit_exact(golden, qt, name):
    blocks, vals = golden[f"{name}_blocks"], golden[f"{name}_values"].reshape(-1)
    got = oracle.np_dequant(qt, blocks)
    assert np.array_equal(got.view(np.uint32), vals.view(np.uint32))


@pytest.mark.parametrize("qt,name", TYPES)
def test_two_restatements_agree_on_fresh_blocks(qt, name):
    blocks = synth.make_blocks(synth.rng(11), qt, 512)
    assert np.array_equal(oracle.dequant(qt, blocks).view(np.uint32), oracle.np_dequant(qt, blocks).view(np.uint32))


def test_geometry_table():
    # Constants.kt:58-90
    assert oracle.GEOMETRY == {2: (32, 18), 8: (32, 34), 12: (256, 144), 14: (256, 210),
                               3: (32, 20), 6: (32, 22), 7: (32, 24), 13: (256, 176),
                               10: (256, 84), 11: (256, 110), 20: (32, 18), 23: (256, 136)}
    assert oracle.row_bytes(12, 4096) == 2304
    assert oracle.row_bytes(14, 14336) == 11760
    with pytest.raises(ValueError):
        oracle.row_bytes(12, 4000)      # Quants.kt:12-16


@pytest.mark.parametrize("qt,name", TYPES)
def test_matmul_matches_numpy_fp64(qt, name):
    g = synth.rng(5)
    N, K, M = 24, 512, 3
    w = synth.make_weight(g, qt, N, K)
    x = synth.make_activations(g, M, K)
    y, absdot = oracle.matmul(qt, w, N, K, x, threads=2)
    W = oracle.dequant(qt, w).reshape(N, K).astype(np.float64)
    ref = x.astype(np.float64) @ W.T
    assert np.allclose(y, ref, rtol=1e-12, atol=1e-12)
    assert np.allclose(absdot, np.abs(x.astype(np.float64))[:, None, :] .__mul__(np.abs(W)[None]).sum(-1), rtol=1e-12)


@pytest.mark.parametrize("M", [1, 2])
def test_reference_loop_order_equals_fused_order(M):
    """Linear.forward restated literally (transposed copy, reference loop nests) gives the
    same fp64 bits as the row-wise fused form used as the parity oracle."""
    g = synth.rng(6)
    N, K = 16, 256
    w = synth.make_weight(g, synth.Q4_K, N, K)
    x = synth.make_activations(g, M, K)
    bias = g.standard_normal(N).astype(np.float32)
    y_ref = oracle.linear_ref(synth.Q4_K, w, N, K, x, bias)
    y, _ = oracle.matmul(synth.Q4_K, w, N, K, x)
    assert np.array_equal(y_ref, y + bias.astype(np.float64)[None, :])


def test_attention_oracle_against_numpy():
    g = synth.rng(7)
    B, Hq, Hkv, D, cap = 2, 4, 2, 16, 12
    q = g.standard_normal((B, Hq, D), dtype=np.float32)
    kc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    vc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    lens = np.array([5, 12], dtype=np.int32)
    out = oracle.attn_decode(q, kc, vc, lens)
    for b in range(B):
        for h in range(Hq):
            kv = h // (Hq // Hkv)
            s = (kc[b, kv, :lens[b]].astype(np.float64) @ q[b, h].astype(np.float64)) / np.sqrt(D)
            p = np.exp(s - s.max())
            p /= p.sum()
            ref = p @ vc[b, kv, :lens[b]].astype(np.float64)
            assert np.allclose(out[b, h], ref, rtol=1e-12, atol=1e-14)


def test_ffn_oracle_against_numpy():
    g = synth.rng(8)
    F, K, N, M = 512, 256, 32, 3
    wg = synth.make_weight(g, synth.Q4_K, F, K)
    wu = synth.make_weight(g, synth.Q4_K, F, K)
    wd = synth.make_weight(g, synth.Q6_K, N, F)
    x = synth.make_activations(g, M, K)
    y = oracle.ffn_swiglu(synth.Q4_K, wg, wu, synth.Q6_K, wd, F, K, N, x)
    Wg = oracle.dequant(synth.Q4_K, wg).reshape(F, K).astype(np.float64)
    Wu = oracle.dequant(synth.Q4_K, wu).reshape(F, K).astype(np.float64)
    Wd = oracle.dequant(synth.Q6_K, wd).reshape(N, F).astype(np.float64)
    a = x.astype(np.float64) @ Wg.T
    h = a / (1 + np.exp(-a)) * (x.astype(np.float64) @ Wu.T)
    assert np.allclose(y, h @ Wd.T, rtol=1e-10, atol=1e-10)


def test_q8_0_quantiser_matches_gguf_py_bit_exact():
    """oracle.np_quantize_q8_0 (the rule of the Q8_0-style KV cache) against blocks gguf-py 0.19.0 made of the
    same rows (tests/golden/make_q8_quant_golden.py): scales and quants bit for bit, ties, an all-zero block, a
    towering value, subnormals and an fp16-overflowing scale included; and the round trip equals the
    pinned Q8_0 dequantiser on those blocks."""
    import os
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "q8_0_quant_golden.npz"))
    x, blocks = z["x"], z["blocks"].reshape(z["x"].shape[0], -1, 34)
    q, dh = oracle.np_quantize_q8_0(x)
    assert np.array_equal(dh.view(np.uint16), np.ascontiguousarray(blocks[:, :, :2]).view(np.uint16).reshape(dh.shape))
    assert np.array_equal(q.reshape(x.shape[0], -1, 32).view(np.uint8), blocks[:, :, 2:])
    finite = np.isfinite(dh.astype(np.float32)).repeat(32, axis=-1).reshape(x.shape)
    rt = oracle.np_q8_0_roundtrip(x)
    want = oracle.dequant(synth.Q8_0, np.ascontiguousarray(z["blocks"]).reshape(-1)).reshape(x.shape)
    assert np.array_equal(rt[finite].view(np.uint32), want[finite].view(np.uint32))
