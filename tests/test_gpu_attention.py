"""K5-K7 parity: KV-cache append / gather (bit-exact copies) and split-K decode attention
against the fp64 textbook oracle, through the C ABI.

Tolerance: fp32 softmax-weighted sums -- |out - ref| <= 1e-5 * sum_t p_t |v_t| per element
(p the oracle's probabilities) and relative L2 <= 1e-5."""
import ctypes

import numpy as np
import pytest

import skainet_b200 as skn
from conftest import FP32_TOL
from oracle import oracle
from skainet_b200 import _ffi, synth

pytestmark = pytest.mark.gpu


def check_attention(out, q, kc, vc, lens, start=None, tol=FP32_TOL):
    ref = oracle.attn_decode(q, kc, vc, lens, start)
    # element-wise bound: sum_t p_t |v_t| <= max_t |v_t| ; use the weighted mean of |v|
    B, Hq, D = q.shape
    Hkv, cap = kc.shape[1], kc.shape[2]
    bound = np.zeros_like(ref)
    for b in range(B):
        L = int(lens[b])
        if L == 0:
            continue
        s0 = 0 if start is None else int(start[b])
        idx = (s0 + np.arange(L)) % cap
        for h in range(Hq):
            kv = h // (Hq // Hkv)
            s = (kc[b, kv, idx].astype(np.float64) @ q[b, h].astype(np.float64)) / np.sqrt(D)
            p = np.exp(s - s.max())
            p /= p.sum()
            bound[b, h] = p @ np.abs(vc[b, kv, idx].astype(np.float64))
    err = np.abs(out.astype(np.float64) - ref)
    assert np.all(err <= tol * bound + 1e-30), f"max excess {np.max(err - tol * bound):.3e}"
    den = np.linalg.norm(ref)
    if den > 0:
        assert np.linalg.norm(out - ref) / den <= tol


@pytest.mark.parametrize("B,Hq,Hkv,D,cap", [(1, 1, 1, 64, 16), (2, 4, 2, 128, 300), (3, 8, 1, 64, 700),
                                            (2, 32, 8, 128, 1100), (2, 8, 8, 128, 513)])
def test_attention_matches_oracle(ctx, B, Hq, Hkv, D, cap):
    g = synth.rng(B * 1000 + Hq + cap)
    kc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    vc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    lens = g.integers(1, cap + 1, size=B).astype(np.int32)
    lens[0] = cap                                    # one full sequence
    q = g.standard_normal((B, Hq, D), dtype=np.float32)
    kv = skn.KVCache(ctx, B, Hkv, D, cap)
    kv.load(kc, vc, lens)
    out = kv.attend(q)
    kv.close()
    check_attention(out, q, kc, vc, lens)


def test_empty_and_single_token_sequences(ctx):
    g = synth.rng(5)
    B, Hq, Hkv, D, cap = 3, 8, 2, 128, 64
    kc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    vc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    lens = np.array([0, 1, 64], dtype=np.int32)
    q = g.standard_normal((B, Hq, D), dtype=np.float32)
    kv = skn.KVCache(ctx, B, Hkv, D, cap)
    kv.load(kc, vc, lens)
    out = kv.attend(q)
    kv.close()
    assert np.all(out[0] == 0)
    # a single cached token: the output is that token's value row, exactly
    for h in range(Hq):
        assert np.allclose(out[1, h], vc[1, h // 4, 0], rtol=1e-6, atol=0)
    check_attention(out, q, kc, vc, lens)


def test_append_gather_and_ring_wrap(ctx):
    """Append past the capacity: the ring overwrites its oldest tokens; gather returns the
    survivors oldest-first, bit for bit; attention sees exactly those tokens."""
    g = synth.rng(6)
    B, Hq, Hkv, D, cap = 2, 4, 2, 64, 20
    kv = skn.KVCache(ctx, B, Hkv, D, cap)
    ks, vs = [], []
    for step in range(27):
        k_new = g.standard_normal((B, Hkv, D), dtype=np.float32)
        v_new = g.standard_normal((B, Hkv, D), dtype=np.float32)
        kv.append(k_new, v_new)
        ks.append(k_new)
        vs.append(v_new)
        lens, start = kv.lengths()
        assert np.all(lens == min(step + 1, cap))
        assert np.all(start == max(0, step + 1 - cap) % cap)
    K = np.stack(ks[-cap:], axis=2)       # [B, Hkv, cap, D], oldest first
    V = np.stack(vs[-cap:], axis=2)
    for b in range(B):
        kg, vg = kv.gather(b, 0, cap)
        assert np.array_equal(kg, K[b]) and np.array_equal(vg, V[b])
        kg, vg = kv.gather(b, 3, 5)
        assert np.array_equal(kg, K[b, :, 3:8]) and np.array_equal(vg, V[b, :, 3:8])
    q = g.standard_normal((B, Hq, D), dtype=np.float32)
    out = kv.attend(q)
    check_attention(out, q, K, V, np.full(B, cap, dtype=np.int32))
    with pytest.raises(ValueError):
        kv.gather(0, 10, 11)
    kv.reset()
    lens, _ = kv.lengths()
    assert np.all(lens == 0)
    kv.close()


def test_cfg4_decode_steps(ctx):
    """Config 4 at reduced step count: 32 query / 8 kv heads, head_dim 128, batch 8, cache
    pre-filled, lengths uniform 1024..4096; each step appends one token and attends."""
    g = synth.rng(3)
    B, Hq, Hkv, D, ctx_len, steps = 8, 32, 8, 128, 4096, 3
    cap = ctx_len + 128
    kc = np.zeros((B, Hkv, cap, D), dtype=np.float32)
    vc = np.zeros((B, Hkv, cap, D), dtype=np.float32)
    kc[:, :, :ctx_len] = g.standard_normal((B, Hkv, ctx_len, D), dtype=np.float32)
    vc[:, :, :ctx_len] = g.standard_normal((B, Hkv, ctx_len, D), dtype=np.float32)
    lens = g.integers(1024, 4097, size=B).astype(np.int32)
    kv = skn.KVCache(ctx, B, Hkv, D, cap)
    kv.load(kc[:, :, :ctx_len], vc[:, :, :ctx_len], lens)
    for _ in range(steps):
        q = g.standard_normal((B, Hq, D), dtype=np.float32)
        k_new = g.standard_normal((B, Hkv, D), dtype=np.float32)
        v_new = g.standard_normal((B, Hkv, D), dtype=np.float32)
        for b in range(B):
            kc[b, :, lens[b]] = k_new[b]
            vc[b, :, lens[b]] = v_new[b]
        lens = lens + 1
        kv.append(k_new, v_new)
        out = kv.attend(q)
        check_attention(out, q, kc, vc, lens)
    kv.close()


def h16(a):
    """What an fp16 cache keeps of fp32 values: round to nearest even, widened back."""
    return a.astype(np.float16).astype(np.float32)


@pytest.mark.parametrize("B,Hq,Hkv,D,cap", [(1, 1, 1, 64, 16), (2, 4, 2, 128, 300), (3, 8, 1, 64, 700),
                                            (2, 32, 8, 128, 1100), (8, 32, 8, 128, 4224)])
def test_fp16_cache_attention_matches_oracle_on_rounded_values(ctx, B, Hq, Hkv, D, cap):
    """An fp16 cache rounds K and V once on their way in; attention over it equals the fp64 oracle over the
    rounded values within the fp32 tolerance (short contexts: per-lane loads; the last case: bulk-copy tiles)."""
    g = synth.rng(B * 1000 + Hq + cap + 7)
    kc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    vc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    lens = g.integers(1, cap + 1, size=B).astype(np.int32)
    lens[0] = cap
    q = g.standard_normal((B, Hq, D), dtype=np.float32)
    kv = skn.KVCache(ctx, B, Hkv, D, cap, dtype="f16")
    kv.load(kc, vc, lens)
    out = kv.attend(q)
    kg, vg = kv.gather(0, 0, min(cap, 40))
    kv.close()
    assert np.array_equal(kg, h16(kc[0, :, :min(cap, 40)])) and np.array_equal(vg, h16(vc[0, :, :min(cap, 40)]))
    check_attention(out, q, h16(kc), h16(vc), lens)


def test_fp16_cache_append_gather_and_ring_wrap(ctx):
    g = synth.rng(16)
    B, Hq, Hkv, D, cap = 2, 8, 2, 128, 20
    kv = skn.KVCache(ctx, B, Hkv, D, cap, dtype="f16")
    ks, vs = [], []
    for step in range(27):
        k_new = g.standard_normal((B, Hkv, D), dtype=np.float32) * 50
        v_new = g.standard_normal((B, Hkv, D), dtype=np.float32) * 1e-3
        kv.append(k_new, v_new)
        ks.append(k_new)
        vs.append(v_new)
    K = h16(np.stack(ks[-cap:], axis=2))
    V = h16(np.stack(vs[-cap:], axis=2))
    for b in range(B):
        kg, vg = kv.gather(b, 0, cap)
        assert np.array_equal(kg, K[b]) and np.array_equal(vg, V[b])
    q = g.standard_normal((B, Hq, D), dtype=np.float32) * 0.02
    out = kv.attend(q)
    check_attention(out, q, K, V, np.full(B, cap, dtype=np.int32))
    kv.close()
    with pytest.raises(ValueError):
        skn.KVCache(ctx, 1, 1, 64, 8, dtype="bf16")
    assert _ffi.lib().skn_kv_create_typed(ctx.handle, 1, 1, 64, 8, 3, ctypes.byref(ctypes.c_void_p())) == 2   # SKN_ERR_TYPE


def q8(a):
    """What a Q8_0-style cache keeps of fp32 values: per 32 head dims d = max|x| / 127 (kept as fp16) and
    int8 q = round(x / d); read back as q * d (oracle.np_quantize_q8_0, pinned to gguf-py)."""
    return oracle.np_q8_0_roundtrip(a)


@pytest.mark.parametrize("D", [128, 64])
def test_q8_0_cache_load_append_gather_and_ring_wrap(ctx, D):
    """Every way into a Q8_0 cache (pre-fill, single-token append, the ring's overwrite) quantises with the pinned
    rule bit for bit: what gather returns equals the oracle's round trip of what went in, magnitudes from 1e-3
    to 50, an all-zero block and exact ties included; attention over it equals the fp64 oracle over those values."""
    g = synth.rng(61 + D)
    B, Hq, Hkv, cap = 2, 8, 2, 20
    kv = skn.KVCache(ctx, B, Hkv, D, cap, dtype="q8_0")
    k0 = g.standard_normal((B, Hkv, 5, D), dtype=np.float32) * 3
    v0 = g.standard_normal((B, Hkv, 5, D), dtype=np.float32) * 1e-3
    k0[0, 0, 1, :32] = 0.0                                         # an all-zero block: scale 0, quants 0
    k0[1, 1, 2, 32:64] = (np.arange(32) - 16) * 0.5                # ties: x / d ends in .5 for odd multiples
    k0[1, 1, 2, 63] = 63.5
    kv.load(k0, v0, np.full(B, 5, dtype=np.int32))
    ks = [k0[:, :, i] for i in range(5)]
    vs = [v0[:, :, i] for i in range(5)]
    for step in range(22):
        k_new = g.standard_normal((B, Hkv, D), dtype=np.float32) * 50
        v_new = g.standard_normal((B, Hkv, D), dtype=np.float32) * (1e-3 if step % 2 else 7.0)
        kv.append(k_new, v_new)
        ks.append(k_new)
        vs.append(v_new)
    K = q8(np.stack(ks[-cap:], axis=2))
    V = q8(np.stack(vs[-cap:], axis=2))
    lens, start = kv.lengths()
    assert np.all(lens == cap) and np.all(start == (5 + 22 - cap))
    for b in range(B):
        kg, vg = kv.gather(b, 0, cap)
        assert np.array_equal(kg.view(np.uint32), K[b].view(np.uint32)) and np.array_equal(vg.view(np.uint32), V[b].view(np.uint32))
    qv = g.standard_normal((B, Hq, D), dtype=np.float32) * 0.02
    out = kv.attend(qv)
    check_attention(out, qv, K, V, np.full(B, cap, dtype=np.int32))
    kv.close()


@pytest.mark.parametrize("B,Hq,Hkv,D,cap", [(1, 1, 1, 64, 16), (2, 4, 2, 128, 300), (3, 8, 1, 64, 700),
                                            (2, 32, 8, 128, 1100), (8, 32, 8, 128, 4224)])
def test_q8_0_cache_attention_matches_oracle_on_quantised_values(ctx, B, Hq, Hkv, D, cap):
    """Attention over a Q8_0 cache equals the fp64 oracle over the quantised-and-restored K and V within the fp32
    tolerance, from a 16-token context to 4224 tokens (every split size, the in-kernel merge and the merge launch)."""
    g = synth.rng(B * 1000 + Hq + cap + 11)
    kc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    vc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    lens = g.integers(1, cap + 1, size=B).astype(np.int32)
    lens[0] = cap
    qv = g.standard_normal((B, Hq, D), dtype=np.float32)
    kv = skn.KVCache(ctx, B, Hkv, D, cap, dtype="q8_0")
    kv.load(kc, vc, lens)
    out = kv.attend(qv)
    kv.close()
    check_attention(out, qv, q8(kc), q8(vc), lens)
    # and the quantisation itself costs what Q8_0 costs: about half a percent of the exact result
    exact = oracle.attn_decode(qv, kc, vc, lens)
    rel = np.linalg.norm(out.astype(np.float64) - exact) / np.linalg.norm(exact)
    assert rel < 2e-2, rel


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_wrapped_ring_in_the_bulk_copy_regime(ctx, dtype):
    """A full cache that has wrapped (start = 37, not a tile boundary) at a size where the 256-token splits run
    on bulk-copied tiles: the tile that straddles the end of the ring arrives as two copies."""
    g = synth.rng(41)
    B, Hq, Hkv, D, cap, extra = 8, 32, 8, 128, 1280, 37
    kc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    vc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
    kv = skn.KVCache(ctx, B, Hkv, D, cap, dtype=dtype)
    kv.load(kc, vc, np.full(B, cap, dtype=np.int32))
    for i in range(extra):
        k_new = g.standard_normal((B, Hkv, D), dtype=np.float32)
        v_new = g.standard_normal((B, Hkv, D), dtype=np.float32)
        kc[:, :, i] = k_new                      # a full ring overwrites its oldest slot
        vc[:, :, i] = v_new
        kv.append(k_new, v_new)
    lens, start = kv.lengths()
    assert np.all(lens == cap) and np.all(start == extra)
    q = g.standard_normal((B, Hq, D), dtype=np.float32)
    out = kv.attend(q)
    kv.close()
    if dtype == "f16":
        kc, vc = h16(kc), h16(vc)
    check_attention(out, q, kc, vc, lens, start)


def test_attention_argument_errors(ctx):
    kv = skn.KVCache(ctx, 1, 2, 64, 8)
    with pytest.raises(ValueError, match="Shapes do not align."):
        kv.attend(np.zeros((1, 3, 64), dtype=np.float32))       # 3 query heads over 2 kv heads
    with pytest.raises(ValueError):
        kv.load(np.zeros((1, 2, 9, 64), np.float32), np.zeros((1, 2, 9, 64), np.float32), [9])  # > capacity
    kv.close()
    with pytest.raises(ValueError):
        skn.KVCache(ctx, 1, 2, 80, 8)                           # unsupported head_dim
