"""Configurations 3 and 5 at their own widths (14336-wide FFN, d_model 4096, vocabulary 32000), where the
intermediates reach 1e6 and the kernels take the tile shapes and launch geometries of the real sizes.  The GPU
computes everything; the fp64 oracle runs on sampled rows / columns and straight from the raw blocks, so the
CPU side stays within seconds.  Neither configuration has a reference oracle (the reference has no SwiGLU, RMSNorm,
RoPE or attention): the restatement is the textbook definition over the pinned dequantiser."""
import numpy as np
import pytest

import skainet_b200 as skn
from conftest import BF16_TOL
from oracle import oracle
from skainet_b200 import synth
from skainet_b200.llama import LlamaConfig, LlamaDecoder

pytestmark = pytest.mark.gpu


def test_cfg3_ffn_prefill_at_full_size(ctx):
    """Config 3: X fp32 [512, 4096], W_gate / W_up 14336 x 4096 Q4_K, W_down 4096 x 14336 Q6_K on the tensor cores
    (bf16 operands, the intermediate kept in bf16).  Oracle: 48 sampled token rows x 96 sampled output columns."""
    M, K, F = 512, 4096, 14336
    g = synth.rng(2)
    x = synth.make_activations(g, M, K)
    wg = synth.make_weight(g, synth.Q4_K, F, K)
    wu = synth.make_weight(g, synth.Q4_K, F, K)
    wd = synth.make_weight(g, synth.Q6_K, K, F)
    tg, tu, td = (skn.QuantTensor(ctx, s, q, w) for s, q, w in (((F, K), synth.Q4_K, wg), ((F, K), synth.Q4_K, wu),
                                                                 ((K, F), synth.Q6_K, wd)))
    y = skn.ffn_swiglu(ctx, tg, tu, td, x)
    for t in (tg, tu, td):
        t.close()
    assert y.shape == (M, K) and np.isfinite(y).all()
    rows = np.sort(g.choice(M, size=48, replace=False))
    cols = np.sort(g.choice(K, size=96, replace=False))
    gate, _ = oracle.matmul(synth.Q4_K, wg, F, K, x[rows])
    up, _ = oracle.matmul(synth.Q4_K, wu, F, K, x[rows])
    h = gate / (1.0 + np.exp(-gate)) * up                                    # fp64 [48, F]
    assert np.abs(h).max() > 1e4                                             # the range fp16 could not hold
    wd_rows = oracle.dequant(synth.Q6_K, np.ascontiguousarray(wd[cols])).reshape(cols.size, F).astype(np.float64)
    ref = h @ wd_rows.T                                                      # [48, 96]
    absdot = np.abs(h) @ np.abs(wd_rows).T
    got = y[np.ix_(rows, cols)].astype(np.float64)
    err = np.abs(got - ref)
    assert np.all(err <= BF16_TOL * absdot), f"worst element error / sum|h w| = {np.max(err / absdot):.3e}"
    assert np.linalg.norm(got - ref) <= BF16_TOL * np.linalg.norm(ref)


class RawRef:
    """fp64 decoder over the raw blocks: every product is oracle.matmul (fused dequant-dot, fp64 accumulation),
    so no dequantised copy of a full-width model is ever held."""

    def __init__(self, cfg, layers, head):
        self.cfg, self.layers, self.head = cfg, layers, head
        self.k = [None] * cfg.n_layers
        self.v = [None] * cfg.n_layers
        self.pos = 0

    def mm(self, qt, w, n, k, x):
        # (the oracle takes fp32 activations, as the library does: the fp64 stream is rounded once per product)
        return oracle.matmul(qt, w, n, k, np.asarray(x, dtype=np.float32))[0]

    def rms(self, x):
        return x / np.sqrt((x * x).mean(-1, keepdims=True) + self.cfg.rms_eps)

    def rope(self, x, pos0):
        B, T, H, D = x.shape
        p = np.arange(D // 2)
        ang = (pos0 + np.arange(T))[:, None] * self.cfg.rope_theta ** (-2.0 * p / D)[None, :]
        c, s = np.cos(ang)[None, :, None, :], np.sin(ang)[None, :, None, :]
        a, b = x[..., 0::2], x[..., 1::2]
        y = np.empty_like(x)
        y[..., 0::2] = a * c - b * s
        y[..., 1::2] = a * s + b * c
        return y

    def forward(self, tokens):
        c = self.cfg
        B, T = tokens.shape
        qd, kd = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
        rb = oracle.row_bytes(c.head_type, c.d_model)
        emb = self.head[0].reshape(c.vocab, rb)
        x = oracle.dequant(c.head_type, np.ascontiguousarray(emb[tokens.reshape(-1)])).reshape(B, T, c.d_model).astype(np.float64)
        for li, l in enumerate(self.layers):
            h = self.rms(x).reshape(B * T, c.d_model)
            q = self.mm(c.proj_type, l["wq"], qd, c.d_model, h).reshape(B, T, c.n_heads, c.head_dim)
            k = self.mm(c.proj_type, l["wk"], kd, c.d_model, h).reshape(B, T, c.n_kv_heads, c.head_dim)
            v = self.mm(c.proj_type, l["wv"], kd, c.d_model, h).reshape(B, T, c.n_kv_heads, c.head_dim)
            q, k = self.rope(q, self.pos), self.rope(k, self.pos)
            kk, vv = k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3)
            self.k[li] = kk if self.k[li] is None else np.concatenate([self.k[li], kk], axis=2)
            self.v[li] = vv if self.v[li] is None else np.concatenate([self.v[li], vv], axis=2)
            att = np.zeros((B, T, c.n_heads, c.head_dim))
            grp = c.n_heads // c.n_kv_heads
            for b in range(B):
                for t in range(T):
                    L = self.pos + t + 1
                    for hh in range(c.n_heads):
                        K, V = self.k[li][b, hh // grp, :L], self.v[li][b, hh // grp, :L]
                        s = K @ q[b, t, hh] / np.sqrt(c.head_dim)
                        p = np.exp(s - s.max())
                        att[b, t, hh] = (p / p.sum()) @ V
            x = x + self.mm(c.proj_type, l["wo"], c.d_model, qd, att.reshape(B * T, qd)).reshape(B, T, c.d_model)
            h = self.rms(x).reshape(B * T, c.d_model)
            gt = self.mm(c.proj_type, l["w_gate"], c.ffn_dim, c.d_model, h)
            up = self.mm(c.proj_type, l["w_up"], c.ffn_dim, c.d_model, h)
            with np.errstate(over="ignore"):
                act = gt / (1.0 + np.exp(-gt)) * up
            x = x + self.mm(c.proj_type, l["w_down"], c.d_model, c.ffn_dim, act).reshape(B, T, c.d_model)
        self.pos += T
        last = self.rms(x[:, -1])
        return self.mm(c.head_type, self.head[1], c.vocab, c.d_model, last)


def _full_width_model(n_layers, seed):
    cfg = LlamaConfig(n_layers=n_layers)
    g = synth.rng(seed)
    qd, kd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    shapes = {"wq": (qd, cfg.d_model), "wk": (kd, cfg.d_model), "wv": (kd, cfg.d_model), "wo": (cfg.d_model, qd),
              "w_gate": (cfg.ffn_dim, cfg.d_model), "w_up": (cfg.ffn_dim, cfg.d_model), "w_down": (cfg.d_model, cfg.ffn_dim)}
    layers = [{k: synth.make_weight(g, cfg.proj_type, *shp) for k, shp in shapes.items()} for _ in range(n_layers)]
    head = (synth.make_weight(g, cfg.head_type, cfg.vocab, cfg.d_model), synth.make_weight(g, cfg.head_type, cfg.vocab, cfg.d_model))
    return cfg, layers, head


def _rel(a, b):
    return np.linalg.norm(np.asarray(a, dtype=np.float64) - b) / np.linalg.norm(b)


def test_cfg5_full_width_decoder_first_tokens(ctx):
    """Config 5's widths (d_model 4096, FFN 14336, 32 / 8 heads of 128, vocabulary 32000, Q4_K projections, Q6_K
    embedding and LM head) on two layers: an 8-token prompt through the fp32 many-row path, then eight greedy
    steps, batch 1; every step's logits against the fp64 restatement over the raw blocks, and the same tokens."""
    cfg, layers, head = _full_width_model(2, seed=4)
    B, T = 1, 8
    dec = LlamaDecoder(ctx, cfg, batch=B, max_tokens=T, max_ctx=32)
    ones = np.ones(cfg.d_model, dtype=np.float32)
    for i, l in enumerate(layers):
        dec.set_layer(i, l, ones, ones)
    dec.set_head(head[0], ones, head[1])
    ref = RawRef(cfg, layers, head)
    prompt = synth.rng(41).integers(0, cfg.vocab, size=(B, T)).astype(np.int32)
    nxt, logits = dec.forward(prompt, want_logits=True)
    want = ref.forward(prompt)
    assert _rel(logits, want) <= 2e-4
    assert np.array_equal(nxt, want.argmax(-1))
    for step in range(8):
        fed = nxt.copy()
        nxt, logits = dec.forward(None, want_logits=True)          # the ids are fed back on the device
        want = ref.forward(fed[:, None])
        assert _rel(logits, want) <= 2e-4, step
        assert np.array_equal(nxt, want.argmax(-1)), step
    dec.close()


def test_cfg5_full_width_layer_at_batch_16(ctx):
    """One full-width layer with fresh inputs at batch 16: sixteen different single-token sequences, then two
    decode steps (sixteen activation rows per product: every weight is streamed once), against the restatement."""
    cfg, layers, head = _full_width_model(1, seed=5)
    B = 16
    dec = LlamaDecoder(ctx, cfg, batch=B, max_tokens=1, max_ctx=8)
    ones = np.ones(cfg.d_model, dtype=np.float32)
    dec.set_layer(0, layers[0], ones, ones)
    dec.set_head(head[0], ones, head[1])
    ref = RawRef(cfg, layers, head)
    g = synth.rng(43)
    for step in range(3):
        tok = g.integers(0, cfg.vocab, size=(B, 1)).astype(np.int32)
        nxt, logits = dec.forward(tok, want_logits=True)
        want = ref.forward(tok)
        assert _rel(logits, want) <= 2e-4, step
        assert np.array_equal(nxt, want.argmax(-1)), step
    dec.close()
