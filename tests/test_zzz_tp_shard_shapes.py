"""Decoder shapes that only a tensor-parallel shard has: few rows per projection against many activation rows.

Collected after every other file on purpose: these shapes were first run on eight GPUs (the gate / up shard of
the 32-layer decoder has 224 sixteen-row groups for 148 CTAs), where a CTA that was left without any group
after the SwiGLU form's rounding to whole gate / up pairs kept its plane producer waiting until the bounded
wait ran out -- two seconds per launch.  One GPU shows the same with a decoder of the shard's own sizes.
"""
import time

import numpy as np
import pytest

from skainet_b200 import synth
from skainet_b200.llama import LlamaConfig, LlamaDecoder, random_model_blocks
from test_gpu_llama import RefModel, rel

pytestmark = pytest.mark.gpu


def test_gate_up_shard_with_fewer_than_two_groups_per_cta(ctx):
    """One layer with the FFN width of an 8-way shard (1792 rows each for gate and up: 224 groups, fewer than two
    per CTA) and K = 3072 (three K chunks, so the plane producer does have to wait for the compute warps), five
    sequences per step: the many-row kernel in its SwiGLU form.  Logits against the fp64 restatement, and no step
    anywhere near the two seconds a run-out wait costs."""
    cfg = LlamaConfig(n_layers=1, d_model=3072, n_heads=24, n_kv_heads=6, head_dim=128, ffn_dim=1792, vocab=512)
    layers, head = random_model_blocks(cfg, seed=14)
    B = 5
    dec = LlamaDecoder(ctx, cfg, batch=B, max_tokens=1, max_ctx=8)
    ones = np.ones(cfg.d_model, dtype=np.float32)
    dec.set_layer(0, layers[0], ones, ones)
    dec.set_head(head[0], ones, head[1])
    ref = RefModel(cfg, layers, head)
    g = synth.rng(44)
    for step in range(3):
        tok = g.integers(0, cfg.vocab, size=(B, 1)).astype(np.int32)
        t0 = time.perf_counter()
        nxt, logits = dec.forward(tok, want_logits=True)          # raises SKN_ERR_TIMEOUT if a bounded wait ran out
        took = time.perf_counter() - t0
        want = ref.forward(tok)
        assert rel(logits, want) <= 2e-4, step
        assert np.array_equal(nxt, want.argmax(-1)), step
        assert step == 0 or took < 1.0, f"step {step} took {took:.2f} s"
    dec.close()
