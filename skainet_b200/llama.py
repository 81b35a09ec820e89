"""Host-side mirror of the decoder entry points (skn_llama_*): a Llama-style model whose
weights are quantized tensors resident in HBM.  Built in the style of the reference's
Module / ModuleParameters classes (core/src/commonMain/kotlin/sk/ai/net/nn/Module.kt:6-16);
the reference itself has no decoder."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import _ffi, synth
from .tensor import Context, QuantTensor, _check, _raise, SKN_OK


@dataclass
class LlamaConfig:
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn_dim: int = 14336
    vocab: int = 32000
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5
    proj_type: int = synth.Q4_K      # the seven projections of every layer
    head_type: int = synth.Q6_K      # token embedding and LM head


class LlamaDecoder:
    """Owns the quantized weights (uploaded from raw blocks) and the native decoder."""

    def __init__(self, ctx: Context, cfg: LlamaConfig, batch: int, max_tokens: int, max_ctx: int, exchange=None,
                 kv_dtype: str = "f32"):
        """exchange (parallel.Exchange): tensor-parallel decoder; this rank then keeps only its
        share of every weight (set_layer / set_head still take the WHOLE tensors' raw blocks and
        upload the rank's shard).  kv_dtype "f16" / "q8_0" keeps the layers' KV caches in fp16 / Q8_0-style blocks."""
        if kv_dtype not in ("f32", "f16", "q8_0"):
            raise ValueError("kv_dtype must be 'f32', 'f16' or 'q8_0'")
        self.ctx, self.cfg, self.batch = ctx, cfg, batch
        self.kv_dtype = kv_dtype
        ctx.set_kv_dtype(kv_dtype)
        self._h = ctypes.c_void_p()
        self._tensors = []
        self.exchange = exchange
        self.world = exchange.world if exchange is not None else 1
        self.rank = exchange.rank if exchange is not None else 0
        rc = _ffi.lib().skn_llama_create_tp(ctx.handle, cfg.n_layers, cfg.d_model, cfg.n_heads, cfg.n_kv_heads,
                                            cfg.head_dim, cfg.ffn_dim, cfg.vocab, cfg.rope_theta, cfg.rms_eps, batch,
                                            max_tokens, max_ctx, None if exchange is None else exchange.handle,
                                            ctypes.byref(self._h))
        ctx.set_kv_dtype("f32")
        if rc != SKN_OK:
            self._h = ctypes.c_void_p()
            _raise(ctx.handle, rc)

    @property
    def handle(self):
        return self._h

    def _up(self, qtype, shape, blocks, split=None) -> QuantTensor:
        """split: None (whole tensor), "rows" (this rank's contiguous range of output rows) or
        "cols" (its range of input columns, in whole blocks)."""
        shard = None
        if self.world > 1 and split == "rows":
            shard = (self.rank * (shape[0] // self.world), shape[0] // self.world, 0, shape[1])
        elif self.world > 1 and split == "cols":
            shard = (0, shape[0], self.rank * (shape[1] // self.world), shape[1] // self.world)
        t = QuantTensor(self.ctx, shape, qtype, blocks, shard=shard)
        self._tensors.append(t)
        return t

    def set_layer(self, layer: int, w: dict, attn_norm: np.ndarray, ffn_norm: np.ndarray):
        """w: raw blocks by name (wq, wk, wv, wo, w_gate, w_up, w_down), each [out, in]."""
        c = self.cfg
        qd, kd = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
        shapes = {"wq": (qd, c.d_model), "wk": (kd, c.d_model), "wv": (kd, c.d_model), "wo": (c.d_model, qd),
                  "w_gate": (c.ffn_dim, c.d_model), "w_up": (c.ffn_dim, c.d_model), "w_down": (c.d_model, c.ffn_dim)}
        split = {"wq": "rows", "wk": "rows", "wv": "rows", "wo": "cols", "w_gate": "rows", "w_up": "rows", "w_down": "cols"}
        ts = {k: self._up(c.proj_type, shapes[k], w[k], split[k]) for k in shapes}
        an = np.ascontiguousarray(attn_norm, dtype=np.float32)
        fn = np.ascontiguousarray(ffn_norm, dtype=np.float32)
        _check(self.ctx.handle, _ffi.lib().skn_llama_set_layer(
            self._h, layer, ts["wq"].handle, ts["wk"].handle, ts["wv"].handle, ts["wo"].handle, ts["w_gate"].handle,
            ts["w_up"].handle, ts["w_down"].handle, an.ctypes.data, fn.ctypes.data))

    def set_head(self, tok_embd: np.ndarray, out_norm: np.ndarray, output: np.ndarray):
        c = self.cfg
        te = self._up(c.head_type, (c.vocab, c.d_model), tok_embd)
        ot = self._up(c.head_type, (c.vocab, c.d_model), output, "rows")
        on = np.ascontiguousarray(out_norm, dtype=np.float32)
        _check(self.ctx.handle, _ffi.lib().skn_llama_set_head(self._h, te.handle, on.ctypes.data, ot.handle))

    def reset(self):
        _check(self.ctx.handle, _ffi.lib().skn_llama_reset(self._h))

    @property
    def position(self) -> int:
        return int(_ffi.lib().skn_llama_position(self._h))

    def forward(self, tokens: Optional[np.ndarray], want_logits: bool = False):
        """tokens [batch, T] int32 (None: feed back the previous greedy ids, T = 1).
        Returns next ids [batch] (and the last-position logits [batch, vocab]; under tensor
        parallelism this rank's vocabulary slice [batch, vocab / world])."""
        if tokens is None:
            tp, T = None, 1
        else:
            tokens = np.ascontiguousarray(tokens, dtype=np.int32)
            if tokens.ndim != 2 or tokens.shape[0] != self.batch:
                raise ValueError("Shapes do not align.")
            tp, T = tokens.ctypes.data, tokens.shape[1]
        nxt = np.empty(self.batch, dtype=np.int32)
        logits = np.empty((self.batch, self.cfg.vocab // self.world), dtype=np.float32) if want_logits else None
        _check(self.ctx.handle, _ffi.lib().skn_llama_forward(self._h, tp, T, nxt.ctypes.data,
                                                            None if logits is None else logits.ctypes.data))
        return (nxt, logits) if want_logits else nxt

    def forward_dev(self, tokens_dev=None, T: int = 1):
        ptr = None if tokens_dev is None else (tokens_dev.data_ptr() if hasattr(tokens_dev, "data_ptr") else tokens_dev)
        _check(self.ctx.handle, _ffi.lib().skn_llama_forward_dev(self._h, ptr, T))

    def close(self):
        if self._h:
            _ffi.lib().skn_llama_destroy(self._h)
            self._h = ctypes.c_void_p()
        for t in self._tensors:
            t.close()
        self._tensors = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def random_model_blocks(cfg: LlamaConfig, seed: int = 4):
    """Random-init raw blocks with the benchmark's value distributions (norm gains = 1).
    Returns (layers, head): layers[i] = dict of raw blocks, head = (tok_embd, output)."""
    g = synth.rng(seed)
    qd, kd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    shapes = {"wq": (qd, cfg.d_model), "wk": (kd, cfg.d_model), "wv": (kd, cfg.d_model), "wo": (cfg.d_model, qd),
              "w_gate": (cfg.ffn_dim, cfg.d_model), "w_up": (cfg.ffn_dim, cfg.d_model),
              "w_down": (cfg.d_model, cfg.ffn_dim)}
    layers = [{k: synth.make_weight(g, cfg.proj_type, *shp) for k, shp in shapes.items()} for _ in range(cfg.n_layers)]
    head = (synth.make_weight(g, cfg.head_type, cfg.vocab, cfg.d_model),
            synth.make_weight(g, cfg.head_type, cfg.vocab, cfg.d_model))
    return layers, head
