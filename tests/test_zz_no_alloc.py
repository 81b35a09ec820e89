"""The allocation-free attention entry point against the ordinary one.

Who needs it: a host that may not allocate device memory at call time -- a serving loop with a
memory plan fixed at start-up, code that cannot afford the device-wide synchronisation a CUDA
allocation implies, or an embedding runtime that owns the allocator.  skn_attn_decode_noalloc_dev
keeps its split partials in a 4 MiB array compiled into the library instead.

This file is collected last on purpose: a run that stops at the first failure has then already
executed every other test.  It passes on its own in a fresh process and after the other tests.
"""
import ctypes

import numpy as np
import pytest

import skainet_b200 as skn
from conftest import FP32_TOL
from oracle import oracle
from skainet_b200 import _ffi, synth

pytestmark = pytest.mark.gpu


# (batch, query heads, kv heads, capacity, cache type, lengths): every route the entry point can take
ROUTES = [
    pytest.param(4, 32, 8, 1000, "f32", None, id="split-and-merge"),
    pytest.param(1, 32, 8, 512, "f32", None, id="one-launch-ticket-merge"),
    pytest.param(8, 32, 8, 4096, "f32", "long", id="bulk-copy-ring"),
    pytest.param(2, 32, 8, 2048, "f16", None, id="fp16-cache"),
]


@pytest.mark.parametrize("B,Hq,Hkv,cap,dtype,lens_kind", ROUTES)
def test_noalloc_attention_matches_regular_entry_point_twice(B, Hq, Hkv, cap, dtype, lens_kind):
    """Two calls in a row on each route, compared with the ordinary entry point and with the fp64 oracle; the
    free device memory after the calls equals the free memory before them (nothing was allocated)."""
    import torch

    L = _ffi.lib()
    own_ctx = skn.Context(0)
    try:
        g = synth.rng(42)
        D = 128
        kv = skn.KVCache(own_ctx, B, Hkv, D, cap, dtype=dtype)
        assert kv.scratch_bytes(Hq) <= 4 << 20
        dev = torch.device("cuda", 0)
        q_dev = torch.empty((B, Hq, D), dtype=torch.float32, device=dev)
        out_ref = torch.empty_like(q_dev)
        out_new = torch.full_like(q_dev, float("nan"))
        scale = ctypes.c_float(1.0 / np.sqrt(D))
        for call in range(2):          # two calls in a row: the shared array keeps the first call's contents
            lo = cap // 2 if lens_kind == "long" else 1
            lens = g.integers(lo, cap + 1, size=B).astype(np.int32)
            kc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
            vc = g.standard_normal((B, Hkv, cap, D), dtype=np.float32)
            kv.load(kc, vc, lens)
            q = g.standard_normal((B, Hq, D), dtype=np.float32)
            q_dev.copy_(torch.from_numpy(q))
            torch.cuda.synchronize()
            rc = L.skn_attn_decode_dev(kv.handle, q_dev.data_ptr(), Hq, scale, out_ref.data_ptr(), None)
            assert rc == 0, L.skn_last_error(own_ctx.handle)
            own_ctx.sync()
            free_before = torch.cuda.mem_get_info(0)[0]
            rc = L.skn_attn_decode_noalloc_dev(kv.handle, q_dev.data_ptr(), Hq, scale, out_new.data_ptr())
            assert rc == 0, L.skn_last_error(own_ctx.handle)
            own_ctx.sync()
            assert torch.cuda.mem_get_info(0)[0] == free_before, "the call changed the free device memory"
            a, b = out_new.cpu().numpy().astype(np.float64), out_ref.cpu().numpy().astype(np.float64)
            assert np.isfinite(a).all()
            assert np.linalg.norm(a - b) <= FP32_TOL * np.linalg.norm(b), f"call {call}"
            assert np.max(np.abs(a - b)) <= FP32_TOL * np.max(np.abs(b)), f"call {call}"
            if dtype == "f16":
                kc, vc = kc.astype(np.float16).astype(np.float32), vc.astype(np.float16).astype(np.float32)
            want = oracle.attn_decode(q, kc, vc, lens)
            assert np.linalg.norm(a - want) <= FP32_TOL * np.linalg.norm(want), f"call {call} against the oracle"
        kv.close()
    finally:
        own_ctx.close()


def test_noalloc_attention_refuses_what_its_array_cannot_hold():
    import torch

    L = _ffi.lib()
    own_ctx = skn.Context(0)
    try:
        dev = torch.device("cuda", 0)
        q_dev = torch.zeros((8, 32, 128), dtype=torch.float32, device=dev)
        out_new = torch.zeros_like(q_dev)
        scale = ctypes.c_float(1.0 / np.sqrt(128))
        # beyond the built-in array: refused with a clear message, nothing is launched
        big = skn.KVCache(own_ctx, 8, 8, 128, 8192)
        assert big.scratch_bytes(32) > 4 << 20
        rc = L.skn_attn_decode_noalloc_dev(big.handle, q_dev.data_ptr(), 32, scale, out_new.data_ptr())
        assert rc == 1   # SKN_ERR_SHAPE
        msg = L.skn_last_error(own_ctx.handle).decode()
        assert "exceeds the built-in" in msg and "4194304" in msg
        big.close()
    finally:
        own_ctx.close()
