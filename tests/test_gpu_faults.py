"""Failure detection, with every failure made on the host: a peer that never joins an exchange, arguments a
confused caller would pass, a box without peer access (simulated), and a second host thread.  No test here
faults, traps or hangs the GPU: the only device-side event is a bounded wait that runs out by design and
reports SKN_ERR_TIMEOUT through the status word."""
import ctypes
import os
import threading
import time

import numpy as np
import pytest

import skainet_b200 as skn
from conftest import FP32_TOL, assert_close_dot
from oracle import oracle
from skainet_b200 import _ffi, synth
from skainet_b200.parallel import Exchange
from skainet_b200.tensor import (SKN_ERR_ALIGN, SKN_ERR_BUSY, SKN_ERR_COMM, SKN_ERR_SHAPE, SKN_ERR_TIMEOUT, SKN_ERR_TYPE,
                                 SknError)

pytestmark = pytest.mark.gpu


def test_exchange_wait_runs_out_when_a_peer_never_joins():
    """Two ranks of an exchange live on cuda:0; only rank 0 ever calls it.  Its kernel pushes, waits for the
    peer's flag for the configured 50 ms, gives up and returns: skn_sync reports SKN_ERR_TIMEOUT, the
    status is cleared by that report, and the context computes correct results afterwards."""
    import torch
    c0, c1 = skn.Context(0), skn.Context(0)
    try:
        c0.set_wait_limit_ms(50)
        ex = Exchange.connect_local([c0, c1], 4096)
        part = torch.ones(1024, device="cuda")
        out = torch.zeros(1024, device="cuda")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ex[0].all_reduce(part, None, out, 1024)
        with pytest.raises(SknError) as err:
            c0.sync()
        waited = time.perf_counter() - t0
        assert err.value.code == SKN_ERR_TIMEOUT and "bounded wait" in err.value.message
        assert 0.04 <= waited < 1.5, f"the wait took {waited:.3f} s for a 50 ms limit"
        c0.sync()                                  # the report cleared the status word
        # the context is still usable: a product on it matches the oracle
        g = synth.rng(5)
        w = synth.make_weight(g, synth.Q4_K, 64, 1024)
        x = synth.make_activations(g, 1, 1024)
        t = skn.QuantTensor(c0, (64, 1024), synth.Q4_K, w)
        y = t.matmul_t(x[0])
        t.close()
        ref, absdot = oracle.matmul(synth.Q4_K, w, 64, 1024, x)
        assert_close_dot(y[None, :], ref, absdot, FP32_TOL, "after the timeout")
        c0.set_wait_limit_ms(0)
        for e in ex:
            e.close()
    finally:
        c0.close()
        c1.close()


def test_arguments_a_confused_caller_would_pass(ctx):
    import torch
    L = _ffi.lib()
    g = synth.rng(6)
    w = synth.make_weight(g, synth.Q4_K, 8, 512)
    out = ctypes.c_void_p()
    # a type id the library does not run (IQ2_XXS = 16), and one that does not exist
    for bad in (16, 99, -1):
        assert L.skn_tensor_upload_quant(ctx.handle, bad, 8, 512, w.ctypes.data, w.size, ctypes.byref(out)) == SKN_ERR_TYPE
        assert not out.value
    # byte length that does not match rows x row bytes; rows that are not whole blocks
    assert L.skn_tensor_upload_quant(ctx.handle, 12, 8, 512, w.ctypes.data, w.size - 144, ctypes.byref(out)) == SKN_ERR_SHAPE
    assert b"byte length" in L.skn_last_error(ctx.handle)
    assert L.skn_tensor_upload_quant(ctx.handle, 12, 8, 500, w.ctypes.data, w.size, ctypes.byref(out)) == SKN_ERR_SHAPE
    assert b"not a multiple" in L.skn_last_error(ctx.handle)
    # device pointers off a 16-byte boundary
    t = skn.QuantTensor(ctx, (8, 512), synth.Q4_K, w)
    x = torch.zeros(516, device="cuda")
    y = torch.zeros(12, device="cuda")
    assert L.skn_matmul_dev(ctx.handle, t.handle, x.data_ptr() + 4, 1, 512, None, y.data_ptr()) == SKN_ERR_ALIGN
    assert L.skn_matmul_dev(ctx.handle, t.handle, x.data_ptr(), 1, 512, None, y.data_ptr() + 8) == SKN_ERR_ALIGN
    assert L.skn_matmul_dev(ctx.handle, t.handle, x.data_ptr(), 1, 512, None, y.data_ptr()) == 0
    ctx.sync()
    t.close()


def test_box_without_peer_access_is_reported(monkeypatch):
    """connect_local on a box whose GPUs cannot reach one another (simulated on the host by an environment
    flag the library reads) answers SKN_ERR_COMM and leaves the exchanges unconnected."""
    import torch
    c0, c1 = skn.Context(0), skn.Context(0)
    try:
        monkeypatch.setenv("SKN_FAKE_NO_PEER_ACCESS", "1")
        with pytest.raises(SknError) as err:
            Exchange.connect_local([c0, c1], 1024)
        assert err.value.code == SKN_ERR_COMM and "cannot access" in err.value.message
        monkeypatch.delenv("SKN_FAKE_NO_PEER_ACCESS")
        ex = Exchange.connect_local([c0, c1], 1024)
        for e in ex:
            e.close()
    finally:
        c0.close()
        c1.close()


def test_second_host_thread_is_refused_while_the_first_is_inside_a_call():
    """One host thread at a time per context: while thread A sits in blocking calls (a 235 MB dequantise to
    pageable memory takes tens of milliseconds), thread B's calls on the same context come back with
    SKN_ERR_BUSY; whichever thread is inside first wins, the other is refused without side effects and may
    simply call again.  Every call returns SKN_OK or SKN_ERR_BUSY, nothing else, and the data is right."""
    L = _ffi.lib()
    own = skn.Context(0)
    try:
        g = synth.rng(7)
        N, K = 14336, 4096
        w = synth.make_weight(g, synth.Q4_K, N, K)
        t = skn.QuantTensor(own, (N, K), synth.Q4_K, w)
        deq = np.empty((N, K), dtype=np.float32)
        a_rc, b_rc = [], []
        running = threading.Event()
        done = threading.Event()

        def thread_a():
            running.set()
            ok = 0
            while ok < 6 and len(a_rc) < 10000:
                a_rc.append(L.skn_dequantize(own.handle, t.handle, deq.ctypes.data))
                ok += a_rc[-1] == 0
            done.set()

        def thread_b():
            running.wait()
            while not done.is_set():
                b_rc.append(L.skn_sync(own.handle))
                if b_rc[-1] == SKN_ERR_BUSY:
                    assert b"another host thread" in L.skn_last_error(None)

        ta, tb = threading.Thread(target=thread_a), threading.Thread(target=thread_b)
        ta.start()
        tb.start()
        ta.join()
        tb.join()
        assert a_rc.count(0) == 6 and set(a_rc) <= {0, SKN_ERR_BUSY}
        assert SKN_ERR_BUSY in b_rc, "the second thread was never refused"
        assert set(b_rc) <= {0, SKN_ERR_BUSY}
        assert L.skn_sync(own.handle) == 0
        want = oracle.dequant(synth.Q4_K, w[:4]).reshape(4, K)
        assert np.array_equal(deq[:4].view(np.uint32), want.view(np.uint32))
        t.close()
    finally:
        own.close()
