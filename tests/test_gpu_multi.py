"""Two-GPU checks of the library's own exchange (skn_comm_*, skn_allreduce_dev) and of the
tensor-parallel decoder, one process driving both devices through peer access (the one-process
model of a JVM host).  Skipped on a single-GPU box; the one-process-per-GPU route (CUDA IPC
handles through torch.distributed) is exercised by tests/tp_worker.py under torchrun.

Tolerances: the exchange sums in rank order, so its result must equal the same sum done by
torch in that order bit for bit; the sharded decoder adds partial products in another order than
the single-GPU one, so its logits are compared with the fp64 restatement (1e-4 relative L2)."""
import threading

import numpy as np
import pytest

import skainet_b200 as skn
from skainet_b200 import synth
from skainet_b200.llama import LlamaConfig, LlamaDecoder, random_model_blocks
from skainet_b200.parallel import Exchange

pytestmark = pytest.mark.gpu


def _two_gpus():
    import torch
    return torch.cuda.is_available() and torch.cuda.device_count() >= 2


needs2 = pytest.mark.skipif(not _two_gpus(), reason="needs two GPUs")


def run_ranks(fns):
    """Run one callable per rank on its own host thread (the calls block until their GPU has
    finished, and the GPUs wait for one another)."""
    out, err = [None] * len(fns), [None] * len(fns)

    def body(i):
        try:
            out[i] = fns[i]()
        except BaseException as e:   # noqa: BLE001 - reported below
            err[i] = e

    ts = [threading.Thread(target=body, args=(i,)) for i in range(len(fns))]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for e in err:
        if e is not None:
            raise e
    return out


@needs2
def test_exchange_sums_in_rank_order_and_replays():
    import torch
    ctxs = [skn.Context(device=d) for d in range(2)]
    exs = Exchange.connect_local(ctxs, 1 << 20)
    g = torch.Generator().manual_seed(5)
    for n in (4, 4096, 1 << 20, 12):          # includes the full capacity and a tiny tail
        parts = [torch.randn(n, generator=g) for _ in range(2)]
        resid = torch.randn(n, generator=g)
        want = (resid + parts[0]) + parts[1]
        dev = [(parts[r].cuda(r), resid.cuda(r), torch.empty(n, device=f"cuda:{r}")) for r in range(2)]
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)

        def rank_fn(r):
            def f():
                p, rs, o = dev[r]
                exs[r].all_reduce(p, rs, o, n)
                ctxs[r].sync()
                return o.cpu()
            return f

        outs = run_ranks([rank_fn(0), rank_fn(1)])
        assert torch.equal(outs[0], want) and torch.equal(outs[1], want)
    # in place and without a residual
    parts = [torch.randn(256, generator=g) for _ in range(2)]
    dev = [parts[r].cuda(r) for r in range(2)]
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)

    def inplace(r):
        def f():
            exs[r].all_reduce(dev[r], None, dev[r], 256)
            ctxs[r].sync()
            return dev[r].cpu()
        return f

    outs = run_ranks([inplace(0), inplace(1)])
    assert torch.equal(outs[0], parts[0] + parts[1]) and torch.equal(outs[1], outs[0])
    with pytest.raises(ValueError, match="exceed the exchange capacity"):
        exs[0].all_reduce(dev[0], None, dev[0], (1 << 20) + 64)
    for e in exs:
        e.close()
    for c in ctxs:
        c.close()


@needs2
@pytest.mark.parametrize("fused_exchange,B", [(False, 2), (True, 2), (False, 5), (True, 5)])
def test_sharded_decoder_matches_fp64_restatement(fused_exchange, B):
    """fused_exchange: single-token steps of one or two sequences push partial products from the matvec
    epilogue and sum them while the next projection prepares x (SKN_OPT_FUSED_EXCHANGE) instead of launching
    the exchange kernel.  Five sequences: the many-row path under tensor parallelism, where the option is
    asked for but does not apply (the separate exchange runs)."""
    from test_gpu_llama import RefModel, rel
    cfg = LlamaConfig(n_layers=2, d_model=256, n_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=512, vocab=512)
    layers, head = random_model_blocks(cfg, seed=9)
    T = 5
    ctxs = [skn.Context(device=d) for d in range(2)]
    for c in ctxs:
        c.set_fused_exchange(fused_exchange)
    exs = Exchange.connect_local(ctxs, B * 8 * cfg.d_model)
    decs = [LlamaDecoder(ctxs[r], cfg, batch=B, max_tokens=8, max_ctx=32, exchange=exs[r]) for r in range(2)]      # noqa: E501
    ones = np.ones(cfg.d_model, dtype=np.float32)
    for dec in decs:
        for i, l in enumerate(layers):
            dec.set_layer(i, l, ones, ones)
        dec.set_head(head[0], ones, head[1])
    ref = RefModel(cfg, layers, head)
    g = synth.rng(78)

    def step(tokens):
        outs = run_ranks([lambda d=d: d.forward(tokens, want_logits=True) for d in decs])
        logits = np.concatenate([o[1] for o in outs], axis=1)      # vocabulary slices in rank order
        assert np.array_equal(outs[0][0], outs[1][0])              # every rank picks the same token
        assert np.array_equal(outs[0][0], logits.argmax(-1))
        return outs[0][0], logits

    prompt = g.integers(0, cfg.vocab, size=(B, T)).astype(np.int32)
    nxt, logits = step(prompt)
    assert rel(logits, ref.forward(prompt)) <= 1e-4
    for s in range(3):
        tok = g.integers(0, cfg.vocab, size=(B, 1)).astype(np.int32)
        nxt, logits = step(tok)
        assert rel(logits, ref.forward(tok)) <= 1e-4, s
    fed, logits = step(None)                                       # greedy feedback on the device
    assert rel(logits, ref.forward(nxt[:, None])) <= 1e-4
    for d in decs:
        d.close()
    for e in exs:
        e.close()
    for c in ctxs:
        c.close()


@needs2
def test_one_process_per_gpu_route():
    """The same checks with one process per GPU: inbox handles cross the process boundary as CUDA
    IPC handles (tests/tp_worker.py under torch.distributed.run)."""
    import os
    import subprocess
    import sys
    import torch
    n = 2 if torch.cuda.device_count() < 4 else 4
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29731", os.path.join(here, "tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
