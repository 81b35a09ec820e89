"""One rank of the one-process-per-GPU checks (run under `python -m torch.distributed.run
--nproc-per-node N tests/tp_worker.py`; tests/test_gpu_multi.py spawns it when the box has at
least two GPUs).  The inbox handles of the exchange cross the process boundary as CUDA IPC
handles carried by torch.distributed (gloo: they are host bytes).

Checks, on every rank: the exchange's sum against the same sum formed on the host in rank order
(bit for bit), and the tensor-parallel toy decoder against the fp64 restatement (1e-4 relative
L2 on the concatenated vocabulary slices).  Prints TP_WORKER_OK from rank 0 on success."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import skainet_b200 as skn  # noqa: E402
from skainet_b200 import synth  # noqa: E402
from skainet_b200.llama import LlamaConfig, LlamaDecoder, random_model_blocks  # noqa: E402
from skainet_b200.parallel import Exchange  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(local)
    ctx = skn.Context(device=local)

    # exchange: every rank generates all partials from one seed and owns the one of its rank
    cap = 1 << 18
    ex = Exchange.connect_processes(ctx, cap)
    g = torch.Generator().manual_seed(11)
    for n in (4, 1000, cap):
        parts = [torch.randn(n, generator=g) for _ in range(world)]
        resid = torch.randn(n, generator=g)
        want = resid.clone()
        for p in parts:
            want = want + p
        mine, rs = parts[rank].cuda(), resid.cuda()
        out = torch.empty(n, device="cuda")
        torch.cuda.synchronize()
        for _ in range(3):                       # repeated use walks through both inbox buffers
            ex.all_reduce(mine, rs, out, n)
        ctx.sync()
        assert torch.equal(out.cpu(), want), f"rank {rank}: exchange sum differs at n={n}"
    ex.close()

    # tensor-parallel decoder at toy size
    from test_gpu_llama import RefModel, rel
    cfg = LlamaConfig(n_layers=2, d_model=256, n_heads=8, n_kv_heads=4, head_dim=128, ffn_dim=2048, vocab=512)
    if cfg.n_kv_heads % world or (cfg.ffn_dim // world) % 256 or (cfg.n_heads * cfg.head_dim // world) % 256:
        cfg = None
    if cfg is not None:
        layers, head = random_model_blocks(cfg, seed=9)
        B, T = 2, 5
        ex = Exchange.connect_processes(ctx, B * 8 * cfg.d_model)
        dec = LlamaDecoder(ctx, cfg, batch=B, max_tokens=8, max_ctx=32, exchange=ex)
        ones = np.ones(cfg.d_model, dtype=np.float32)
        for i, l in enumerate(layers):
            dec.set_layer(i, l, ones, ones)
        dec.set_head(head[0], ones, head[1])
        ref = RefModel(cfg, layers, head)
        gg = synth.rng(78)
        seq = [gg.integers(0, cfg.vocab, size=(B, T)).astype(np.int32)]
        seq += [gg.integers(0, cfg.vocab, size=(B, 1)).astype(np.int32) for _ in range(2)] + [None]
        prev = None
        for tok in seq:
            nxt, logits = dec.forward(tok, want_logits=True)
            slices = [None] * world
            dist.all_gather_object(slices, (nxt, logits))
            full = np.concatenate([s[1] for s in slices], axis=1)
            for s in slices:
                assert np.array_equal(s[0], slices[0][0]), "ranks picked different tokens"
            assert np.array_equal(nxt, full.argmax(-1))
            want = ref.forward(tok if tok is not None else prev[:, None])
            assert rel(full, want) <= 1e-4, f"rank {rank}: logits off by {rel(full, want)}"
            prev = nxt
        dec.close()
        ex.close()
    ctx.close()
    dist.barrier()
    if rank == 0:
        print("TP_WORKER_OK" + ("" if cfg is not None else " (decoder skipped: toy shapes do not divide)"))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
