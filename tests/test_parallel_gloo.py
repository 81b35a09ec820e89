"""The N > 1 host logic on CPU: two gloo ranks shard a quantized layer by rows (column-parallel,
all-gather of y slices) and by columns (row-parallel, all-reduce of partials) and reproduce
the single-rank oracle result.  The per-rank products come from the CPU oracle here; on GPUs the
same ranges go to skn_tensor_upload_quant_shard."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from skainet_b200 import parallel


def test_shard_ranges_cover_exactly():
    for n, w in ((4096, 8), (14336, 8), (32000, 3), (5, 8), (8, 8)):
        got = [parallel.shard_rows(n, w, r) for r in range(w)]
        assert got[0][0] == 0 and sum(c for _, c in got) == n
        for (b0, c0), (b1, _) in zip(got, got[1:]):
            assert b0 + c0 == b1
    assert parallel.shard_cols(14336, 256, 8, 3) == (3 * 1792, 1792)
    assert parallel.shard_cols(4096, 256, 3, 0) == (0, 6 * 256)      # 16 blocks over 3 ranks: 6, 5, 5
    with pytest.raises(ValueError, match="not a multiple"):
        parallel.shard_cols(1000, 256, 2, 0)
    with pytest.raises(ValueError):
        parallel.shard_rows(8, 2, 2)


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle
        from skainet_b200 import synth
        g = synth.rng(123)                       # same seed on every rank: same full layer
        N, K, M = 50, 1024, 2
        qt = synth.Q6_K
        w = synth.make_weight(g, qt, N, K)
        x = synth.make_activations(g, M, K)
        full, _ = oracle.matmul(qt, w, N, K, x)
        rb = oracle.row_bytes(qt, K)
        # column-parallel: rows [r0, r0+rc) are a contiguous byte range of the raw blocks
        r0, rc = parallel.shard_rows(N, world, rank)
        ys, _ = oracle.matmul(qt, w.reshape(-1)[r0 * rb:(r0 + rc) * rb], rc, K, x)
        y = parallel.all_gather_rows(torch.from_numpy(ys))
        np.testing.assert_array_equal(y.numpy(), full)
        # row-parallel: whole blocks of columns, partial sums all-reduced
        c0, cc = parallel.shard_cols(K, 256, world, rank)
        sub = w.reshape(N, K // 256, 210)[:, c0 // 256:(c0 + cc) // 256].copy()
        yp, _ = oracle.matmul(qt, sub, N, cc, x[:, c0:c0 + cc].copy())
        tot = parallel.all_reduce_partials(torch.from_numpy(yp))
        np.testing.assert_allclose(tot.numpy(), full, rtol=1e-12, atol=1e-12)
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_reproduces_the_full_product(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
