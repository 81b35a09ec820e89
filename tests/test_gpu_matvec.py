"""K2 parity: fused dequant-dot through the C ABI against the fp64 oracle.

Tolerance (fp32 accumulation): |y - y_ref| <= 1e-5 * sum_k |w_k x_k| per output and
relative L2 error <= 1e-5 (conftest.assert_close_dot)."""
import numpy as np
import pytest

import skainet_b200 as skn
from conftest import FP32_TOL, assert_close_dot
from oracle import oracle
from skainet_b200 import synth

pytestmark = pytest.mark.gpu
TYPES = list(synth.TYPE_NAMES.items())


def run_case(ctx, qt, N, K, M, seed, bias=False):
    g = synth.rng(seed)
    w = synth.make_weight(g, qt, N, K)
    x = synth.make_activations(g, M, K)
    b = g.standard_normal(N).astype(np.float32) if bias else None
    t = skn.QuantTensor(ctx, (N, K), qt, w)
    y = t.matmul_t(x if M > 1 else x[0], b)
    t.close()
    y_ref, absdot = oracle.matmul(qt, w, N, K, x)
    if bias:
        y_ref = y_ref + b.astype(np.float64)[None, :]
        absdot = absdot + np.abs(b.astype(np.float64))[None, :]
    assert_close_dot(np.asarray(y).reshape(M, N), y_ref, absdot, FP32_TOL, f"type {qt} {N}x{K} M={M}")
    return y


def test_cfg1_q4k_matvec(ctx):
    """Config 1: Q4_K 4096x4096, x fp32[4096], seed 0."""
    w, x = synth.cfg1(0)
    t = skn.QuantTensor(ctx, (4096, 4096), synth.Q4_K, w)
    y = t.matmul_t(x[0])
    y2 = t.matmul_t(x[0])
    t.close()
    assert y.shape == (4096,)
    assert np.array_equal(y, y2), "matvec must be deterministic run to run"
    y_ref, absdot = oracle.matmul(synth.Q4_K, w, 4096, 4096, x)
    assert_close_dot(y[None, :], y_ref, absdot, FP32_TOL, "cfg1")


@pytest.mark.parametrize("qt,name", TYPES)
@pytest.mark.parametrize("N,K", [(1, 256), (5, 512), (33, 2048), (148, 4096), (300, 2304), (64, 14336), (4096, 4096)])
def test_matvec_m1_shapes(ctx, qt, name, N, K):
    run_case(ctx, qt, N, K, 1, seed=1000 + N + K)


@pytest.mark.parametrize("qt,name", TYPES)
@pytest.mark.parametrize("M", [2, 3, 4, 5, 16, 17])
def test_small_batch(ctx, qt, name, M):
    run_case(ctx, qt, 96, 1024, M, seed=2000 + M, bias=(M % 2 == 0))


@pytest.mark.parametrize("qt,name", TYPES)
def test_bias_m1(ctx, qt, name):
    run_case(ctx, qt, 200, 4096, 1, seed=77, bias=True)


@pytest.mark.parametrize("qt", [synth.Q4_0, synth.Q8_0])
@pytest.mark.parametrize("N,K", [(14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("M", [1, 4])
def test_cfg2_shapes(ctx, qt, N, K, M):
    """Config 2's large shapes at M = 1 and 4 (M = 16, 64 are covered at reduced N)."""
    run_case(ctx, qt, N, K, M, seed=1)


def _sampled_rows_case(ctx, qt, N, K, M, seed, tol, n_sample=96, bias=False):
    """The product at full size on the GPU, the oracle on `n_sample` sampled output rows (all M activation rows)."""
    g = synth.rng(seed)
    w = synth.make_weight(g, qt, N, K)
    x = synth.make_activations(g, M, K)
    b = g.standard_normal(N).astype(np.float32) if bias else None
    t = skn.QuantTensor(ctx, (N, K), qt, w)
    y = np.asarray(t.matmul_t(x if M > 1 else x[0], b)).reshape(M, N)
    t.close()
    assert np.isfinite(y).all()
    rows = np.unique(np.concatenate([g.choice(N, size=min(N, n_sample - 4), replace=False), [0, 1, N - 2, N - 1]]))
    y_ref, absdot = oracle.matmul(qt, np.ascontiguousarray(w[rows]), rows.size, K, x)
    if bias:
        y_ref = y_ref + b[rows].astype(np.float64)[None, :]
        absdot = absdot + np.abs(b[rows].astype(np.float64))[None, :]
    assert_close_dot(y[:, rows], y_ref, absdot, tol, f"type {qt} {N}x{K} M={M}")


@pytest.mark.parametrize("qt", [synth.Q4_0, synth.Q8_0])
@pytest.mark.parametrize("N,K", [(4096, 4096), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("M", [16, 64])
def test_cfg2_full_shapes_at_batch_16_and_64(ctx, qt, N, K, M):
    """Config 2 at its own shapes: M = 16 is the many-row fp32 path (1e-5), M = 64 the bf16 tensor-core path (1e-2);
    the oracle runs on sampled output rows."""
    from conftest import BF16_TOL
    _sampled_rows_case(ctx, qt, N, K, M, seed=1, tol=FP32_TOL if M < 64 else BF16_TOL)


@pytest.mark.parametrize("qt,name", TYPES)
@pytest.mark.parametrize("N,K,M", [(28672, 4096, 16), (4096, 14336, 16), (6144, 4096, 8), (4096, 4096, 5), (32000, 4096, 16),
                                   (300, 2304, 7), (33, 256, 3), (1000, 5120, 12)])
def test_many_rows_in_one_pass(ctx, qt, name, N, K, M):
    """3 to 16 activation rows: every weight is read once (the many-row kernel for Q4_K / Q8_0 / Q4_0; Q6_K keeps four
    rows per pass), decoder-size shapes and odd ones (short rows, a row count that does not fill a tile, a short
    last K chunk), with a bias."""
    _sampled_rows_case(ctx, qt, N, K, M, seed=6000 + N + K + M, tol=FP32_TOL, n_sample=64, bias=(M % 2 == 1))


@pytest.mark.parametrize("N,K,M", [(32000, 4096, 1), (32000, 4096, 4), (4096, 14336, 1), (4096, 14336, 3), (1000, 2816, 2),
                                   (37, 768, 4)])
def test_q6k_at_lm_head_and_down_projection_sizes(ctx, N, K, M):
    """Q6_K on the integer tensor-core path: 16-weight scale groups, blocks on 2-byte boundaries, short
    last K chunks (11 and 3 blocks), 1 to 4 activation rows."""
    run_case(ctx, synth.Q6_K, N, K, M, seed=5000 + N + K + M, bias=(M == 2))


@pytest.mark.parametrize("pinned", [False, True])
def test_asynchronous_host_calls_run_in_order(ctx, pinned):
    """skn_matmul_async: two dependent products enqueued back to back (the first result is the second call's
    x_host), one skn_sync; results equal the blocking calls bit for bit.  Pageable buffers go through staged
    copies, page-locked ones are read and written by the kernels themselves."""
    import ctypes
    from skainet_b200 import _ffi
    L = _ffi.lib()
    g = synth.rng(61)
    N1, K, N2 = 512, 1024, 96
    w1, w2 = synth.make_weight(g, synth.Q4_K, N1, K), synth.make_weight(g, synth.Q6_K, N2, N1)
    x = synth.make_activations(g, 1, K)[0]
    t1, t2 = skn.QuantTensor(ctx, (N1, K), synth.Q4_K, w1), skn.QuantTensor(ctx, (N2, N1), synth.Q6_K, w2)
    if pinned:
        torch = pytest.importorskip("torch")
        keep = [torch.zeros(n, dtype=torch.float32).pin_memory() for n in (K, N1, N2)]
        xp, y1, y2 = (t.numpy() for t in keep)
        xp[:] = x
        x = xp
    else:
        y1 = np.zeros(N1, dtype=np.float32)
        y2 = np.zeros(N2, dtype=np.float32)
    ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    assert L.skn_matmul_async(ctx.handle, t1.handle, ptr(x), 1, K, None, ptr(y1)) == 0
    t2.matmul_t_async(y1, y2)                # the Python mirror of the same call
    assert L.skn_sync(ctx.handle) == 0
    b1 = t1.matmul_t(x)
    b2 = t2.matmul_t(b1)
    t1.close()
    t2.close()
    assert np.array_equal(y1, b1) and np.array_equal(y2, b2)
    ref1, ad1 = oracle.matmul(synth.Q4_K, w1, N1, K, x[None, :])
    assert_close_dot(y1[None, :], ref1, ad1, FP32_TOL, "first product")


def test_host_pointer_calls_keep_their_own_order_under_relaxed_order(ctx):
    """SKN_OPT_RELAXED_ORDER describes the caller's consecutive calls, not the fetch -> product chain inside
    one host-pointer call: with the option on, page-locked buffers, a different x for every call and a
    second call that consumes the first call's result, every result still equals the stream-order bits."""
    import ctypes
    torch = pytest.importorskip("torch")
    from skainet_b200 import _ffi
    L = _ffi.lib()
    g = synth.rng(63)
    N1, K, N2 = 512, 4096, 256
    w1, w2 = synth.make_weight(g, synth.Q4_K, N1, K), synth.make_weight(g, synth.Q4_K, N2, N1)
    t1, t2 = skn.QuantTensor(ctx, (N1, K), synth.Q4_K, w1), skn.QuantTensor(ctx, (N2, N1), synth.Q4_K, w2)
    reps = 24
    xs = synth.make_activations(g, reps, K)
    want1 = np.stack([t1.matmul_t(xs[i]) for i in range(reps)])
    want2 = np.stack([t2.matmul_t(want1[i]) for i in range(reps)])
    keep = [torch.zeros(n, dtype=torch.float32).pin_memory() for n in (reps * K, reps * N1, reps * N2)]
    xp, y1, y2 = (a.numpy() for a in keep)
    xp[:] = xs.reshape(-1)
    at = lambda a, off: ctypes.c_void_p(a.ctypes.data + 4 * off)
    ctx.set_relaxed_order(True)
    try:
        for i in range(reps):
            assert L.skn_matmul_async(ctx.handle, t1.handle, at(xp, i * K), 1, K, None, at(y1, i * N1)) == 0
            assert L.skn_matmul_async(ctx.handle, t2.handle, at(y1, i * N1), 1, N1, None, at(y2, i * N2)) == 0
        assert L.skn_sync(ctx.handle) == 0
    finally:
        ctx.set_relaxed_order(False)
    t1.close()
    t2.close()
    assert np.array_equal(y1.reshape(reps, N1), want1)
    assert np.array_equal(y2.reshape(reps, N2), want2)


def test_blocking_call_on_page_locked_buffers(ctx):
    """skn_matmul with page-locked x, bias and y (no copy-engine transfer: x is fetched by a kernel, y and the
    status word are written to the mapped buffers) returns the bits of the pageable route, for 1 and 3 rows."""
    import ctypes
    torch = pytest.importorskip("torch")
    from skainet_b200 import _ffi
    L = _ffi.lib()
    g = synth.rng(62)
    N, K = 328, 768
    w = synth.make_weight(g, synth.Q4_K, N, K)
    t = skn.QuantTensor(ctx, (N, K), synth.Q4_K, w)
    for M in (1, 3):
        x = synth.make_activations(g, M, K)
        b = g.standard_normal(N).astype(np.float32)
        want = t.matmul_t(x if M > 1 else x[0], b)
        keep = [torch.zeros(n, dtype=torch.float32).pin_memory() for n in (M * K, N, M * N)]
        xp, bp, yp = (a.numpy() for a in keep)
        xp[:] = x.reshape(-1)
        bp[:] = b
        rc = L.skn_matmul(ctx.handle, t.handle, xp.ctypes.data_as(ctypes.c_void_p), M, K, bp.ctypes.data_as(ctypes.c_void_p),
                          yp.ctypes.data_as(ctypes.c_void_p))
        assert rc == 0
        assert np.array_equal(yp.reshape(np.shape(want)), want)
    t.close()


def test_linearity_at_full_size(ctx):
    """Size-independent property at cfg1's size: W(a x1 + b x2) = a W x1 + b W x2."""
    w, _ = synth.cfg1(0)
    g = synth.rng(9)
    x1, x2 = synth.make_activations(g, 1, 4096)[0], synth.make_activations(g, 1, 4096)[0]
    t = skn.QuantTensor(ctx, (4096, 4096), synth.Q4_K, w)
    y1, y2, y3 = t.matmul_t(x1), t.matmul_t(x2), t.matmul_t((2.0 * x1 - 0.5 * x2).astype(np.float32))
    t.close()
    lin = 2.0 * y1.astype(np.float64) - 0.5 * y2.astype(np.float64)
    scale = np.abs(y1).max() + np.abs(y2).max()
    assert np.max(np.abs(y3 - lin)) <= 2e-5 * scale * 10


def test_sharded_matvec_equals_slices(ctx):
    """Column-parallel shards (row ranges) give slices of y; row-parallel shards (column
    ranges, Q6_K pitch not a multiple of 16) sum to y."""
    g = synth.rng(3)
    N, K = 64, 14336
    for qt in (synth.Q4_K, synth.Q6_K):
        w = synth.make_weight(g, qt, N, K)
        x = synth.make_activations(g, 1, K)
        y_ref, absdot = oracle.matmul(qt, w, N, K, x)
        # row ranges
        parts = []
        for r in range(4):
            t = skn.QuantTensor(ctx, (N, K), qt, w, shard=(r * 16, 16, 0, K))
            parts.append(t.matmul_t(x[0]))
            t.close()
        assert_close_dot(np.concatenate(parts)[None, :], y_ref, absdot, FP32_TOL, "row shards")
        # column ranges: 8 shards of 1792 columns (Q6_K: 1470 bytes per row -> padded pitch)
        acc = np.zeros(N, dtype=np.float64)
        for c in range(8):
            t = skn.QuantTensor(ctx, (N, K), qt, w, shard=(0, N, c * 1792, 1792))
            acc += t.matmul_t(x[0, c * 1792:(c + 1) * 1792])
            t.close()
        assert_close_dot(acc[None, :], y_ref, absdot, FP32_TOL, "column shards")


def test_shapes_do_not_align(ctx):
    # TensorTest.kt:65-70: IllegalArgumentException("Shapes do not align.")
    w = synth.make_weight(synth.rng(1), synth.Q4_K, 4, 512)
    t = skn.QuantTensor(ctx, (4, 512), synth.Q4_K, w)
    with pytest.raises(ValueError, match="Shapes do not align."):
        t.matmul_t(np.zeros(256, dtype=np.float32))
    with pytest.raises(ValueError, match="Shapes do not align."):
        t.matmul_t(np.zeros((2, 3, 512), dtype=np.float32))
    t.close()


def test_empty_inputs(ctx):
    w = synth.make_weight(synth.rng(1), synth.Q8_0, 4, 64)
    t = skn.QuantTensor(ctx, (4, 64), synth.Q8_0, w)
    y = t.matmul_t(np.zeros((0, 64), dtype=np.float32))
    assert y.shape == (0, 4)
    t.close()
    t0 = skn.QuantTensor(ctx, (0, 64), synth.Q8_0, np.zeros(0, dtype=np.uint8))
    assert t0.matmul_t(np.zeros(64, dtype=np.float32)).shape == (0,)
    t0.close()


def test_extreme_activations(ctx):
    """Zero, tiny and large activations stay within tolerance (the streaming kernel
    pre-scales x by a power of two, which is exact over this range)."""
    g = synth.rng(21)
    N, K = 64, 4096
    w = synth.make_weight(g, synth.Q4_K, N, K)
    t = skn.QuantTensor(ctx, (N, K), synth.Q4_K, w)
    for scale in (0.0, 1e-20, 1e-6, 1e6, 1e12):
        x = (synth.make_activations(g, 1, K) * np.float32(scale)).astype(np.float32)
        y = t.matmul_t(x[0])
        y_ref, absdot = oracle.matmul(synth.Q4_K, w, N, K, x)
        assert_close_dot(y[None, :], y_ref, absdot, FP32_TOL, f"x scale {scale}")
    t.close()


def _zero_weight_at(qt, w, N, K, pos):
    """Raw blocks with the weight at column block * blk + pos[block] of every row made an exact zero (the
    value a quantiser produces for a zero weight): Q4_0 q = 8, Q8_0 q = 0, Q4_K scale and min of the weight's
    sub-block 0, Q6_K scale of its 16-weight group 0."""
    e, bb = synth.GEOMETRY[qt]
    nb = K // e
    blk = w.reshape(N, nb, bb).copy()
    for b in range(nb):
        k = int(pos[b])
        if qt == synth.Q4_0:
            i = 2 + (k % 16)
            blk[:, b, i] = (blk[:, b, i] & 0xF0) | 8 if k < 16 else (blk[:, b, i] & 0x0F) | 0x80
        elif qt == synth.Q8_0:
            blk[:, b, 2 + k] = 0
        elif qt == synth.Q4_K:
            j, sc = k // 32, blk[:, b, 4:16]
            if j < 4:
                sc[:, j] &= 0xC0
                sc[:, j + 4] &= 0xC0
            else:
                sc[:, j + 4] = 0
                sc[:, j - 4] &= 0x3F
                sc[:, j] &= 0x3F
        else:
            h, l = k // 128, k % 128
            blk[:, b, 192 + 8 * h + 2 * (l // 32) + (l % 32) // 16] = 0
    return blk.reshape(N, nb * bb)


@pytest.mark.parametrize("qt,name", TYPES)
@pytest.mark.parametrize("M", [1, 3])
@pytest.mark.parametrize("ratio", [1e2, 1e3, 1e4, 1e6])
@pytest.mark.parametrize("zero_weight", [False, True])
def test_in_block_outliers(ctx, qt, name, M, ratio, zero_weight):
    """One activation per 256-block `ratio` times the rest (the channel outliers of a residual stream), met by
    ordinary weights or by an exactly zero weight (then only its neighbours contribute, and they must not have
    lost their precision to the outlier): the stated fp32 tolerance holds unchanged."""
    g = synth.rng(8000 + int(np.log10(ratio)) * 10 + M)
    N, K = 64, 2048
    e, _ = synth.GEOMETRY[qt]
    w = synth.make_weight(g, qt, N, K)
    x = synth.make_activations(g, M, K)
    big = g.integers(0, 256, size=K // 256)                       # position of the outlier inside every 256-block
    cols = np.arange(K // 256) * 256 + big
    x[:, cols] *= np.float32(ratio) * np.where(g.random((M, cols.size)) < 0.5, -1, 1).astype(np.float32)
    if zero_weight:
        pos = np.full(K // e, -1)
        pos[cols // e] = cols % e
        w0 = w.reshape(N, K // e, -1).copy()
        keep = pos < 0
        w = _zero_weight_at(qt, w, N, K, np.where(keep, 0, pos))
        w.reshape(N, K // e, -1)[:, keep] = w0[:, keep]             # blocks without an outlier stay as drawn
        deq = oracle.dequant(qt, w).reshape(N, K)
        assert np.all(deq[:, cols] == 0.0)
    t = skn.QuantTensor(ctx, (N, K), qt, w)
    y = t.matmul_t(x if M > 1 else x[0])
    t.close()
    y_ref, absdot = oracle.matmul(qt, w, N, K, x)
    assert_close_dot(np.asarray(y).reshape(M, N), y_ref, absdot, FP32_TOL, f"{name} M={M} outlier x{ratio:g} zero={zero_weight}")


def test_many_outlier_blocks_and_mixed_scales(ctx):
    """Every block of a row carries an outlier (more blocks than the kernel has second-tier slots for), and one
    block mixes three scales (1e6, 1e3, 1): the result stays within the bound of one tier, 2^-30 of a block's
    largest activation per activation, far inside the tolerance for ordinary weights."""
    g = synth.rng(8100)
    N, K = 48, 14336
    for qt in (synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.Q4_0):
        w = synth.make_weight(g, qt, N, K)
        x = synth.make_activations(g, 2, K)
        x[:, ::256] *= np.float32(3e4)
        x[:, 7] *= np.float32(1e6)
        x[:, 9] *= np.float32(1e3)
        t = skn.QuantTensor(ctx, (N, K), qt, w)
        y = t.matmul_t(x)
        t.close()
        y_ref, absdot = oracle.matmul(qt, w, N, K, x)
        assert_close_dot(y, y_ref, absdot, FP32_TOL, f"type {qt}")


def test_grouped_matvec_equals_separate_products(ctx):
    """Q/K/V-style group: three weights of one type and K in one launch, with an added vector
    (bias / residual, in place) on one of them; results are bit-identical to separate calls."""
    import ctypes
    import torch
    from skainet_b200 import _ffi
    L = _ffi.lib()
    g = synth.rng(31)
    K = 4096
    for qt in (synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.Q4_0):
        shapes = [(256, K), (64, K), (40, K)]
        ws = [skn.QuantTensor(ctx, s, qt, synth.make_weight(g, qt, *s)) for s in shapes]
        x = torch.from_numpy(synth.make_activations(g, 1, K)[0].copy()).cuda()
        res = torch.randn(shapes[0][0], device="cuda")
        ys_ref = [torch.empty(s[0], device="cuda") for s in shapes]
        for w, y, add in zip(ws, ys_ref, (res, None, None)):
            w.matmul_t_dev(x, 1, y, bias_dev=add)
        ys = [res.clone(), torch.empty(shapes[1][0], device="cuda"), torch.empty(shapes[2][0], device="cuda")]
        wp = (ctypes.c_void_p * 3)(*[w.handle.value for w in ws])
        yp = (ctypes.c_void_p * 3)(*[y.data_ptr() for y in ys])
        ap = (ctypes.c_void_p * 3)(ys[0].data_ptr(), None, None)         # y[0] aliases its residual
        rc = L.skn_matvec_group_dev(ctx.handle, 3, wp, x.data_ptr(), yp, ap)
        assert rc == 0, L.skn_last_error(ctx.handle)
        ctx.sync()
        for a, b in zip(ys, ys_ref):
            assert torch.equal(a, b)
        for w in ws:
            w.close()


def test_fused_norm_and_swiglu_preparation(ctx):
    """RMSNorm or silu(x) * u folded into the matvec's preparation of x, against the oracle's
    product over the separately transformed vector (fp32 tolerance on sum |w . x|); a group of
    mixed block types takes the element-wise kernels plus separate launches instead."""
    import ctypes
    import torch
    from skainet_b200 import _ffi
    L = _ffi.lib()
    g = synth.rng(77)
    K, eps = 4096, 1e-5
    for types in ((synth.Q4_K, synth.Q4_K), (synth.Q6_K, synth.Q6_K), (synth.Q8_0, synth.Q8_0), (synth.Q4_0, synth.Q4_0),
                  (synth.Q4_K, synth.Q8_0)):
        shapes = [(192, K), (72, K)]
        blocks = [synth.make_weight(g, qt, *s) for qt, s in zip(types, shapes)]
        ws = [skn.QuantTensor(ctx, s, qt, b) for qt, s, b in zip(types, shapes, blocks)]
        x = synth.make_activations(g, 1, K)[0].astype(np.float32)
        gain = (1.0 + 0.1 * g.standard_normal(K)).astype(np.float32)
        u = g.standard_normal(K).astype(np.float32)
        res = g.standard_normal(shapes[0][0]).astype(np.float32)
        x64 = x.astype(np.float64)
        x_norm = (x64 / np.sqrt(np.mean(x64 * x64) + eps) * gain).astype(np.float32)
        x_silu = (x64 / (1.0 + np.exp(-x64)) * u).astype(np.float32)
        xd, gd, ud = (torch.from_numpy(a.copy()).cuda() for a in (x, gain, u))
        wp = (ctypes.c_void_p * 2)(*[w.handle.value for w in ws])
        for name, xin, gp, up in (("norm", x_norm, gd.data_ptr(), None), ("swiglu", x_silu, None, ud.data_ptr())):
            ys = [torch.from_numpy(res.copy()).cuda(), torch.empty(shapes[1][0], device="cuda")]
            yp = (ctypes.c_void_p * 2)(*[y.data_ptr() for y in ys])
            ap = (ctypes.c_void_p * 2)(ys[0].data_ptr(), None)
            rc = L.skn_matvec_fused_dev(ctx.handle, 2, wp, xd.data_ptr(), yp, ap, gp, eps, up)
            assert rc == 0, L.skn_last_error(ctx.handle)
            ctx.sync()
            for t, (qt, s, b) in enumerate(zip(types, shapes, blocks)):
                y_ref, absdot = oracle.matmul(qt, b, s[0], K, xin[None, :])
                if t == 0:
                    y_ref = y_ref + res[None, :]
                    absdot = absdot + np.abs(res)[None, :]
                # the in-kernel transform rounds x once more than the reference vector does
                assert_close_dot(ys[t].cpu().numpy()[None, :], y_ref, absdot, 4 * FP32_TOL, f"{name} types {types} tensor {t}")
        rc = L.skn_matvec_fused_dev(ctx.handle, 2, wp, xd.data_ptr(), yp, ap, gd.data_ptr(), eps, ud.data_ptr())
        assert rc == 8 and "not both" in L.skn_last_error(ctx.handle).decode()
        for w in ws:
            w.close()


@pytest.mark.parametrize("qt,name", list(synth.EXTRA_TYPE_NAMES.items()))
@pytest.mark.parametrize("M", [1, 3, 16])
def test_further_block_types_on_the_generic_kernel(ctx, qt, name, M):
    """Q4_1 / Q5_0 / Q5_1 / Q5_K / Q2_K / Q3_K / IQ4_NL / IQ4_XS have no streaming or tensor-core kernel: every M runs the generic
    fused dequant-dot in fp32 (also from the prefill threshold on)."""
    run_case(ctx, qt, 96, 1024, M, seed=300 + qt, bias=(M == 3))
    run_case(ctx, qt, 40, 256, M, seed=400 + qt)
