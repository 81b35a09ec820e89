"""K3 / K4 parity: tensor-core prefill matmul (bf16 operands, fp32 accumulation in TMEM) and the
SwiGLU feed-forward block against the fp64 oracle, through the C ABI.

Tolerance for bf16 operands: |y - y_ref| <= 1e-2 * sum_k |w_k x_k| per output and relative L2
<= 1e-2.  With the tensor-core path switched off the same calls meet the fp32 tolerance 1e-5."""
import numpy as np
import pytest

import skainet_b200 as skn
from conftest import BF16_TOL, FP32_TOL, assert_close_dot
from oracle import oracle
from skainet_b200 import synth

pytestmark = pytest.mark.gpu
TYPES = list(synth.TYPE_NAMES.items())


def matmul_case(ctx, qt, N, K, M, seed, tol, bias=False):
    g = synth.rng(seed)
    w = synth.make_weight(g, qt, N, K)
    x = synth.make_activations(g, M, K)
    b = g.standard_normal(N).astype(np.float32) if bias else None
    t = skn.QuantTensor(ctx, (N, K), qt, w)
    y = t.matmul_t(x, b)
    t.close()
    y_ref, absdot = oracle.matmul(qt, w, N, K, x)
    if bias:
        y_ref = y_ref + b.astype(np.float64)[None, :]
        absdot = absdot + np.abs(b.astype(np.float64))[None, :]
    assert_close_dot(y, y_ref, absdot, tol, f"type {qt} {N}x{K} M={M}")


@pytest.mark.parametrize("qt,name", TYPES)
@pytest.mark.parametrize("M,N,K", [(64, 128, 256), (128, 256, 1024), (200, 300, 512), (65, 4, 320)])
def test_prefill_matmul(ctx, qt, name, M, N, K):
    e, _ = synth.GEOMETRY[qt]
    if K % e:
        K = (K // e + 1) * e
    if K % 64:
        pytest.skip("tensor-core path needs K % 64 == 0")
    matmul_case(ctx, qt, N, K, M, seed=500 + M + N, tol=BF16_TOL, bias=(M == 128))


def test_prefill_cfg2_m64(ctx):
    """Config 2 at M = 64 on its largest shapes (Q4_0 and Q8_0)."""
    for qt in (synth.Q4_0, synth.Q8_0):
        matmul_case(ctx, qt, 1024, 4096, 64, seed=1, tol=BF16_TOL)
        matmul_case(ctx, qt, 512, 14336, 64, seed=1, tol=BF16_TOL)


def test_large_m_without_tensor_cores_meets_fp32_tolerance(ctx):
    ctx.set_prefill_min_m(0)
    try:
        matmul_case(ctx, synth.Q4_K, 96, 1024, 64, seed=9, tol=FP32_TOL)
    finally:
        ctx.set_prefill_min_m(64)


def ffn_case(ctx, M, F, K, N, seed, tol):
    g = synth.rng(seed)
    wg = synth.make_weight(g, synth.Q4_K, F, K)
    wu = synth.make_weight(g, synth.Q4_K, F, K)
    wd = synth.make_weight(g, synth.Q6_K, N, F)
    x = synth.make_activations(g, M, K)
    tg = skn.QuantTensor(ctx, (F, K), synth.Q4_K, wg)
    tu = skn.QuantTensor(ctx, (F, K), synth.Q4_K, wu)
    td = skn.QuantTensor(ctx, (N, F), synth.Q6_K, wd)
    y = skn.ffn_swiglu(ctx, tg, tu, td, x)
    for t in (tg, tu, td):
        t.close()
    ref = oracle.ffn_swiglu(synth.Q4_K, wg, wu, synth.Q6_K, wd, F, K, N, x)
    assert np.isfinite(y).all()
    rel = np.linalg.norm(y - ref) / np.linalg.norm(ref)
    mx = np.max(np.abs(y - ref)) / np.max(np.abs(ref))
    assert rel <= tol and mx <= tol, (rel, mx)


def test_ffn_decode_size_fp32(ctx):
    ffn_case(ctx, M=1, F=512, K=512, N=256, seed=3, tol=FP32_TOL * 10)   # three chained fp32 products
    ffn_case(ctx, M=5, F=768, K=256, N=128, seed=4, tol=FP32_TOL * 10)


def test_ffn_prefill_tensor_cores(ctx):
    ffn_case(ctx, M=64, F=512, K=256, N=128, seed=5, tol=BF16_TOL)
    ffn_case(ctx, M=192, F=1024, K=512, N=384, seed=6, tol=BF16_TOL)


def test_ffn_shape_errors(ctx):
    g = synth.rng(1)
    tg = skn.QuantTensor(ctx, (512, 256), synth.Q4_K, synth.make_weight(g, synth.Q4_K, 512, 256))
    tu = skn.QuantTensor(ctx, (256, 256), synth.Q4_K, synth.make_weight(g, synth.Q4_K, 256, 256))
    td = skn.QuantTensor(ctx, (128, 512), synth.Q6_K, synth.make_weight(g, synth.Q6_K, 128, 512))
    with pytest.raises(ValueError, match="Shapes do not align."):
        skn.ffn_swiglu(ctx, tg, tu, td, np.zeros((2, 256), dtype=np.float32))
    for t in (tg, tu, td):
        t.close()
