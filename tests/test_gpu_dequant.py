"""K1 parity: dequantised weights are bit-exact -- against the committed gguf-py golden
vectors and against the oracle on seeded blocks.  Everything goes through the C ABI."""
import numpy as np
import pytest

import skainet_b200 as skn
from oracle import oracle
from skainet_b200 import synth

pytestmark = pytest.mark.gpu
TYPES = list(synth.ALL_TYPE_NAMES.items())


@pytest.mark.parametrize("qt,name", TYPES)
def test_golden_blocks_bit_exact(ctx, golden, qt, name):
    blocks, vals = golden[f"{name}_blocks"], golden[f"{name}_values"]
    e, _ = synth.GEOMETRY[qt]
    # lay the golden blocks out as one row each, then as a single long row
    for shape in ((blocks.shape[0], e), (1, blocks.shape[0] * e), (8, blocks.shape[0] // 8 * e)):
        t = skn.QuantTensor(ctx, shape, qt, blocks)
        got = t.dequantize()
        t.close()
        assert np.array_equal(got.reshape(-1).view(np.uint32), vals.reshape(-1).view(np.uint32))


@pytest.mark.parametrize("qt,name", TYPES)
@pytest.mark.parametrize("n_rows,n_cols", [(1, 256), (3, 512), (257, 1024), (64, 4096)])
def test_seeded_blocks_bit_exact(ctx, qt, name, n_rows, n_cols):
    w = synth.make_weight(synth.rng(100 + qt), qt, n_rows, n_cols)
    t = skn.QuantTensor(ctx, (n_rows, n_cols), qt, w)
    got = t.dequantize()
    t.close()
    ref = oracle.dequant(qt, w).reshape(n_rows, n_cols)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_cfg1_weight_bit_exact(ctx):
    w, _ = synth.cfg1(0)
    t = skn.QuantTensor(ctx, (4096, 4096), synth.Q4_K, w)
    got = t.dequantize()
    t.close()
    ref = oracle.dequant(synth.Q4_K, w).reshape(4096, 4096)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("qt,name", TYPES)
def test_sharded_upload_keeps_blocks_unchanged(ctx, qt, name):
    """A row/column shard dequantises to the matching sub-matrix (row pitch is padded on
    the device when the shard's row bytes are not a multiple of 16)."""
    e, _ = synth.GEOMETRY[qt]
    n_rows, n_cols = 12, 7 * e if e == 256 else 7 * 8 * e
    w = synth.make_weight(synth.rng(7), qt, n_rows, n_cols)
    full = oracle.dequant(qt, w).reshape(n_rows, n_cols)
    c0, cc = 2 * e, 3 * e
    t = skn.QuantTensor(ctx, (n_rows, n_cols), qt, w, shard=(4, 5, c0, cc))
    info = t.info()
    assert info["row_pitch_bytes"] % 16 == 0 and info["n_rows"] == 5 and info["n_cols"] == cc
    got = t.dequantize()
    t.close()
    assert np.array_equal(got.view(np.uint32), full[4:9, c0:c0 + cc].view(np.uint32))


def test_upload_errors(ctx):
    w = synth.make_weight(synth.rng(1), synth.Q4_K, 2, 256)
    with pytest.raises(ValueError, match="not a multiple"):
        skn.QuantTensor(ctx, (2, 250), synth.Q4_K, w)
    with pytest.raises(ValueError, match="byte length"):
        skn.QuantTensor(ctx, (3, 256), synth.Q4_K, w)
    with pytest.raises(skn.SknError) as ei:
        skn.QuantTensor(ctx, (2, 256), 16, w)   # IQ2_XXS: in the reference's table, not built here
    assert ei.value.code == 2
