"""The memory-mapped GGUF reader against fixtures written by gguf-py 0.19.0 and what gguf-py's
own reader sees in them (tests/golden/gguf_expected.json, tests/golden/make_gguf_fixtures.py).
CPU only: parsing needs no GPU.  The toy file has the layout of the reference's own fixture
(gguf/src/jvmTest/resources/test_experiment.gguf: string keys + three F32 3x3 tensors with
result = x + y), which GGUFReaderTest.kt:45-81 only prints."""
import json
import os

import numpy as np
import pytest

import skainet_b200 as skn
from skainet_b200.gguf import GGUFFile

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
EXPECTED = json.load(open(os.path.join(GOLD, "gguf_expected.json")))


@pytest.mark.parametrize("name", ["toy_f32.gguf", "mixed_quant.gguf", "quant_mlp.gguf"])
def test_matches_gguf_py(name):
    exp = EXPECTED[name]
    with GGUFFile(os.path.join(GOLD, name)) as f:
        assert f.version == 3 and f.alignment == exp["alignment"] and f.data_offset == exp["data_offset"]
        assert len(f.tensors) == len(exp["tensors"])
        for t, e in zip(f.tensors, exp["tensors"]):
            assert (t.name, t.tensor_type, list(t.shape), t.n_elements, t.n_bytes, t.data_offset) == \
                   (e["name"], e["type"], e["shape"], e["n_elements"], e["n_bytes"], e["data_offset"])
            assert int(np.asarray(t.data).view(np.uint8).astype(np.uint64).sum()) == e["sha_sum"]
        for k, v in exp["fields"].items():
            if k.startswith("GGUF."):
                continue                      # gguf-py's synthetic header fields
            got = f.fields[k]
            if isinstance(v, list):
                assert list(np.asarray(got).tolist() if not isinstance(got, list) else got) == v, k
            elif isinstance(v, float):
                assert got == pytest.approx(v), k
            else:
                assert got == v, k
        assert set(f.fields) == {k for k in exp["fields"] if not k.startswith("GGUF.")}


def test_toy_file_contents():
    with GGUFFile(os.path.join(GOLD, "toy_f32.gguf")) as f:
        t = {x.name: x for x in f.tensors}
        assert set(t) == {"x", "y", "result"}
        assert all(v.tensor_type == 0 and v.shape == (3, 3) for v in t.values())
        np.testing.assert_array_equal(t["x"].data + t["y"].data, t["result"].data)
        assert f.fields["experiment.name"] == "tensor addition"


def test_quantized_tensors_are_raw_blocks_and_f16_is_supported():
    from oracle import oracle
    from skainet_b200 import synth
    with GGUFFile(os.path.join(GOLD, "mixed_quant.gguf")) as f:
        t = {x.name: x for x in f.tensors}
        g = synth.rng(2)
        for qt, name, (n, k) in ((synth.Q4_0, "blk.q4_0", (4, 64)), (synth.Q8_0, "blk.q8_0", (3, 96)),
                                 (synth.Q4_K, "blk.q4_k", (5, 512)), (synth.Q6_K, "blk.q6_k", (2, 256))):
            raw = synth.make_weight(g, qt, n, k)                       # the generator's draw order is the file's
            assert t[name].shape == (k, n) and t[name].tensor_type == qt
            assert t[name].n_bytes == n * oracle.row_bytes(qt, k)
            np.testing.assert_array_equal(t[name].data, raw.reshape(-1))
        assert t["emb.f16"].data.dtype == np.float16 and t["emb.f16"].data.shape == (2, 6)   # the reference throws here
        assert t["norm.f32"].data.shape == (7,)


def test_errors(tmp_path):
    with pytest.raises(skn.SknError, match="cannot open"):
        GGUFFile(str(tmp_path / "missing.gguf"))
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"NOPE" + bytes(40))
    with pytest.raises(skn.SknError, match="magic"):
        GGUFFile(str(bad))
    good = open(os.path.join(GOLD, "mixed_quant.gguf"), "rb").read()
    v9 = tmp_path / "v9.gguf"
    v9.write_bytes(good[:4] + (9).to_bytes(4, "little") + good[8:])
    with pytest.raises(skn.SknError, match="version 9"):
        GGUFFile(str(v9))
    # header counts the file cannot hold are refused before anything is reserved for them
    huge = tmp_path / "huge.gguf"
    huge.write_bytes(good[:8] + (len(good)).to_bytes(8, "little") + good[16:])
    with pytest.raises(skn.SknError, match="corrupt header counts"):
        GGUFFile(str(huge))
    # a tensor whose data offset is off the file's alignment (64 here): the offset field of the first tensor record
    first = good.index(b"blk.q4_0")
    off_pos = first + len(b"blk.q4_0") + 4 + 2 * 8 + 4          # name, rank, two dims, type -> offset
    assert int.from_bytes(good[off_pos:off_pos + 8], "little") == 0
    mis = tmp_path / "misaligned.gguf"
    mis.write_bytes(good[:off_pos] + (8).to_bytes(8, "little") + good[off_pos + 8:])
    with pytest.raises(skn.SknError, match="not a multiple of the alignment"):
        GGUFFile(str(mis))
    for cut in (30, 200, len(good) - 100):          # truncated metadata / truncated tensor data
        tr = tmp_path / f"cut{cut}.gguf"
        tr.write_bytes(good[:cut])
        with pytest.raises((skn.SknError, ValueError)):
            GGUFFile(str(tr))


@pytest.mark.gpu
def test_upload_from_mapping_dequantises_exactly(ctx):
    from oracle import oracle
    with GGUFFile(os.path.join(GOLD, "mixed_quant.gguf")) as f:
        for t in f.tensors:
            if t.tensor_type not in (2, 8, 12, 14):
                with pytest.raises((skn.SknError, ValueError)):
                    f.upload(ctx, t)
                continue
            q = f.upload(ctx, t)
            got = q.dequantize()
            ref = oracle.dequant(t.tensor_type, np.array(t.data)).reshape(t.shape[1], t.shape[0])
            assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
            q.close()
