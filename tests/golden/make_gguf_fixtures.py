"""Writes the GGUF fixtures under tests/golden/ with gguf-py's GGUFWriter (0.19.0) and records
what gguf-py's own GGUFReader sees in them (tests/golden/gguf_expected.json).

    python tests/golden/make_gguf_fixtures.py

toy_f32.gguf       the layout of the reference's own fixture (3 string keys, three F32 3x3
                   tensors x, y, result = x + y), re-created from a seed
mixed_quant.gguf   scalar / string / array metadata of every value type, custom alignment 64,
                   and Q4_0, Q8_0, Q4_K, Q6_K, F16, F32 tensors (seeded blocks)
quant_mlp.gguf     a 512-256-256-10 MLP in the naming of the reference's sample loader ("model.<layer>.weight" /
                   "model.<layer>.bias"): Q4_K, Q6_K and Q8_0 weights, F32 and F16 biases (seeded blocks)
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from skainet_b200 import synth  # noqa: E402

import gguf  # noqa: E402
from gguf.constants import GGMLQuantizationType as T  # noqa: E402


def toy(path):
    g = synth.rng(1)
    w = gguf.GGUFWriter(path, "toy")
    w.add_string("experiment.name", "tensor addition")
    w.add_string("experiment.author", "skainet_b200 tests")
    x = g.standard_normal((3, 3)).astype(np.float32)
    y = g.standard_normal((3, 3)).astype(np.float32)
    for name, a in (("x", x), ("y", y), ("result", x + y)):
        w.add_tensor(name, a)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def mixed(path):
    g = synth.rng(2)
    w = gguf.GGUFWriter(path, "llama")
    w.add_custom_alignment(64)
    w.add_uint8("t.u8", 200)
    w.add_int8("t.i8", -5)
    w.add_uint16("t.u16", 60000)
    w.add_int16("t.i16", -1234)
    w.add_uint32("t.u32", 4000000000)
    w.add_int32("t.i32", -7)
    w.add_float32("t.f32", 1.5)
    w.add_bool("t.bool", True)
    w.add_uint64("t.u64", 2 ** 40 + 3)
    w.add_int64("t.i64", -(2 ** 41))
    w.add_float64("t.f64", 2.25)
    w.add_string("t.str", "héllo")
    w.add_array("t.arr_i32", [1, -2, 3])
    w.add_array("t.arr_f32", [0.5, 1.5])
    w.add_array("t.arr_str", ["a", "bc", ""])
    tensors = {}
    for qt, name, (n, k) in ((synth.Q4_0, "blk.q4_0", (4, 64)), (synth.Q8_0, "blk.q8_0", (3, 96)),
                             (synth.Q4_K, "blk.q4_k", (5, 512)), (synth.Q6_K, "blk.q6_k", (2, 256))):
        raw = synth.make_weight(g, qt, n, k)
        w.add_tensor(name, raw, raw_dtype=T(qt))
        tensors[name] = (qt, n, k)
    w.add_tensor("norm.f32", g.standard_normal(7).astype(np.float32))
    w.add_tensor("emb.f16", g.standard_normal((2, 6)).astype(np.float16))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


MLP_LAYERS = (("fc1", synth.Q4_K, 256, 512, np.float32), ("fc2", synth.Q6_K, 256, 256, np.float16),
              ("fc3", synth.Q8_0, 10, 256, np.float32))


def quant_mlp(path):
    g = synth.rng(3)
    w = gguf.GGUFWriter(path, "mlp")
    w.add_string("general.name", "quantized MLP fixture")
    for name, qt, n, k, bias_dtype in MLP_LAYERS:
        raw = synth.make_weight(g, qt, n, k)
        w.add_tensor(f"model.{name}.weight", raw, raw_dtype=T(qt))
        w.add_tensor(f"model.{name}.bias", g.standard_normal(n).astype(bias_dtype))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def describe(path):
    r = gguf.GGUFReader(path)
    out = {"alignment": int(r.alignment), "data_offset": int(r.data_offset), "tensors": [], "fields": {}}
    for t in r.tensors:
        out["tensors"].append({"name": t.name, "type": int(t.tensor_type), "shape": [int(d) for d in t.shape],
                               "n_elements": int(t.n_elements), "n_bytes": int(t.n_bytes),
                               "data_offset": int(t.data_offset),
                               "sha_sum": int(np.asarray(t.data).view(np.uint8).astype(np.uint64).sum())})
    for k, f in r.fields.items():
        v = f.contents()
        if isinstance(v, np.generic):
            v = v.item()
        out["fields"][k] = v
    return out


def main():
    exp = {}
    for name, fn in (("toy_f32.gguf", toy), ("mixed_quant.gguf", mixed), ("quant_mlp.gguf", quant_mlp)):
        p = os.path.join(HERE, name)
        fn(p)
        exp[name] = describe(p)
        print(name, os.path.getsize(p), "bytes,", len(exp[name]["tensors"]), "tensors")
    json.dump(exp, open(os.path.join(HERE, "gguf_expected.json"), "w"), indent=1, sort_keys=True, ensure_ascii=False)


if __name__ == "__main__":
    main()
