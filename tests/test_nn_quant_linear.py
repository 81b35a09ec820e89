"""QuantLinear in the reference's `nn` style (Module + ModuleParameters with an assignable weight value) and the
loader loop of the reference's sample (samples/mnist-mlp-cli/.../Main.kt:171-242) with its quantized branch
filled in, end to end on tests/golden/quant_mlp.gguf (written by gguf-py 0.19.0, see make_gguf_fixtures.py)."""
import os

import numpy as np
import pytest

import skainet_b200 as skn
from conftest import FP32_TOL, assert_close_dot
from skainet_b200 import nn, synth
from skainet_b200.gguf import GGUFFile

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MLP_FILE = os.path.join(GOLD, "quant_mlp.gguf")
LAYERS = (("fc1", synth.Q4_K, 256, 512), ("fc2", synth.Q6_K, 256, 256), ("fc3", synth.Q8_0, 10, 256))


def build_mlp():
    return nn.MLP(nn.QuantLinear(512, 256, "fc1"), nn.ReLU(), nn.QuantLinear(256, 256, "fc2"), nn.ReLU(),
                  nn.QuantLinear(256, 10, "fc3"))


def test_module_and_parameter_surface():
    lin = nn.QuantLinear(512, 256, "fc1")
    assert isinstance(lin, nn.Module) and isinstance(lin, nn.ModuleParameters) and lin.modules == []
    assert [p.name for p in lin.params] == ["fc1.weight", "fc1.bias"]
    assert isinstance(nn.weights(lin.params), nn.WeightParameter) and isinstance(nn.bias(lin.params), nn.BiasParameter)
    assert nn.by(lin.params, "FC1.BIAS") is lin.params[1] and nn.by(lin.params, "nothing") is None
    assert isinstance(lin.weight, nn.UnsetWeight) and lin.weight.shape == skn.Shape(256, 512)
    with pytest.raises(RuntimeError, match="has not been assigned"):
        lin(np.zeros(512, dtype=np.float32))
    lin.params[1].value = np.ones(256, dtype=np.float32)          # `value` is assignable, as in the reference
    assert lin.bias[0] == 1.0
    with pytest.raises(LookupError):
        nn.weights([nn.BiasParameter("b", None)])
    mlp = build_mlp()
    assert [m.name for m in nn.find_linear_layers(mlp)] == ["fc1", "fc2", "fc3"]
    assert len(mlp.modules) == 5
    with pytest.raises(ValueError, match="Shapes do not align."):
        nn.QuantLinear(4, 4, init_bias=np.zeros(3, dtype=np.float32))


def test_fixture_has_the_sample_loaders_naming():
    with GGUFFile(MLP_FILE) as f:
        names = [t.name for t in f.tensors]
        assert names == [f"model.{n}.{k}" for n, _, _, _ in LAYERS for k in ("weight", "bias")]
        g = synth.rng(3)
        for (name, qt, n, k), w, b in zip(LAYERS, f.tensors[0::2], f.tensors[1::2]):
            raw = synth.make_weight(g, qt, n, k)                  # the generator's draw order is the file's
            assert w.tensor_type == qt and w.shape == (k, n) and np.array_equal(w.data, raw.reshape(-1))
            want_b = g.standard_normal(n).astype(np.float16 if name == "fc2" else np.float32)
            assert np.array_equal(np.asarray(b.data).reshape(-1), want_b)


@pytest.mark.gpu
def test_loader_assigns_quantized_tensors_and_the_mlp_runs(ctx):
    from oracle import oracle
    mlp = build_mlp()
    applied, skipped = nn.load_model_weights(mlp, MLP_FILE, ctx)
    assert sorted(applied) == sorted((f"model.{n}.{k}", f"{n}.{k}") for n, _, _, _ in LAYERS for k in ("weight", "bias"))
    assert skipped == []
    layers = nn.find_linear_layers(mlp)
    g = synth.rng(3)
    raws, biases = [], []
    for (name, qt, n, k), lin in zip(LAYERS, layers):
        raws.append(synth.make_weight(g, qt, n, k))
        biases.append(g.standard_normal(n).astype(np.float16 if name == "fc2" else np.float32).astype(np.float32))
        assert isinstance(lin.weight, skn.QuantTensor) and lin.weight.quant_type == qt
        assert lin.weight.shape == skn.Shape(n, k)
        # the blocks reached HBM unchanged: dequantised bit for bit
        assert np.array_equal(lin.weight.dequantize().view(np.uint32), oracle.dequant(qt, raws[-1]).reshape(n, k).view(np.uint32))
        assert np.array_equal(lin.bias, biases[-1])
    for M in (1, 5):
        x = synth.make_activations(synth.rng(40 + M), M, 512)
        xin = x[0] if M == 1 else x
        # every layer against the oracle on the layer's own input (the stated fp32 tolerance) ...
        h = xin
        for (name, qt, n, k), lin, raw, b in zip(LAYERS, layers, raws, biases):
            y = lin(h)
            ref, absdot = oracle.matmul(qt, raw, n, k, np.asarray(h).reshape(M, k))
            assert_close_dot(np.asarray(y).reshape(M, n), ref + b[None, :], absdot + np.abs(b)[None, :], FP32_TOL, f"{name} M={M}")
            h = np.maximum(y, 0) if name != "fc3" else y
        # ... and the whole network against the fp64 chain
        got = mlp(xin)
        assert np.array_equal(got, h)
        r = x.astype(np.float64)
        for (name, qt, n, k), raw, b in zip(LAYERS, raws, biases):
            W = oracle.dequant(qt, raw).reshape(n, k).astype(np.float64)
            r = r @ W.T + b
            if name != "fc3":
                r = np.maximum(r, 0)
        assert np.linalg.norm(np.asarray(got).reshape(M, 10) - r) <= 1e-4 * np.linalg.norm(r)
    # a second load replaces the device tensors (the old ones are released) and changes nothing
    nn.load_model_weights(mlp, MLP_FILE, ctx)
    assert np.array_equal(mlp(xin), got)
    # a layer of another shape refuses the tensor, as the reference's shape checks would
    wrong = nn.MLP(nn.QuantLinear(512, 128, "fc1"))
    with pytest.raises(ValueError, match="Shapes do not align."):
        nn.load_model_weights(wrong, MLP_FILE, ctx)
    for lin in layers:
        lin.weight.close()
