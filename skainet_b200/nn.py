"""Host-side mirror of the reference's `nn` style for quantized layers:

  Module            core/src/commonMain/kotlin/sk/ai/net/nn/Module.kt:6-16    (name, modules, forward, invoke)
  ModuleParameter   nn/reflection/ModuleParameters.kt:5-18   (WeightParameter / BiasParameter, `value` is assignable)
  ModuleParameters  nn/reflection/ModuleParameters.kt:20-22  (params) with the helpers by / bias / weights (:24-37)
  QuantLinear       nn/Linear.kt:22-50 with a weight parameter that holds raw GGUF blocks in HBM
  ReLU, MLP         nn/activations/ReLU.kt, nn/topology/MLP.kt:13-19 (a sequence of modules)
  load_model_weights  the loader loop of samples/mnist-mlp-cli/src/jvmMain/kotlin/sk/ai/net/samples/mnist/mlp/
                    Main.kt:171-242, whose `else ->` branch (:229-232) skips every quantized tensor; here that
                    branch uploads the raw blocks and assigns the device tensor to the parameter

The reference's Linear multiplies through `input.matmul(weight.t())`, and DoublesTensor.matmul down-casts its
right operand (impl/DoublesTensor.kt:260), so a foreign tensor class cannot be the right-hand side: the quantized
layer owns the product instead (`weight.matmul_t(x)` = x . W^T without a transposed copy).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Sequence

import numpy as np

from .gguf import GGUFFile
from .tensor import GGML_QUANT_SIZES, GGMLQuantizationType, Context, QuantTensor, Shape


class Module:
    """Module.kt:6-16."""

    name: str = "Module"

    @property
    def modules(self) -> List["Module"]:
        return []

    def forward(self, input):
        raise NotImplementedError

    def __call__(self, input):
        return self.forward(input)


@dataclass
class ModuleParameter:
    """ModuleParameters.kt:5-18: a named slot whose `value` the loader replaces."""
    name: str
    value: Any


class WeightParameter(ModuleParameter):
    pass


class BiasParameter(ModuleParameter):
    pass


class ModuleParameters:
    """ModuleParameters.kt:20-22."""
    params: List[ModuleParameter]


def by(params: Sequence[ModuleParameter], name: str) -> Optional[ModuleParameter]:
    """ModuleParameters.kt:24-25: first parameter whose name contains `name`, ignoring case."""
    for p in params:
        if name.upper() in p.name.upper():
            return p
    return None


def weights(params: Sequence[ModuleParameter]) -> WeightParameter:
    """ModuleParameters.kt:33-37."""
    for p in params:
        if isinstance(p, WeightParameter):
            return p
    raise LookupError("No weight parameter found!")


def bias(params: Sequence[ModuleParameter]) -> BiasParameter:
    """ModuleParameters.kt:27-31."""
    for p in params:
        if isinstance(p, BiasParameter):
            return p
    raise LookupError("No bias parameter found!")


class UnsetWeight:
    """Placeholder value of a weight parameter before a loader has assigned it (the reference fills a zero
    DoublesTensor, Linear.kt:26-29; a zero-filled block tensor would cost HBM for nothing)."""

    def __init__(self, shape: Shape):
        self.shape = shape

    def __repr__(self):
        return f"UnsetWeight({self.shape!r})"


class QuantLinear(Module, ModuleParameters):
    """Linear.kt:22-50: forward(x) = x . W^T + b with W [out, in] a QuantTensor (raw GGUF blocks in HBM) and b a
    host fp32 vector.  The weight may be given at construction or assigned later through `params`."""

    def __init__(self, in_features: int, out_features: int, name: str = "Linear", init_weights: Optional[QuantTensor] = None,
                 init_bias: Optional[np.ndarray] = None):
        self.in_features, self.out_features, self.name = int(in_features), int(out_features), name
        w = init_weights if init_weights is not None else UnsetWeight(Shape(out_features, in_features))
        b = np.zeros(out_features, dtype=np.float32) if init_bias is None else np.ascontiguousarray(init_bias, dtype=np.float32)
        if init_weights is not None and init_weights.shape != Shape(out_features, in_features):
            raise ValueError("Shapes do not align.")
        if b.shape != (out_features,):
            raise ValueError("Shapes do not align.")
        self.params = [WeightParameter(f"{name}.weight", w), BiasParameter(f"{name}.bias", b)]

    @classmethod
    def of(cls, weight: QuantTensor, bias: Optional[np.ndarray] = None, name: str = "Linear") -> "QuantLinear":
        out_f, in_f = weight.shape.dimensions
        return cls(in_f, out_f, name, weight, bias)

    @property
    def weight(self):
        return weights(self.params).value

    @property
    def bias(self):
        return bias(self.params).value

    def forward(self, input: np.ndarray) -> np.ndarray:
        w, b = weights(self.params).value, bias(self.params).value
        if not isinstance(w, QuantTensor):
            raise RuntimeError(f"{self.name}: the weight parameter has not been assigned a quantized tensor")
        if w.shape != Shape(self.out_features, self.in_features):
            raise ValueError("Shapes do not align.")
        return w.matmul_t(input, None if b is None else np.ascontiguousarray(b, dtype=np.float32))


class ReLU(Module):
    """nn/activations/ReLU.kt: max(x, 0) element-wise (host)."""

    def __init__(self, name: str = "ReLU"):
        self.name = name

    def forward(self, input):
        return np.maximum(np.asarray(input, dtype=np.float32), np.float32(0))


class MLP(Module):
    """nn/topology/MLP.kt:13-19: the modules applied in order."""

    def __init__(self, *modules: Module, name: str = "MLP"):
        self.name = name
        self._modules = list(modules)

    @property
    def modules(self) -> List[Module]:
        return self._modules

    def forward(self, input):
        x = input
        for m in self._modules:
            x = m.forward(x)
        return x


def find_linear_layers(module: Module) -> List[QuantLinear]:
    """Main.kt:194-203: depth-first walk collecting the linear layers."""
    found: List[QuantLinear] = []

    def walk(m: Module):
        if isinstance(m, QuantLinear):
            found.append(m)
        for child in m.modules:
            walk(child)

    walk(module)
    return found


def load_model_weights(model: Module, model_path: str, ctx: Context, prefix: str = "model."):
    """Main.kt:171-242 for quantized files: every tensor of the GGUF file whose name (without `prefix`) occurs in
    a parameter's name, ignoring case (:216-218), is assigned to that parameter.  Quantized 2-D tensors go to HBM
    unchanged and become the weight's QuantTensor (the branch the reference skips, :229-232); F32 / F16 1-D
    tensors become fp32 bias vectors (:221-228).  A tensor whose shape does not fit the parameter raises
    ValueError("Shapes do not align.").  Returns (applied, skipped): lists of (tensor name, parameter name) and
    of (tensor name, reason)."""
    layers = find_linear_layers(model)
    applied, skipped = [], []
    with GGUFFile(model_path) as f:
        for t in f.tensors:
            name = t.name[len(prefix):] if t.name.startswith(prefix) else t.name
            hit = False
            for layer in layers:
                for p in layer.params:
                    if name.upper() not in p.name.upper():
                        continue
                    hit = True
                    quantized = t.tensor_type in {int(q) for q in GGML_QUANT_SIZES}
                    if isinstance(p, WeightParameter):
                        if not quantized:
                            skipped.append((t.name, f"{p.name}: weight of type {t.tensor_type} is not a block-quantized tensor"))
                            continue
                        want = Shape(layer.out_features, layer.in_features)
                        if len(t.shape) != 2 or Shape(t.shape[1], t.shape[0]) != want:
                            raise ValueError("Shapes do not align.")
                        old = p.value
                        p.value = f.upload(ctx, t)
                        if isinstance(old, QuantTensor):
                            old.close()
                    else:
                        if t.tensor_type not in (0, 1):          # F32, F16 (the reader hands both out as arrays)
                            skipped.append((t.name, f"{p.name}: bias of type {t.tensor_type} is not F32 / F16"))
                            continue
                        v = np.array(t.data, dtype=np.float32).reshape(-1)
                        if v.shape != (layer.out_features,):
                            raise ValueError("Shapes do not align.")
                        p.value = v
                    applied.append((t.name, p.name))
            if not hit:
                skipped.append((t.name, "no parameter of this name"))
    return applied, skipped


__all__ = ["Module", "ModuleParameter", "WeightParameter", "BiasParameter", "ModuleParameters", "by", "weights", "bias",
           "QuantLinear", "ReLU", "MLP", "UnsetWeight", "find_linear_layers", "load_model_weights", "GGMLQuantizationType"]
