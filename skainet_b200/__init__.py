"""B200 (sm_100a) backend for skainet's quantized-inference hot path.

The product is ``libskainet_cuda.so`` (C ABI in ``include/skainet_cuda.h``); this package
is the Python host-side mirror of the reference's tensor / module interface over that ABI.
"""
from .tensor import (Context, KVCache, GGML_QUANT_SIZES, GGMLQuantizationType, QK_K, QuantTensor, Shape,
                     SknError, ffn_swiglu, quant_shape_to_byte_shape)

__all__ = ["Context", "KVCache", "GGML_QUANT_SIZES", "GGMLQuantizationType", "QK_K", "QuantLinear", "QuantTensor", "Shape",
           "SknError", "ffn_swiglu", "quant_shape_to_byte_shape"]
from .llama import LlamaConfig, LlamaDecoder  # noqa: E402
from .nn import MLP, Module, QuantLinear, ReLU, load_model_weights  # noqa: E402

__all__ += ["LlamaConfig", "LlamaDecoder", "MLP", "Module", "ReLU", "load_model_weights"]
