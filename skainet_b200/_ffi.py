"""ctypes binding of libskainet_cuda.so -- the same C ABI a Kotlin/JVM host binds through
FFM or JNI.  Signatures are parsed from nothing: they are written out here and checked
against include/skainet_cuda.h by the test-suite (every declared symbol must be exported).

The library is required: there is no Python or CPU fallback for any compute entry point.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# SKAINET_CUDA_LIB points at an alternative build of the same library (e.g. a debug build)
LIB_PATH = os.environ.get("SKAINET_CUDA_LIB") or os.path.join(_HERE, "libskainet_cuda.so")

c_i32, c_i64, c_vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p
P = ctypes.POINTER

# name -> (restype, argtypes)
SIGNATURES = {
    "skn_version": (c_i32, []),
    "skn_last_error": (ctypes.c_char_p, [c_vp]),
    "skn_ctx_create": (c_i32, [c_i32, P(c_vp)]),
    "skn_ctx_destroy": (c_i32, [c_vp]),
    "skn_ctx_set_stream": (c_i32, [c_vp, c_vp]),
    "skn_ctx_set_option": (c_i32, [c_vp, c_i32, c_i64]),
    "skn_sync": (c_i32, [c_vp]),
    "skn_quant_geometry": (c_i32, [c_i32, P(c_i32), P(c_i32)]),
    "skn_quant_row_bytes": (c_i32, [c_i32, c_i64, P(c_i64)]),
    "skn_tensor_upload_quant": (c_i32, [c_vp, c_i32, c_i64, c_i64, c_vp, c_i64, P(c_vp)]),
    "skn_tensor_upload_quant_shard": (c_i32, [c_vp, c_i32, c_i64, c_i64, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64,
                                              P(c_vp)]),
    "skn_tensor_destroy": (c_i32, [c_vp]),
    "skn_tensor_info": (c_i32, [c_vp, P(c_i32), P(c_i64), P(c_i64), P(c_i64), P(c_i64), P(c_vp)]),
    "skn_dequantize": (c_i32, [c_vp, c_vp, c_vp]),
    "skn_dequantize_dev": (c_i32, [c_vp, c_vp, c_vp]),
    "skn_matmul": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp, c_vp]),
    "skn_matmul_async": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp, c_vp]),
    "skn_matmul_dev": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i64, c_vp, c_vp]),
    "skn_rows_plan_query": (c_i32, [c_i32, c_i32, c_i64, c_i64, c_i32, c_i32, P(c_i64)]),
    "skn_matvec_group_dev": (c_i32, [c_vp, c_i32, c_vp, c_vp, c_vp, c_vp]),
    "skn_matvec_fused_dev": (c_i32, [c_vp, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, ctypes.c_float, c_vp]),
    "skn_ffn_swiglu": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_vp]),
    "skn_ffn_swiglu_dev": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_vp]),
    "skn_kv_create": (c_i32, [c_vp, c_i32, c_i32, c_i32, c_i32, P(c_vp)]),
    "skn_kv_create_typed": (c_i32, [c_vp, c_i32, c_i32, c_i32, c_i32, c_i32, P(c_vp)]),
    "skn_kv_dtype": (c_i32, [c_vp, P(c_i32)]),
    "skn_kv_destroy": (c_i32, [c_vp]),
    "skn_kv_reset": (c_i32, [c_vp]),
    "skn_kv_load": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_vp]),
    "skn_kv_lengths": (c_i32, [c_vp, c_vp, c_vp]),
    "skn_kv_append": (c_i32, [c_vp, c_vp, c_vp]),
    "skn_kv_append_dev": (c_i32, [c_vp, c_vp, c_vp]),
    "skn_kv_gather": (c_i32, [c_vp, c_i32, c_i32, c_i32, c_vp, c_vp]),
    "skn_kv_info": (c_i32, [c_vp, P(c_i32), P(c_i32), P(c_i32), P(c_i32), P(c_vp), P(c_vp), P(c_vp), P(c_vp)]),
    "skn_attn_decode": (c_i32, [c_vp, c_vp, c_i32, ctypes.c_float, c_vp]),
    "skn_attn_decode_dev": (c_i32, [c_vp, c_vp, c_i32, ctypes.c_float, c_vp, c_vp]),
    "skn_attn_scratch_bytes": (c_i64, [c_vp, c_i32]),
    "skn_kv_append_many_dev": (c_i32, [c_vp, c_vp, c_vp, c_i32, c_i32]),
    "skn_attn_causal_dev": (c_i32, [c_vp, c_vp, c_i32, c_i32, ctypes.c_float, c_vp, c_vp]),
    "skn_comm_create": (c_i32, [c_vp, c_i32, c_i32, c_i64, P(c_vp)]),
    "skn_comm_destroy": (c_i32, [c_vp]),
    "skn_comm_handle_bytes": (c_i32, []),
    "skn_comm_handle": (c_i32, [c_vp, c_vp]),
    "skn_comm_connect": (c_i32, [c_vp, c_vp]),
    "skn_comm_connect_local": (c_i32, [c_vp, c_i32]),
    "skn_comm_info": (c_i32, [c_vp, c_vp, c_vp, c_vp]),
    "skn_allreduce_dev": (c_i32, [c_vp, c_vp, c_vp, c_vp, c_i64]),
    "skn_llama_create_tp": (c_i32, [c_vp, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, ctypes.c_float, ctypes.c_float,
                                    c_i32, c_i32, c_i32, c_vp, P(c_vp)]),
    "skn_llama_create": (c_i32, [c_vp, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, ctypes.c_float, ctypes.c_float,
                                 c_i32, c_i32, c_i32, P(c_vp)]),
    "skn_llama_destroy": (c_i32, [c_vp]),
    "skn_llama_set_layer": (c_i32, [c_vp, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "skn_llama_set_head": (c_i32, [c_vp, c_vp, c_vp, c_vp]),
    "skn_llama_reset": (c_i32, [c_vp]),
    "skn_llama_forward": (c_i32, [c_vp, c_vp, c_i32, c_vp, c_vp]),
    "skn_llama_forward_dev": (c_i32, [c_vp, c_vp, c_i32]),
    "skn_llama_position": (c_i32, [c_vp]),
    "skn_gguf_open": (c_i32, [ctypes.c_char_p, P(c_vp)]),
    "skn_gguf_close": (c_i32, [c_vp]),
    "skn_gguf_counts": (c_i32, [c_vp, P(c_i32), P(c_i64), P(c_i64), P(c_i64), P(c_i64)]),
    "skn_gguf_kv": (c_i32, [c_vp, c_i64, P(ctypes.c_char_p), P(c_i32), P(c_i32), P(c_vp), P(c_i64)]),
    "skn_gguf_tensor": (c_i32, [c_vp, c_i64, P(ctypes.c_char_p), P(c_i32), P(c_i64), P(c_i32), P(c_i64), P(c_i64), P(c_vp)]),
    "skn_gguf_find_tensor": (c_i32, [c_vp, ctypes.c_char_p, P(c_i64)]),
    "skn_gguf_upload": (c_i32, [c_vp, c_vp, c_i64, P(c_vp)]),
    "skn_attn_decode_noalloc_dev": (c_i32, [c_vp, c_vp, c_i32, ctypes.c_float, c_vp]),
}

_lib = None


class LibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Load the shared library (once).  Raises LibraryMissing if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} is missing: build it with `python -m skainet_b200.build` "
                "(there is no fallback implementation)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib
