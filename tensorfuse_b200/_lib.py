"""ctypes binding of libtensorfuse.so.

The shared library is the product; this module only declares its C ABI to
Python.  There is no fallback of any kind: if the library has not been built,
importing this module raises, and every operator either launches CUDA kernels
through the library or raises the library's error.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# TENSORFUSE_B200_LIB selects another build of the same library (e.g. one
# compiled with different tuning constants); it is never a different backend.
LIB_PATH = os.environ.get("TENSORFUSE_B200_LIB") or os.path.join(_PKG, "lib", "libtensorfuse.so")

MAX_DIMS = 8


class Shape(C.Structure):
    _fields_ = [("ndims", C.c_int), ("dims", C.c_int * MAX_DIMS), ("strides", C.c_int * MAX_DIMS)]


class Tensor(C.Structure):
    """TensorFuseTensor (include/tensorfuse/types.h)."""
    _fields_ = [("data", C.c_void_p), ("shape", Shape), ("dtype", C.c_int), ("layout", C.c_int),
                ("device_id", C.c_int), ("size_bytes", C.c_size_t), ("is_contiguous", C.c_bool),
                ("scale", C.c_void_p), ("zero_point", C.c_void_p)]


class TransformerParams(C.Structure):
    """TensorFuseTransformerParams (include/tensorfuse/types.h)."""
    _fields_ = [(n, C.POINTER(Tensor)) for n in (
        "query_weight", "key_weight", "value_weight", "output_weight",
        "query_bias", "key_bias", "value_bias", "output_bias",
        "ffn_weight1", "ffn_weight2", "ffn_bias1", "ffn_bias2",
        "ln1_weight", "ln1_bias", "ln2_weight", "ln2_bias")] + [
        ("num_heads", C.c_int), ("dropout_prob", C.c_float), ("ffn_activation", C.c_int),
        ("layer_norm_eps", C.c_float), ("use_bias", C.c_bool), ("use_flash_attention", C.c_bool)]


class Config(C.Structure):
    """TensorFuseConfig (include/tensorfuse/types.h)."""
    _fields_ = [("device_count", C.c_int), ("device_ids", C.POINTER(C.c_int)),
                ("workspace_size_bytes", C.c_size_t), ("enable_profiling", C.c_bool),
                ("enable_autotuning", C.c_bool), ("enable_fp8", C.c_bool), ("log_level", C.c_int),
                ("cache_dir", C.c_char_p)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python tensorfuse_b200/build.py` "
            "(needs nvcc; there is no CPU or PyTorch fallback)")
    L = C.CDLL(LIB_PATH)
    vp, i, f, ll, ull, st = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_ulonglong, C.c_void_p
    TP = C.POINTER(Tensor)

    def sig(name, res, args):
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args

    sig("tensorfuse_init", i, [C.POINTER(Config)])
    sig("tensorfuse_shutdown", i, [])
    sig("tensorfuse_cleanup", i, [])
    sig("tensorfuse_get_version", C.c_char_p, [])
    sig("tensorfuse_get_error_string", C.c_char_p, [i])
    sig("tensorfuse_fused_gemm_bias_gelu", i, [TP, TP, TP, TP, st])
    sig("tensorfuse_fused_softmax_dropout", i, [TP, TP, vp, f, st])
    sig("tensorfuse_fused_multi_head_attention", i, [TP, TP, TP, TP, i, f, st])
    sig("tensorfuse_fused_transformer_layer", i, [TP, TP, vp, st])
    sig("tensorfuse_autotune", i, [vp, C.c_char_p])
    sig("tensorfuse_load_tuned_config", i, [C.c_char_p])
    sig("tensorfuse_start_profiling", i, [vp])
    sig("tensorfuse_stop_profiling", i, [C.c_char_p])
    sig("tensorfuse_allocate_tensor", i, [TP, C.POINTER(Shape), i, i])
    sig("tensorfuse_free_tensor", i, [TP])
    gemm = [vp, vp, vp, vp, i, i, i, f, f, st]
    for n in ("fused_gemm_bias_gelu_fp32_wrapper", "fused_gemm_bias_gelu_fp16_wrapper",
              "optimized_fused_gemm_bias_gelu_fp32_wrapper",
              "optimized_fused_gemm_bias_gelu_fp16_wrapper", "fused_gemm_bias_gelu_int8_wrapper"):
        sig(n, i, gemm)
    sig("fused_gemm_bias_gelu_int8_wrapper_with_scales", i, [vp, vp, vp, vp, i, i, i, f, f, f, f, st])
    sm = [vp, vp, vp, i, i, i, i, f, ull, st]
    sig("fused_softmax_dropout_fp16_wrapper", i, sm)
    sig("fused_softmax_dropout_fp32_wrapper", i, sm)
    sig("tensorfuse_b200_gemm_int8", i, [vp, vp, vp, vp, i, i, i, f, f, i, i, i, st])
    sig("tensorfuse_b200_gemm_fp8", i, [vp, vp, vp, vp, i, i, i, f, f, i, i, st])
    sig("tensorfuse_b200_gemm_bias_act", i, [vp, vp, vp, vp, i, i, i, i, i, f, f, st])
    sig("tensorfuse_b200_softmax_dropout_masked", i, [vp, vp, vp, ll, ll, i, i, f, vp, f, ull, st])
    sig("tensorfuse_b200_add_layernorm", i, [vp, vp, vp, vp, vp, ll, i, i, f, st])
    sig("tensorfuse_b200_quantize_int8_columns", i, [vp, i, i, i, vp, vp, st])
    sig("tensorfuse_b200_gemm_int8_channelwise", i, [vp, vp, vp, vp, i, i, i, vp, vp, i, i, st])
    sig("tensorfuse_b200_quantize_int8", i, [vp, i, ll, vp, vp, st])
    sig("tensorfuse_b200_attention", i, [vp, vp, vp, vp, i, i, i, i, i] + [ll] * 12 + [i, f, f, ull, vp, st])
    sig("tensorfuse_b200_softmax_dropout_rows", i, [vp, vp, vp, ll, i, i, f, ull, ull, st])
    sig("tensorfuse_b200_softmax_schedule", None, [i, i, i, C.POINTER(i), C.POINTER(i)])
    sig("tensorfuse_b200_softmax_schedule_ex", None, [i, i, i, C.POINTER(i), C.POINTER(i), C.POINTER(i)])
    sig("tensorfuse_b200_set_random_seed", None, [ull])
    sig("tensorfuse_b200_last_softmax_seed", ull, [])
    sig("tensorfuse_b200_gemm_bias_gelu_host", i, [vp, vp, vp, vp, i, i, i, i, i, i, i, f, f])
    sig("tensorfuse_b200_softmax_dropout_host", i, [vp, vp, vp, ll, i, i, f, ull])
    sig("tensorfuse_b200_softmax_dropout_host_noalloc", i, [vp, vp, vp, ll, i, i, f, ull, st])
    sig("tensorfuse_b200_register_weights", i, [vp, C.c_size_t])
    sig("tensorfuse_b200_invalidate_weights", i, [vp])
    sig("tensorfuse_simple_init", i, [i])
    sig("tensorfuse_simple_cleanup", None, [])
    sig("tensorfuse_b200_memcpy", i, [vp, vp, C.c_size_t, i])
    sig("tensorfuse_b200_mem_info", i, [i, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)])
    sig("tensorfuse_b200_device_info", i, [i, C.c_char_p, i, C.POINTER(i), C.POINTER(i), C.POINTER(C.c_size_t),
                                           C.POINTER(i)])
    sig("tensorfuse_b200_alloc_pinned", vp, [C.c_size_t])
    sig("tensorfuse_b200_free_pinned", None, [vp])
    sig("tensorfuse_b200_plan_shards", None, [ll, i, i, C.POINTER(ll), C.POINTER(ll)])
    sig("tensorfuse_b200_device_count", i, [])
    sig("tensorfuse_b200_device_id", i, [i])
    sig("tensorfuse_b200_watchdog_status", i, [])
    sig("tensorfuse_b200_watchdog_reset", None, [])
    sig("tensorfuse_b200_launch_count", ull, [])
    return L


lib = _load()
