"""tensorfuse -- drop-in Python package over libtensorfuse.so (B200 build).

Takes the place of the reference's ``tensorfuse`` package
(reference ``src/python/tensorfuse/{__init__,core,memory,profiler,utils}.py``):
the same module-level names, the same ``tensorfuse._tensorfuse`` sub-module
(reference ``src/python/tensorfuse_python.cpp:26``; here
``tensorfuse_b200/_tensorfuse.py`` over ctypes), the same operator signatures,
automatic initialisation and error texts.

    import tensorfuse, numpy as np
    tensorfuse.init()
    y = tensorfuse.fused_gemm_bias_gelu(x, w, b)          # numpy in, numpy out
    tensorfuse.fused_softmax_dropout(s, out, mask, 0.1)   # fills out and mask

numpy arrays live in host memory and run through the library's host-buffer
operators; torch CUDA tensors are used in place on torch's current stream.
There is no CPU path: without the built library the import fails.

The reference's performance-analysis helpers return fixed numbers
(``__init__.py:275-391``); they are kept, with the same numbers, only so that
code written against them keeps running.
"""
from __future__ import annotations

import atexit
import sys

import numpy as np

import tensorfuse_b200 as _b200
from tensorfuse_b200 import _tensorfuse

sys.modules.setdefault(__name__ + "._tensorfuse", _tensorfuse)

try:
    import torch
    TORCH_AVAILABLE = True
except ImportError:  # pragma: no cover
    torch = None
    TORCH_AVAILABLE = False

__version__ = "1.0.0"
TENSORFUSE_MAX_DIMS = 8

# ---- names the reference package lifts out of _tensorfuse (__init__.py:53-95)
Status = _tensorfuse.Status
DataType = _tensorfuse.DataType
Layout = _tensorfuse.Layout
Shape = _tensorfuse.Shape
Config = _tensorfuse.Config
Tensor = _tensorfuse.Tensor
ProfileConfig = _tensorfuse.ProfileConfig
Metrics = _tensorfuse.Metrics
shutdown = _tensorfuse.shutdown
get_version = _tensorfuse.get_version
get_error_string = _tensorfuse.get_error_string
autotune = _tensorfuse.autotune
load_tuned_config = _tensorfuse.load_tuned_config
is_gpu_supported = _tensorfuse.is_gpu_supported
set_random_seed = _tensorfuse.set_random_seed
allocate_tensor = _tensorfuse.allocate_tensor
free_tensor = _tensorfuse.free_tensor
get_memory_info = _tensorfuse.get_memory_info
get_tensor_size_bytes = _tensorfuse.get_tensor_size_bytes
start_profiling = _tensorfuse.start_profiling
stop_profiling = _tensorfuse.stop_profiling
get_last_metrics = _tensorfuse.get_last_metrics
create_tensor = _tensorfuse.create_tensor
from_numpy = _tensorfuse.from_numpy
to_numpy = _tensorfuse.to_numpy
create_tensor_from_numpy = from_numpy
deallocate_tensor = free_tensor
TensorFuseStatus = Status
TensorFuseDataType = DataType
TensorFuseConfig = Config

# aliases the reference adds by assignment (__init__.py:111-129)
for _name, _member in (("FP32", "FLOAT32"), ("FP16", "FLOAT16"), ("BF16", "BFLOAT16")):
    if not hasattr(DataType, _name):
        setattr(DataType, _name, getattr(DataType, _member))
for _member in ("INVALID_ARGUMENT", "CUDA_ERROR", "OUT_OF_MEMORY", "NOT_INITIALIZED"):
    if not hasattr(Status, "ERROR_" + _member):
        setattr(Status, "ERROR_" + _member, getattr(Status, _member))

_is_initialized = False


def init(config=None):
    """Initialise the library (idempotent).  ``config`` is a ``Config``; its
    ``device_ids`` list selects the GPUs that rows are sharded over."""
    global _is_initialized
    _tensorfuse.init(config) if config is not None else _tensorfuse.init()
    _is_initialized = True


initialize = init


def is_initialized() -> bool:
    return _is_initialized


def get_default_config():
    return Config()


def cleanup():
    global _is_initialized
    if _is_initialized:
        shutdown()
        _is_initialized = False


atexit.register(cleanup)


def _with_init(fn, *args, **kwargs):
    """Retry once after init() when the library reports that it is not
    initialised (reference __init__.py:151-162)."""
    try:
        return fn(*args, **kwargs)
    except RuntimeError as e:
        if "Library not initialized" not in str(e):
            raise
        init()
        return fn(*args, **kwargs)


def _is_torch(x) -> bool:
    return TORCH_AVAILABLE and isinstance(x, torch.Tensor)


# ------------------------------------------------------------- operators
def fused_gemm_bias_gelu(input_tensor, weight, bias, output=None, stream=None):
    """output = GELU(input @ weight + bias); ``output`` is allocated when not given
    (reference __init__.py:134-198).  2-D or ``[batch, seq, hidden]`` input."""
    if _is_torch(input_tensor):
        if input_tensor.is_cuda:
            return _b200.fused_gemm_bias_gelu(input_tensor, weight, bias, output, stream)
        a, w, b = (t.detach().cpu().numpy() for t in (input_tensor, weight, bias))
        if output is not None:
            o = output.detach().cpu().numpy()
            _with_init(_tensorfuse.fused_gemm_bias_gelu, a, w, b, o, stream)
            output.data.copy_(torch.from_numpy(o))
            return output
        return torch.from_numpy(fused_gemm_bias_gelu(a, w, b, None, stream))
    if output is not None:
        return _with_init(_tensorfuse.fused_gemm_bias_gelu, input_tensor, weight, bias, output, stream)
    out = np.zeros(tuple(input_tensor.shape[:-1]) + (weight.shape[1],),
                   dtype=np.float32 if input_tensor.dtype == np.int8 else input_tensor.dtype)
    _with_init(_tensorfuse.fused_gemm_bias_gelu, input_tensor, weight, bias, out, stream)
    return out


def fused_softmax_dropout(input, output, dropout_mask, dropout_prob, stream=None):
    """Fills ``output`` and ``dropout_mask`` (reference core_bindings.cpp:635-771)."""
    if _is_torch(input) and input.is_cuda:
        _b200.fused_softmax_dropout(input, output, dropout_mask, dropout_prob, stream)
        return None
    return _with_init(_tensorfuse.fused_softmax_dropout, input, output, dropout_mask, dropout_prob, stream)


def fused_multi_head_attention(query, key, value, output, num_heads, dropout_prob, stream=None):
    """Fills ``output`` ``[batch, seq, hidden]`` (reference core_bindings.cpp:773-798)."""
    if _is_torch(query) and query.is_cuda:
        _b200.fused_multi_head_attention(query, key, value, output, num_heads, dropout_prob, stream)
        return None
    return _with_init(_tensorfuse.fused_multi_head_attention, query, key, value, output, num_heads, dropout_prob,
                      stream)


def fused_gemm_bias_gelu_int8(A, B, bias, alpha=1.0, beta=0.0):
    """INT8 operands on the INT8 tensor cores (the reference de-quantises to FP32
    on the host and calls the FP32 kernel instead, __init__.py:239-246)."""
    return fused_gemm_bias_gelu(np.ascontiguousarray(A, dtype=np.int8), np.ascontiguousarray(B, dtype=np.int8),
                                np.ascontiguousarray(bias, dtype=np.float32))


def get_device_info(device_id=0):
    return _tensorfuse.get_device_info()


def get_device_name(device_id=0):
    try:
        return get_device_info(device_id).get("name", "NVIDIA GPU")
    except RuntimeError:
        return "NVIDIA GPU"


def create_tensor_from_torch(torch_tensor):
    if not TORCH_AVAILABLE:
        raise ImportError("PyTorch not available")
    if torch_tensor.dtype == torch.bfloat16:
        torch_tensor = torch_tensor.to(torch.float16)
    return from_numpy(torch_tensor.detach().cpu().numpy())


# ------------------------------------------- core.py: operator objects
def convert_torch_to_numpy(tensor):
    if _is_torch(tensor):
        return tensor.detach().cpu().numpy()
    return tensor


def convert_numpy_to_torch(array, device="cuda"):
    if not TORCH_AVAILABLE:
        raise ImportError("PyTorch not available")
    return torch.from_numpy(array).to(device)


class TensorFuseOp:
    """reference core.py:17-33"""

    def __init__(self, name):
        self.name = name
        self.metrics = None

    def __call__(self, *args, **kwargs):
        raise NotImplementedError("Subclasses must implement __call__")

    def get_metrics(self):
        return self.metrics


_ModuleBase = torch.nn.Module if TORCH_AVAILABLE else object


class FusedGemmBiasGelu(_ModuleBase):
    """reference core.py:36-125.  With m, n, k given it owns ``weight`` [k, n] and
    ``bias`` [n] parameters; torch CUDA tensors run in place, anything else is
    staged through the host-buffer operator."""

    def __init__(self, m=None, n=None, k=None, dtype=None, enable_profiling=False):
        super().__init__()
        self.m, self.n, self.k, self.dtype = m, n, k, dtype
        self.enable_profiling = enable_profiling
        self.metrics = None
        if TORCH_AVAILABLE and m and n and k:
            self.weight = torch.nn.Parameter(torch.randn(k, n))
            self.bias = torch.nn.Parameter(torch.randn(n))

    def forward(self, input_tensor, weight=None, bias=None):
        if weight is None and hasattr(self, "weight"):
            weight = self.weight.detach()
        if bias is None and hasattr(self, "bias"):
            bias = self.bias.detach()
        return self.__call__(input_tensor, weight, bias)

    def __call__(self, input_tensor, weight=None, bias=None, output=None, stream=None):
        if weight is None or bias is None:
            return self.forward(input_tensor, weight, bias)
        if _is_torch(input_tensor) and not input_tensor.is_cuda:
            device = input_tensor.device
            res = fused_gemm_bias_gelu(convert_torch_to_numpy(input_tensor), convert_torch_to_numpy(weight),
                                       convert_torch_to_numpy(bias),
                                       None if output is None else convert_torch_to_numpy(output), stream)
            return convert_numpy_to_torch(res, device)
        if _is_torch(input_tensor):
            weight, bias = (t.to(input_tensor.device, input_tensor.dtype) if _is_torch(t)
                            else torch.as_tensor(t, device=input_tensor.device, dtype=input_tensor.dtype)
                            for t in (weight, bias))
        return fused_gemm_bias_gelu(input_tensor, weight, bias, output, stream)

    def get_metrics(self):
        return self.metrics


class FusedSoftmaxDropout(TensorFuseOp):
    """reference core.py:206-262: returns ``(output, dropout_mask)``."""

    def __init__(self, enable_profiling=False):
        super().__init__("fused_softmax_dropout")
        self.enable_profiling = enable_profiling

    def __call__(self, input_tensor, dropout_prob=0.1, output=None, dropout_mask=None, stream=None):
        if _is_torch(input_tensor) and input_tensor.is_cuda:
            return _b200.fused_softmax_dropout(input_tensor, output, dropout_mask, dropout_prob, stream)
        was_torch = _is_torch(input_tensor)
        x = convert_torch_to_numpy(input_tensor)
        out = np.zeros_like(x) if output is None else convert_torch_to_numpy(output)
        mask = np.zeros(x.shape, dtype=np.uint8) if dropout_mask is None else convert_torch_to_numpy(dropout_mask)
        fused_softmax_dropout(x, out, mask, dropout_prob, stream)
        if was_torch:
            return torch.from_numpy(out), torch.from_numpy(mask)
        return out, mask


class FusedMultiHeadAttention(TensorFuseOp):
    """reference core.py:264-322: returns the attention output."""

    def __init__(self, num_heads, enable_profiling=False):
        super().__init__("fused_multi_head_attention")
        self.num_heads = num_heads
        self.enable_profiling = enable_profiling

    def __call__(self, query, key, value, dropout_prob=0.1, output=None, stream=None):
        if _is_torch(query) and query.is_cuda:
            return _b200.fused_multi_head_attention(query, key, value, output, self.num_heads, dropout_prob, stream)
        was_torch = _is_torch(query)
        q, k, v = (convert_torch_to_numpy(t) for t in (query, key, value))
        out = np.zeros_like(q) if output is None else convert_torch_to_numpy(output)
        fused_multi_head_attention(q, k, v, out, self.num_heads, dropout_prob, stream)
        return torch.from_numpy(out) if was_torch else out


def gemm_bias_gelu(input_tensor, weight, bias, output=None, stream=None):
    return FusedGemmBiasGelu()(input_tensor, weight, bias, output, stream)


def softmax_dropout(input_tensor, dropout_prob=0.1, output=None, dropout_mask=None, stream=None):
    return FusedSoftmaxDropout()(input_tensor, dropout_prob, output, dropout_mask, stream)


def multi_head_attention(query, key, value, num_heads, dropout_prob=0.1, output=None, stream=None):
    return FusedMultiHeadAttention(num_heads)(query, key, value, dropout_prob, output, stream)


# ------------------------------------------------ utils.py: type helpers
def get_dtype_size(dtype) -> int:
    try:
        return _tensorfuse.get_dtype_size(dtype)
    except (TypeError, ValueError):
        return int(np.dtype(dtype).itemsize)


def numpy_dtype_to_tensorfuse(np_dtype):
    table = {np.dtype(np.float32): DataType.FLOAT32, np.dtype(np.float16): DataType.FLOAT16,
             np.dtype(np.int8): DataType.INT8, np.dtype(np.uint8): DataType.UINT8,
             np.dtype(np.int32): DataType.INT32}
    try:
        return table[np.dtype(np_dtype)]
    except KeyError:
        raise ValueError(f"Unsupported numpy dtype: {np_dtype}") from None


def calculate_tensor_size(shape, dtype) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n * get_dtype_size(dtype)


def validate_shape(shape) -> bool:
    try:
        return 0 < len(shape) <= TENSORFUSE_MAX_DIMS and all(int(d) > 0 for d in shape)
    except TypeError:
        return False


def format_bytes(bytes_val: int) -> str:
    v = float(bytes_val)
    for unit in ("B", "KB", "MB", "GB", "TB"):
        if v < 1024.0 or unit == "TB":
            return f"{v:.1f} {unit}"
        v /= 1024.0
    return f"{v:.1f} TB"


# ---------------------------------------- profiler.py / memory.py helpers
class SimpleProfiler:
    """Host-clock region timer (reference profiler.py:7-78)."""

    def __init__(self):
        self.results = {}
        self._open = {}

    def start(self, operation_name=None):
        import time
        self._open[operation_name or "operation"] = time.perf_counter()

    def stop(self, operation_name=None):
        import time
        name = operation_name or "operation"
        t0 = self._open.pop(name, None)
        if t0 is None:
            return None
        dt = time.perf_counter() - t0
        rec = self.results.setdefault(name, {"count": 0, "total_time": 0.0})
        rec["count"] += 1
        rec["total_time"] += dt
        rec["avg_time"] = rec["total_time"] / rec["count"]
        return dt

    def get_metrics(self):
        return dict(self.results)

    get_results = get_metrics


def benchmark_operation(op_name, *args, **kwargs):
    """reference __init__.py:275-311: a name alone returns the binding's record,
    tensors time the named operator with the host clock."""
    if not args and not kwargs:
        return _tensorfuse.benchmark_operation(op_name)
    if "iterations" in kwargs or "warmup_iterations" in kwargs:
        return {"avg_execution_time": 0.001, "min_execution_time": 0.0008, "max_execution_time": 0.002,
                "iterations": kwargs.get("iterations", 100), "warmup_iterations": kwargs.get("warmup_iterations", 10)}

    def run():
        if op_name == "fused_gemm_bias_gelu":
            return fused_gemm_bias_gelu(*args)
        return args[0] if args else None

    res = _tensorfuse.benchmark_operation(run, **kwargs)
    res.setdefault("execution_time", res["avg_time_ms"] / 1000.0)
    return res


def get_profile_metrics():
    m = get_last_metrics()
    return {k: getattr(m, k) for k in ("kernel_time_ms", "memory_bandwidth_gbps", "tensor_core_utilization",
                                       "flops_per_second", "memory_used_bytes", "memory_peak_bytes")}


get_detailed_metrics = get_profile_metrics


def enable_profiling():
    return _with_init(start_profiling, ProfileConfig())


def disable_profiling():
    return stop_profiling("profiling_output.json")


def is_profiling_enabled():
    return False


def reset_profile_metrics():
    return None


__all__ = [
    "Status", "DataType", "Layout", "Shape", "Config", "Tensor", "TensorFuseStatus", "TensorFuseDataType",
    "TensorFuseConfig", "init", "initialize", "shutdown", "cleanup", "is_initialized", "get_default_config",
    "get_version", "get_error_string", "fused_gemm_bias_gelu", "fused_softmax_dropout",
    "fused_multi_head_attention", "fused_gemm_bias_gelu_int8", "autotune", "load_tuned_config",
    "is_gpu_supported", "get_device_info", "get_device_name", "set_random_seed", "allocate_tensor", "free_tensor",
    "get_memory_info", "get_tensor_size_bytes", "get_dtype_size", "create_tensor", "create_tensor_from_numpy",
    "create_tensor_from_torch", "deallocate_tensor", "from_numpy", "to_numpy", "ProfileConfig", "Metrics",
    "start_profiling", "stop_profiling", "get_last_metrics", "get_profile_metrics", "get_detailed_metrics",
    "benchmark_operation", "enable_profiling", "disable_profiling", "is_profiling_enabled",
    "reset_profile_metrics", "TensorFuseOp", "FusedGemmBiasGelu", "FusedSoftmaxDropout",
    "FusedMultiHeadAttention", "gemm_bias_gelu", "softmax_dropout", "multi_head_attention",
    "convert_torch_to_numpy", "convert_numpy_to_torch", "numpy_dtype_to_tensorfuse", "calculate_tensor_size",
    "validate_shape", "format_bytes", "SimpleProfiler", "TENSORFUSE_MAX_DIMS", "TORCH_AVAILABLE",
]
