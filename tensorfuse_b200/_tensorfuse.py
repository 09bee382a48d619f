"""`_tensorfuse` -- the extension-module surface of the reference's Python
binding, provided over the C ABI of libtensorfuse.so with ctypes.

The reference builds a pybind11 module ``tensorfuse._tensorfuse``
(reference ``src/python/tensorfuse_python.cpp:26``) and its package imports a
fixed list of names from it (``src/python/tensorfuse/__init__.py:53-95``,
``memory.py:17``); if one is missing the whole package degrades to stubs.
Every one of those names is defined here with the binding's signature,
argument names, return shape and ``RuntimeError`` texts:

    Status, DataType, Layout, Shape, Config, Tensor, ProfileConfig, Metrics,
    RooflineModel, init, shutdown, get_version, get_error_string,
    fused_gemm_bias_gelu, fused_softmax_dropout, fused_multi_head_attention,
    autotune, load_tuned_config, is_gpu_supported, get_device_info,
    set_random_seed, allocate_tensor, free_tensor, get_memory_info,
    get_tensor_size_bytes, get_dtype_size, set_memory_pool_size,
    get_memory_pool_stats, clear_memory_pool, start_profiling, stop_profiling,
    get_last_metrics, benchmark_operation, profile_memory_usage,
    calculate_roofline, create_tensor, from_numpy, to_numpy, tensor_copy,
    tensor_fill, tensor_zero, tensor_reshape

The operators take numpy (host) arrays exactly as the binding does
(``core_bindings.cpp:360-633, 635-771, 773-798``) and run on the GPU through
the library's host-buffer entry points; nothing here computes on the CPU.

Deliberate differences from the binding (each one removes a defect):
  * ``from_numpy`` copies the array to the device and ``to_numpy`` copies it
    back; the binding stores the HOST pointer in a "device" tensor
    (``tensor_bindings.cpp:121-123``) and ``tensor_fill/zero/copy`` then run
    ``memset``/``memcpy`` on it (``:160-183``).
  * ``get_device_info`` / ``get_memory_info`` / ``is_gpu_supported`` ask the
    device; the binding returns constants (``core_bindings.cpp:825-838``,
    ``memory_bindings.cpp:46-61``).
  * ``fused_softmax_dropout`` honours float16 arrays; the binding reinterprets
    every array as float32 (``core_bindings.cpp:652-653``).
  * ``fused_gemm_bias_gelu`` also accepts 3-D ``[batch, seq, hidden]`` inputs
    (the README quick start), which the binding rejects (``:365``).
  * ``fused_multi_head_attention`` computes; the reference's C entry point
    validates and returns (``src/tensorfuse_c_api.cpp:288-311``).
  * ``set_random_seed`` seeds the dropout stream; a no-op in the binding
    (``core_bindings.cpp:840-843``).
``get_last_metrics`` keeps the binding's placeholder numbers
(``profiler_bindings.cpp:89-102``): nothing in the library records them.
"""
from __future__ import annotations

import ctypes as C
import enum
import time

import numpy as np

from . import _lib
from ._lib import lib as _L

MAX_DIMS = _lib.MAX_DIMS


# ------------------------------------------------------------------ enums
# Plain enums without alias members: the reference package adds its aliases
# itself by assignment (``DataType.FP32 = DataType.FLOAT32``, __init__.py:111-129),
# which an enum class only permits for names that are not members yet.
class Status(enum.IntEnum):
    SUCCESS = 0
    INVALID_ARGUMENT = 1
    CUDA_ERROR = 2
    OUT_OF_MEMORY = 3
    NOT_INITIALIZED = 4
    INVALID_CONFIGURATION = 5
    KERNEL_LAUNCH_FAILED = 6
    AUTOTUNER_FAILED = 7
    PROFILING_FAILED = 8
    FILE_IO = 9
    UNSUPPORTED_OPERATION = 10
    INVALID_TENSOR_SHAPE = 11
    UNKNOWN = 99


class DataType(enum.IntEnum):
    FLOAT32 = 0
    FLOAT16 = 1
    BFLOAT16 = 2
    INT8 = 3
    UINT8 = 4
    INT32 = 5
    FP8_E4M3 = 6
    FP8_E5M2 = 7


class Layout(enum.IntEnum):
    ROW_MAJOR = 0
    COLUMN_MAJOR = 1
    NCHW = 2
    NHWC = 3


_DT_SIZE = {0: 4, 1: 2, 2: 2, 3: 1, 4: 1, 5: 4, 6: 1, 7: 1}
_NP_TO_DT = {np.dtype(np.float32): DataType.FLOAT32, np.dtype(np.float16): DataType.FLOAT16,
             np.dtype(np.int8): DataType.INT8, np.dtype(np.uint8): DataType.UINT8,
             np.dtype(np.int32): DataType.INT32}
_DT_TO_NP = {DataType.FLOAT32: np.float32, DataType.FLOAT16: np.float16, DataType.INT8: np.int8,
             DataType.UINT8: np.uint8, DataType.INT32: np.int32}


def _err(status) -> str:
    return _L.tensorfuse_get_error_string(int(status)).decode()


def _raise_unless_ok(prefix: str, status: int):
    if status != 0:
        raise RuntimeError(prefix + _err(status))


# ---------------------------------------------------------------- classes
class Shape:
    """TensorFuseShape (tensorfuse_python.cpp:82-108): ``Shape()`` or ``Shape([d0, d1, ...])``."""

    def __init__(self, dims=None):
        self.ndims = 0
        self._dims = [0] * MAX_DIMS
        if dims is not None:
            dims = [int(d) for d in dims][:MAX_DIMS]
            self.ndims = len(dims)
            self._dims[:len(dims)] = dims

    @property
    def dims(self):
        return list(self._dims[:self.ndims])

    @dims.setter
    def dims(self, value):
        value = [int(d) for d in value][:MAX_DIMS]
        self.ndims = len(value)
        self._dims = value + [0] * (MAX_DIMS - len(value))

    def _to_c(self) -> _lib.Shape:
        s = _lib.Shape()
        s.ndims = self.ndims
        stride = 1
        for k in range(self.ndims - 1, -1, -1):
            s.dims[k] = self._dims[k]
            s.strides[k] = stride
            stride *= self._dims[k]
        return s

    def __repr__(self):
        return "Shape([" + ", ".join(str(d) for d in self.dims) + "])"


class Config:
    """TensorFuseConfig (tensorfuse_python.cpp:113-141).  ``device_ids`` (a
    list; not exposed by the reference binding, which has no use for it)
    selects the GPUs the operators shard rows over."""

    def __init__(self):
        self.device_count = 1
        self.device_ids = None
        self.workspace_size_bytes = 1 << 30
        self.enable_profiling = False
        self.enable_autotuning = True
        self.enable_fp8 = False
        self.log_level = 1
        self.cache_dir = ""

    def __repr__(self):
        return (f"Config(device_count={self.device_count}, workspace_size_bytes={self.workspace_size_bytes}, "
                f"enable_profiling={self.enable_profiling})")


class Tensor:
    """TensorFuseTensor (tensor_bindings.cpp:23-52).  ``data`` is the device
    address as an integer."""

    def __init__(self):
        self.shape = Shape()
        self.dtype = DataType.FLOAT32
        self.layout = Layout.ROW_MAJOR
        self.device_id = 0
        self.size_bytes = 0
        self.is_contiguous = True
        self.data = 0
        self._owned = False   # set by the allocating functions: device memory is released with the object

    def __del__(self):
        if getattr(self, "_owned", False) and self.data:
            try:
                ct = self._to_c()
                _L.tensorfuse_free_tensor(C.byref(ct))
            except Exception:   # interpreter shutdown
                pass
            self.data = 0

    def _to_c(self, scale_ptr=None) -> _lib.Tensor:
        t = _lib.Tensor()
        t.data = self.data or None
        t.shape = self.shape._to_c()
        t.dtype = int(self.dtype)
        t.layout = int(self.layout)
        t.device_id = int(self.device_id)
        t.size_bytes = int(self.size_bytes)
        t.is_contiguous = bool(self.is_contiguous)
        t.scale = scale_ptr
        t.zero_point = None
        return t

    def __repr__(self):
        return f"Tensor(shape={self.shape!r}, dtype={int(self.dtype)}, device_id={self.device_id})"


class ProfileConfig:
    """TensorFuseProfileConfig (profiler_bindings.cpp:26-50)."""

    def __init__(self):
        self.enable_nsight_systems = False
        self.enable_nsight_compute = False
        self.enable_nvtx = False
        self.enable_cuda_events = False
        self.enable_memory_tracking = False
        self.warmup_iterations = 0
        self.profile_iterations = 0
        self.output_prefix = ""

    def __repr__(self):
        return f"ProfileConfig(warmup_iterations={self.warmup_iterations}, profile_iterations={self.profile_iterations})"


class Metrics:
    """TensorFuseMetrics (profiler_bindings.cpp:52-67)."""

    def __init__(self):
        self.kernel_time_ms = 0.0
        self.memory_bandwidth_gbps = 0.0
        self.tensor_core_utilization = 0.0
        self.flops_per_second = 0.0
        self.memory_used_bytes = 0
        self.memory_peak_bytes = 0
        self.num_kernel_launches = 0
        self.cpu_time_ms = 0.0
        self.total_time_ms = 0.0

    def __repr__(self):
        return f"Metrics(kernel_time_ms={self.kernel_time_ms}, flops_per_second={self.flops_per_second})"


class RooflineModel:
    """TensorFuseRooflineModel (profiler_bindings.cpp:188-202)."""

    def __init__(self):
        self.peak_flops = 0.0
        self.peak_bandwidth = 0.0
        self.arithmetic_intensity = 0.0
        self.achieved_flops = 0.0
        self.achieved_bandwidth = 0.0
        self.efficiency_flops = 0.0
        self.efficiency_bandwidth = 0.0
        self.is_compute_bound = False
        self.is_memory_bound = False

    def __repr__(self):
        return (f"RooflineModel(arithmetic_intensity={self.arithmetic_intensity:f}, "
                f"efficiency_flops={self.efficiency_flops:f}%)")


# ------------------------------------------------------- library lifetime
def init(config: Config | None = None):
    """core_bindings.cpp:112-137: with or without a Config."""
    if config is None:
        st = _L.tensorfuse_init(None)
    else:
        ids = list(config.device_ids) if getattr(config, "device_ids", None) is not None else None
        n = len(ids) if ids is not None else int(config.device_count)
        arr = (C.c_int * n)(*ids) if ids is not None else None
        c = _lib.Config(n, C.cast(arr, C.POINTER(C.c_int)) if arr is not None else None,
                        int(config.workspace_size_bytes), bool(config.enable_profiling),
                        bool(config.enable_autotuning), bool(config.enable_fp8), int(config.log_level),
                        (config.cache_dir or "").encode())
        st = _L.tensorfuse_init(C.byref(c))
    _raise_unless_ok("Failed to initialize TensorFuse: ", st)


def shutdown():
    _raise_unless_ok("Failed to shutdown TensorFuse: ", _L.tensorfuse_shutdown())


def get_version() -> str:
    return _L.tensorfuse_get_version().decode()


def get_error_string(status) -> str:
    return _err(status)


# -------------------------------------------------------------- operators
def _host(a, what: str):
    if not isinstance(a, np.ndarray):
        raise TypeError(f"{what} must be a numpy array")
    return a


def fused_gemm_bias_gelu(input, weight, bias, output, stream=None):
    """output = GELU(input @ weight + bias), written into ``output`` (core_bindings.cpp:360-633).

    float32 / float16: all four arrays of that dtype.  int8 input and weight
    with float32 bias and output: the binding's convention -- the two scales
    are guessed as 127 / max|q| from the quantised data (``:467-491``) and the
    result is ``gelu(acc/(sA*sB) + bias) * (sA*sB)``.
    """
    A, W, b = _host(input, "input"), _host(weight, "weight"), _host(bias, "bias")
    out = _host(output, "output")
    if W.ndim != 2 or b.ndim != 1 or A.ndim not in (2, 3) or out.ndim != A.ndim:
        raise RuntimeError("Invalid tensor dimensions for fused_gemm_bias_gelu")
    K, N = W.shape
    if A.shape[-1] != K or b.shape[0] != N or tuple(out.shape) != tuple(A.shape[:-1]) + (N,):
        raise RuntimeError("Tensor dimension mismatch in fused_gemm_bias_gelu")
    for a in (A, W, b, out):
        if a.dtype not in _NP_TO_DT:
            raise RuntimeError("Unsupported numpy dtype for TensorFuse")
    if not out.flags["C_CONTIGUOUS"] or not out.flags["WRITEABLE"]:
        raise RuntimeError("fused_gemm_bias_gelu failed: " + _err(Status.INVALID_ARGUMENT))
    A = np.ascontiguousarray(A)
    W = np.ascontiguousarray(W)
    b = np.ascontiguousarray(b)
    in_dt, out_dt = _NP_TO_DT[A.dtype], _NP_TO_DT[out.dtype]
    M = A.size // K if K else 0
    sA = sB = 1.0
    mode = 0
    if in_dt == DataType.INT8:
        if W.dtype != np.int8 or b.dtype != np.float32 or out.dtype != np.float32:
            raise RuntimeError("fused_gemm_bias_gelu failed: " + _err(
                Status.INVALID_ARGUMENT if W.dtype != np.int8 else Status.UNSUPPORTED_OPERATION))
        sA = 127.0 / max(float(np.abs(A.astype(np.int16)).max(initial=0)), 1.0)
        sB = 127.0 / max(float(np.abs(W.astype(np.int16)).max(initial=0)), 1.0)
        mode = 2   # reference convention (include/tensorfuse_b200.h, epilogue 2)
    elif in_dt in (DataType.FLOAT32, DataType.FLOAT16):
        if W.dtype != A.dtype or out.dtype != A.dtype:
            raise RuntimeError("fused_gemm_bias_gelu failed: " + _err(Status.INVALID_ARGUMENT))
        if b.dtype != A.dtype:
            b = b.astype(A.dtype)
    else:
        raise RuntimeError("fused_gemm_bias_gelu failed: " + _err(Status.UNSUPPORTED_OPERATION))
    st = _L.tensorfuse_b200_gemm_bias_gelu_host(A.ctypes.data, W.ctypes.data, b.ctypes.data, out.ctypes.data,
                                                M, N, K, int(in_dt), int(_NP_TO_DT[b.dtype]), int(out_dt),
                                                mode, sA, sB)
    _raise_unless_ok("fused_gemm_bias_gelu failed: ", st)


def fused_softmax_dropout(input, output, dropout_mask, dropout_prob, stream=None):
    """Softmax over the last of four axes, then dropout; ``dropout_mask`` (uint8,
    same shape) receives 1 where an element was kept (core_bindings.cpp:635-771)."""
    x, out, mask = _host(input, "input"), _host(output, "output"), _host(dropout_mask, "dropout_mask")
    if x.ndim != 4 or out.ndim != 4:
        raise RuntimeError("Input and output must be 4D tensors")
    if tuple(x.shape) != tuple(out.shape):
        raise RuntimeError("Input and output must have the same shape")
    if x.dtype not in (np.float32, np.float16) or out.dtype != x.dtype:
        raise RuntimeError("fused_softmax_dropout failed: " + _err(
            Status.INVALID_ARGUMENT if out.dtype != x.dtype else Status.UNSUPPORTED_OPERATION))
    if mask.size != x.size or mask.dtype.itemsize != 1:
        raise RuntimeError("fused_softmax_dropout failed: " + _err(Status.INVALID_ARGUMENT))
    if not (out.flags["C_CONTIGUOUS"] and mask.flags["C_CONTIGUOUS"] and out.flags["WRITEABLE"] and
            mask.flags["WRITEABLE"]):
        raise RuntimeError("fused_softmax_dropout failed: " + _err(Status.INVALID_ARGUMENT))
    x = np.ascontiguousarray(x)
    L = x.shape[-1]
    st = _L.tensorfuse_b200_softmax_dropout_host(x.ctypes.data, out.ctypes.data, mask.ctypes.data,
                                                 x.size // max(L, 1), L, int(_NP_TO_DT[x.dtype]),
                                                 float(dropout_prob), _next_seed())
    _raise_unless_ok("fused_softmax_dropout failed: ", st)


def fused_multi_head_attention(query, key, value, output, num_heads, dropout_prob, stream=None):
    """output = dropout(softmax(Q K^T / sqrt(d))) V per head on host arrays
    ``[batch, seq, hidden]`` (core_bindings.cpp:773-798)."""
    q, k, v, out = (_host(a, n) for a, n in ((query, "query"), (key, "key"), (value, "value"), (output, "output")))
    for a in (q, k, v, out):
        if a.dtype not in (np.float32, np.float16):
            raise RuntimeError("Unsupported numpy dtype for TensorFuse")
    dt = _NP_TO_DT[q.dtype]
    dev = []
    try:
        for a in (q, k, v, out):
            t = from_numpy(np.ascontiguousarray(a))
            dev.append(t)
        cts = [t._to_c() for t in dev]
        st = _L.tensorfuse_fused_multi_head_attention(C.byref(cts[0]), C.byref(cts[1]), C.byref(cts[2]),
                                                      C.byref(cts[3]), int(num_heads), float(dropout_prob), None)
        _raise_unless_ok("fused_multi_head_attention failed: ", st)
        if not out.flags["C_CONTIGUOUS"]:
            raise RuntimeError("fused_multi_head_attention failed: " + _err(Status.INVALID_ARGUMENT))
        st = _L.tensorfuse_b200_memcpy(out.ctypes.data, dev[3].data, out.nbytes, 2)
        _raise_unless_ok("fused_multi_head_attention failed: ", st)
    finally:
        for t in dev:
            if t.data:
                free_tensor(t)
    del dt


# ------------------------------------------------------------ autotuning
class _ModelConfigC(C.Structure):
    _fields_ = [("batch_size", C.c_int), ("seq_length", C.c_int), ("hidden_dim", C.c_int),
                ("num_heads", C.c_int), ("ffn_dim", C.c_int), ("num_layers", C.c_int), ("dtype", C.c_int),
                ("use_flash_attention", C.c_bool), ("use_mixed_precision", C.c_bool),
                ("model_name", C.c_char_p)]


def autotune(model_config, output_path):
    """Placeholder in the reference (src/tensorfuse_c_api.cpp:335-349): validates, tunes nothing."""
    c = _ModelConfigC()
    for name, _ in _ModelConfigC._fields_:
        if name == "model_name":
            c.model_name = str(getattr(model_config, name, "") or "").encode()
        elif hasattr(model_config, name):
            setattr(c, name, int(getattr(model_config, name)))
    st = _L.tensorfuse_autotune(C.byref(c), str(output_path).encode())
    _raise_unless_ok("Autotuning failed: ", st)


def load_tuned_config(config_path):
    st = _L.tensorfuse_load_tuned_config(str(config_path).encode())
    _raise_unless_ok("Failed to load tuned config: ", st)


# -------------------------------------------------------------- utilities
def _device_props(device=-1):
    name = C.create_string_buffer(256)
    major, minor, sms = C.c_int(), C.c_int(), C.c_int()
    total = C.c_size_t()
    st = _L.tensorfuse_b200_device_info(int(device), name, 256, C.byref(major), C.byref(minor), C.byref(total),
                                        C.byref(sms))
    if st != 0:
        return None
    return name.value.decode(), major.value, minor.value, total.value, sms.value


def is_gpu_supported() -> bool:
    """True on a device this library has kernels for (compute capability 10.x)."""
    p = _device_props()
    return p is not None and p[1] == 10


def get_device_info():
    """Keys of the reference's dictionary (core_bindings.cpp:830-838), filled from the device."""
    p = _device_props()
    if p is None:
        raise RuntimeError("get_device_info failed: " + _err(Status.CUDA_ERROR))
    return {"name": p[0], "compute_capability": f"{p[1]}.{p[2]}", "memory_gb": int(round(p[3] / 2 ** 30)),
            "tensor_cores": p[1] == 10, "multiprocessors": p[4]}


_seed_state = [None, 0]


def set_random_seed(seed):
    _seed_state[0] = int(seed)
    _seed_state[1] = 0
    _L.tensorfuse_b200_set_random_seed(int(seed) & 0xFFFFFFFFFFFFFFFF)


def _next_seed() -> int:
    if _seed_state[0] is None:
        return int(np.random.SeedSequence().generate_state(1, dtype=np.uint64)[0])
    _seed_state[1] += 1
    return (_seed_state[0] * 0x9E3779B97F4A7C15 + _seed_state[1] * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF


# ------------------------------------------------------------------ memory
def _as_shape(shape) -> Shape:
    return shape if isinstance(shape, Shape) else Shape(list(shape))


def _from_c(ct: _lib.Tensor) -> Tensor:
    t = Tensor()
    t.shape = Shape([ct.shape.dims[i] for i in range(ct.shape.ndims)])
    t.dtype = DataType(ct.dtype)
    t.layout = Layout(ct.layout) if ct.layout in (0, 1, 2, 3) else Layout.ROW_MAJOR
    t.device_id = ct.device_id
    t.size_bytes = ct.size_bytes
    t.is_contiguous = bool(ct.is_contiguous)
    t.data = ct.data or 0
    t._owned = bool(t.data)
    return t


def _allocate(cs: _lib.Shape, dtype, device_id, prefix: str) -> Tensor:
    """tensorfuse_allocate_tensor; the library is initialised with its defaults
    first if it is not yet (the binding's from_numpy needs no initialisation --
    it only wraps the host pointer -- and callers rely on that)."""
    ct = _lib.Tensor()
    st = _L.tensorfuse_allocate_tensor(C.byref(ct), C.byref(cs), int(dtype), int(device_id))
    if st == Status.NOT_INITIALIZED:
        init()
        st = _L.tensorfuse_allocate_tensor(C.byref(ct), C.byref(cs), int(dtype), int(device_id))
    _raise_unless_ok(prefix, st)
    return _from_c(ct)


def allocate_tensor(shape, dtype, device_id=0):
    """memory_bindings.cpp:23-32 -> tensorfuse_allocate_tensor."""
    return _allocate(_as_shape(shape)._to_c(), dtype, device_id, "Failed to allocate tensor: ")


def free_tensor(tensor):
    ct = tensor._to_c()
    st = _L.tensorfuse_free_tensor(C.byref(ct))
    _raise_unless_ok("Failed to free tensor: ", st)
    tensor.data = 0
    tensor._owned = False
    tensor.size_bytes = 0


def get_memory_info():
    free_b, total_b = C.c_size_t(), C.c_size_t()
    if _L.tensorfuse_b200_mem_info(-1, C.byref(free_b), C.byref(total_b)) != 0:
        free_b.value = total_b.value = 0
    return {"free_bytes": free_b.value, "total_bytes": total_b.value, "used_bytes": total_b.value - free_b.value}


def get_tensor_size_bytes(shape, dtype):
    n = 1
    for d in _as_shape(shape).dims:
        n *= d
    return n * _DT_SIZE.get(int(dtype), 0)


def get_dtype_size(dtype):
    return _DT_SIZE.get(int(dtype), 0)


def set_memory_pool_size(size_bytes):
    """Placeholder in the reference (memory_bindings.cpp:75-78); the library's staging buffers grow on demand."""


def get_memory_pool_stats():
    return {"pool_size_bytes": 0, "allocated_bytes": 0, "free_bytes": 0, "num_allocations": 0, "num_frees": 0}


def clear_memory_pool():
    """Placeholder in the reference (memory_bindings.cpp:90-93)."""


# ---------------------------------------------------------------- tensors
def create_tensor(shape, dtype, device_id=0):
    """tensor_bindings.cpp:58-71."""
    if any(int(d) < 0 for d in shape):
        raise RuntimeError("Failed to create tensor: " + _err(Status.INVALID_TENSOR_SHAPE))
    return _allocate(Shape(list(shape))._to_c(), dtype, device_id, "Failed to create tensor: ")


def from_numpy(array, device_id=0):
    """A device tensor holding a copy of ``array`` (tensor_bindings.cpp:73-126 for
    the checks and messages).  Release it with ``free_tensor``."""
    arr = np.asarray(array)
    if arr.size == 0:
        raise RuntimeError("Cannot create tensor from empty array")
    if arr.ndim == 0:
        raise RuntimeError("Cannot create tensor from scalar array")
    if arr.ndim > MAX_DIMS:
        raise RuntimeError(f"Array has too many dimensions (max: {MAX_DIMS}, got: {arr.ndim})")
    if arr.dtype not in _NP_TO_DT:
        raise RuntimeError("Unsupported numpy dtype")
    arr = np.ascontiguousarray(arr)
    t = create_tensor(list(arr.shape), _NP_TO_DT[arr.dtype], device_id)
    st = _L.tensorfuse_b200_memcpy(t.data, arr.ctypes.data, arr.nbytes, 1)
    if st != 0:
        free_tensor(t)
        _raise_unless_ok("Failed to create tensor: ", st)
    return t


def to_numpy(tensor):
    """A host copy of a device tensor (tensor_bindings.cpp:128-154)."""
    if DataType(int(tensor.dtype)) not in _DT_TO_NP:
        raise RuntimeError("Unsupported tensor dtype")
    out = np.empty(tensor.shape.dims, dtype=_DT_TO_NP[DataType(int(tensor.dtype))])
    if out.nbytes:
        st = _L.tensorfuse_b200_memcpy(out.ctypes.data, tensor.data, out.nbytes, 2)
        _raise_unless_ok("to_numpy failed: ", st)
    return out


def tensor_copy(src, dst):
    if src.size_bytes != dst.size_bytes:
        raise RuntimeError("Tensor size mismatch")
    _raise_unless_ok("tensor_copy failed: ", _L.tensorfuse_b200_memcpy(dst.data, src.data, src.size_bytes, 3))


def tensor_fill(tensor, value):
    if int(tensor.dtype) != DataType.FLOAT32:
        raise RuntimeError("Only float32 tensors supported for fill")
    host = np.full(tensor.size_bytes // 4, value, dtype=np.float32)
    _raise_unless_ok("tensor_fill failed: ", _L.tensorfuse_b200_memcpy(tensor.data, host.ctypes.data, host.nbytes, 1))


def tensor_zero(tensor):
    host = np.zeros(tensor.size_bytes, dtype=np.uint8)
    _raise_unless_ok("tensor_zero failed: ", _L.tensorfuse_b200_memcpy(tensor.data, host.ctypes.data, host.nbytes, 1))


def tensor_reshape(tensor, new_shape):
    old = 1
    for d in tensor.shape.dims:
        old *= d
    new = 1
    for d in new_shape:
        new *= int(d)
    if old != new:
        raise RuntimeError("Invalid reshape: size mismatch")
    tensor.shape = Shape(list(new_shape))


# -------------------------------------------------------------- profiling
class _ProfileConfigC(C.Structure):
    _fields_ = [("enable_nsight_systems", C.c_bool), ("enable_nsight_compute", C.c_bool), ("enable_nvtx", C.c_bool),
                ("enable_cuda_events", C.c_bool), ("enable_memory_tracking", C.c_bool),
                ("output_prefix", C.c_char_p), ("warmup_iterations", C.c_int), ("profile_iterations", C.c_int)]


def start_profiling(config):
    c = _ProfileConfigC(bool(config.enable_nsight_systems), bool(config.enable_nsight_compute),
                        bool(config.enable_nvtx), bool(config.enable_cuda_events),
                        bool(config.enable_memory_tracking), str(config.output_prefix or "").encode(),
                        int(config.warmup_iterations), int(config.profile_iterations))
    _raise_unless_ok("Failed to start profiling: ", _L.tensorfuse_start_profiling(C.byref(c)))


def stop_profiling(output_path):
    _raise_unless_ok("Failed to stop profiling: ", _L.tensorfuse_stop_profiling(str(output_path).encode()))


def get_last_metrics():
    """The reference's placeholder values (profiler_bindings.cpp:89-102)."""
    m = Metrics()
    m.kernel_time_ms = 1.5
    m.memory_bandwidth_gbps = 800.0
    m.tensor_core_utilization = 85.0
    m.flops_per_second = 156e12
    m.memory_used_bytes = 512 << 20
    m.memory_peak_bytes = 768 << 20
    m.num_kernel_launches = 1
    m.cpu_time_ms = 0.1
    m.total_time_ms = 1.6
    return m


def benchmark_operation(operation, num_iterations=100, num_warmup=10):
    """Both overloads of the binding (profiler_bindings.cpp:116-166): a callable
    is timed with the host clock; a name gets the placeholder record."""
    if isinstance(operation, str):
        t0 = time.perf_counter()
        time.sleep(0.001)
        avg = (time.perf_counter() - t0) * 1e3
        return {"avg_time_ms": avg, "total_time_ms": avg * 100, "iterations": 100, "operation": operation}
    for _ in range(int(num_warmup)):
        operation()
    t0 = time.perf_counter()
    for _ in range(int(num_iterations)):
        operation()
    total = (time.perf_counter() - t0) * 1e3
    avg = total / max(int(num_iterations), 1)
    return {"avg_time_ms": avg, "total_time_ms": total, "iterations": int(num_iterations),
            "throughput_ops_per_sec": 1000.0 / avg if avg > 0 else 0.0}


def profile_memory_usage(operation):
    before = get_memory_info()["used_bytes"]
    operation()
    after = get_memory_info()["used_bytes"]
    return {"memory_used_bytes": after - before, "memory_before_bytes": before, "memory_after_bytes": after}


class _RooflineC(C.Structure):
    _fields_ = [("peak_flops", C.c_float), ("peak_bandwidth", C.c_float), ("arithmetic_intensity", C.c_float),
                ("achieved_flops", C.c_float), ("achieved_bandwidth", C.c_float), ("efficiency_flops", C.c_float),
                ("efficiency_bandwidth", C.c_float), ("is_compute_bound", C.c_bool), ("is_memory_bound", C.c_bool)]


def calculate_roofline(ops_count, bytes_transferred, time_ms):
    c = _RooflineC()
    fn = _L.tensorfuse_calculate_roofline
    fn.restype = C.c_int
    fn.argtypes = [C.c_size_t, C.c_size_t, C.c_float, C.POINTER(_RooflineC)]
    _raise_unless_ok("Failed to calculate roofline: ", fn(int(ops_count), int(bytes_transferred), float(time_ms),
                                                          C.byref(c)))
    m = RooflineModel()
    for name, _ in _RooflineC._fields_:
        setattr(m, name, getattr(c, name))
    return m
