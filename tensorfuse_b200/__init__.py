"""tensorfuse_b200 -- the Python face of libtensorfuse.so (B200 build).

Mirrors the operator surface of the reference's ``tensorfuse`` package
(reference ``src/python/tensorfuse/__init__.py:53-198`` and the binding
``src/python/core_bindings.cpp:360-771``): ``init``, ``shutdown``,
``fused_gemm_bias_gelu``, ``fused_softmax_dropout``,
``fused_multi_head_attention``, ``set_random_seed``, ``Status``, ``DataType``,
``Config``; same argument meaning, same ``RuntimeError("<op> failed: <error
string>")`` on failure, same automatic initialisation on first use.

Differences, all additive:
  * numpy (host) operands go through the library's pipelined host-buffer
    operators (row-sharded over the GPUs chosen at ``init``) instead of a
    cudaMalloc / synchronous-copy round trip;
  * torch CUDA tensors are used in place (no copy) on torch's current stream;
  * FP16 is supported by the softmax binding, INT8 GEMM takes explicit scales
    and can produce FP16 (multiply convention) or raw INT32 accumulators;
  * 3-D ``[batch, seq, hidden]`` inputs are accepted (flattened).

    import tensorfuse_b200 as tensorfuse
    tensorfuse.init()
    y = tensorfuse.fused_gemm_bias_gelu(x, w, b)
"""
from __future__ import annotations

import ctypes as C
import enum
import weakref

import numpy as np

from ._lib import Config as _CConfig
from ._lib import Shape as _CShape
from ._lib import Tensor as _CTensor
from ._lib import lib as _L

__version__ = "1.0.0"
TENSORFUSE_MAX_DIMS = 8


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
    # aliases the reference package adds (__init__.py:119-129)
    ERROR_INVALID_ARGUMENT = 1
    ERROR_CUDA_ERROR = 2
    ERROR_OUT_OF_MEMORY = 3
    ERROR_NOT_INITIALIZED = 4


class DataType(enum.IntEnum):
    FLOAT32 = 0
    FLOAT16 = 1
    BFLOAT16 = 2
    INT8 = 3
    UINT8 = 4
    INT32 = 5
    FP8_E4M3 = 6
    FP8_E5M2 = 7
    FP32 = 0
    FP16 = 1
    BF16 = 2


TensorFuseStatus = Status
TensorFuseDataType = DataType

# INT8 epilogue selectors (include/tensorfuse_b200.h)
INT8_DEQUANT = 1   # out = gelu(acc * sA * sB + bias), scale = max|x|/127
INT8_LEGACY = 2    # reference convention, scale = 127/max|x|, FP32 bias/out
INT8_RAW = 3       # raw INT32 accumulators

_NP_TO_DT = {np.dtype(np.float32): DataType.FLOAT32, np.dtype(np.float16): DataType.FLOAT16,
             np.dtype(np.int8): DataType.INT8, np.dtype(np.uint8): DataType.UINT8,
             np.dtype(np.int32): DataType.INT32}
_DT_TO_NP = {DataType.FLOAT32: np.float32, DataType.FLOAT16: np.float16, DataType.INT8: np.int8,
             DataType.INT32: np.int32, DataType.UINT8: np.uint8}


class Config:
    """TensorFuseConfig.  ``device_ids`` (a list) selects the GPUs the
    host-buffer operators shard rows over."""

    def __init__(self, device_count=1, device_ids=None, workspace_size_bytes=1 << 30,
                 enable_profiling=False, enable_autotuning=True, enable_fp8=False, log_level=1,
                 cache_dir="./cache"):
        self.device_count = device_count
        self.device_ids = device_ids
        self.workspace_size_bytes = workspace_size_bytes
        self.enable_profiling = enable_profiling
        self.enable_autotuning = enable_autotuning
        self.enable_fp8 = enable_fp8
        self.log_level = log_level
        self.cache_dir = cache_dir

    def _to_c(self):
        ids = list(self.device_ids) if self.device_ids is not None else None
        n = len(ids) if ids is not None else int(self.device_count)
        arr = (C.c_int * n)(*ids) if ids is not None else None
        c = _CConfig(n, C.cast(arr, C.POINTER(C.c_int)) if arr is not None else None,
                     int(self.workspace_size_bytes), bool(self.enable_profiling),
                     bool(self.enable_autotuning), bool(self.enable_fp8), int(self.log_level),
                     (self.cache_dir or "").encode())
        return c, arr


TensorFuseConfig = Config


def get_error_string(status) -> str:
    return _L.tensorfuse_get_error_string(int(status)).decode()


def get_version() -> str:
    return _L.tensorfuse_get_version().decode()


def _check(op: str, status: int):
    if status != 0:
        raise RuntimeError(f"{op} failed: {get_error_string(status)}")


def init(config: Config | None = None):
    """reference tensorfuse.init (core_bindings.cpp:286-310): idempotent."""
    if config is None:
        st = _L.tensorfuse_init(None)
    else:
        c, keep = config._to_c()
        st = _L.tensorfuse_init(C.byref(c))
        del keep
    _check("tensorfuse_init", st)
    return Status.SUCCESS


def shutdown():
    _check("tensorfuse_shutdown", _L.tensorfuse_shutdown())
    return Status.SUCCESS


cleanup = shutdown


_seed_src = [None, 0]   # host-path seed source: [base seed or None, calls made]


def set_random_seed(seed: int):
    """Seed the dropout streams: the library's seed source (device-pointer
    calls) and the host-buffer path of this module."""
    _seed_src[0] = int(seed)
    _seed_src[1] = 0
    _L.tensorfuse_b200_set_random_seed(int(seed) & 0xFFFFFFFFFFFFFFFF)


def _next_host_seed() -> int:
    if _seed_src[0] is None:
        return int(np.random.SeedSequence().generate_state(1, dtype=np.uint64)[0])
    _seed_src[1] += 1
    return (int(_seed_src[0]) * 0x9E3779B97F4A7C15 + _seed_src[1] * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF


def device_ids():
    return [_L.tensorfuse_b200_device_id(i) for i in range(_L.tensorfuse_b200_device_count())]


def watchdog_status() -> int:
    return int(_L.tensorfuse_b200_watchdog_status())


def launch_count() -> int:
    return int(_L.tensorfuse_b200_launch_count())


def softmax_schedule(row_len: int, dtype=np.float16, aligned16: bool = True):
    v, w = C.c_int(), C.c_int()
    _L.tensorfuse_b200_softmax_schedule(int(row_len), int(_NP_TO_DT[np.dtype(dtype)]),
                                        int(aligned16), C.byref(v), C.byref(w))
    return v.value, w.value


def softmax_schedule_ex(row_len: int, dtype=np.float16, aligned16: bool = True):
    """(vec, warps, online): softmax_schedule plus whether the row is summed online."""
    v, w, o = C.c_int(), C.c_int(), C.c_int()
    _L.tensorfuse_b200_softmax_schedule_ex(int(row_len), int(_NP_TO_DT[np.dtype(dtype)]), int(aligned16),
                                           C.byref(v), C.byref(w), C.byref(o))
    return v.value, w.value, o.value


def plan_shards(rows: int, parts: int, align: int = 1):
    b = (C.c_longlong * parts)()
    c = (C.c_longlong * parts)()
    _L.tensorfuse_b200_plan_shards(rows, parts, align, b, c)
    return list(b), list(c)


# ------------------------------------------------------- immutable weights
def _ptr_and_bytes(x):
    if _is_torch(x):
        return int(x.data_ptr()), int(x.numel() * x.element_size())
    a = np.asarray(x)
    return int(a.ctypes.data), int(a.nbytes)


def register_weights(*tensors):
    """Declare weight buffers (numpy arrays in host memory or torch CUDA tensors)
    immutable: the host-buffer GEMM then keeps one device copy per GPU instead of
    uploading them on every call, and ``fused_transformer_layer`` builds its
    fused query/key/value weight once.  Call ``invalidate_weights`` before
    changing or freeing them."""
    for t in tensors:
        ptr, nbytes = _ptr_and_bytes(t)
        st = _auto_init(_L.tensorfuse_b200_register_weights, ptr, nbytes)
        _check("register_weights", st)


def invalidate_weights(*tensors):
    """Forget registered weight buffers (all of them when called without arguments)."""
    if not tensors:
        _check("invalidate_weights", _L.tensorfuse_b200_invalidate_weights(None))
    for t in tensors:
        _check("invalidate_weights", _L.tensorfuse_b200_invalidate_weights(_ptr_and_bytes(t)[0]))


# ------------------------------------------------------------ pinned memory
def pinned_empty(shape, dtype) -> np.ndarray:
    """numpy array in page-locked host memory owned by the library."""
    dtype = np.dtype(dtype)
    n = int(np.prod(shape)) * dtype.itemsize
    p = _L.tensorfuse_b200_alloc_pinned(max(n, 1))
    if not p:
        raise MemoryError("tensorfuse_b200_alloc_pinned failed")
    buf = (C.c_char * max(n, 1)).from_address(p)
    arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
    weakref.finalize(buf, _L.tensorfuse_b200_free_pinned, p)
    return arr


# ------------------------------------------------------------------ helpers
def _is_torch(x) -> bool:
    return hasattr(x, "detach") and hasattr(x, "data_ptr")


def _auto_init(fn, *args):
    """The reference wrapper retries once after init() when the library reports
    'Library not initialized' (__init__.py:151-162)."""
    st = fn(*args)
    if st == Status.NOT_INITIALIZED:
        init()
        st = fn(*args)
    return st


def _np_ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c_tensor(ptr: int, shape, dtype: DataType, scale_ptr: int | None = None) -> _CTensor:
    s = _CShape()
    s.ndims = len(shape)
    stride = 1
    for k in range(len(shape) - 1, -1, -1):
        s.dims[k] = int(shape[k])
        s.strides[k] = stride
        stride *= int(shape[k])
    t = _CTensor()
    t.data = ptr
    t.shape = s
    t.dtype = int(dtype)
    t.layout = 0
    t.device_id = 0
    t.size_bytes = int(np.prod(shape)) * {0: 4, 1: 2, 2: 2, 3: 1, 4: 1, 5: 4}.get(int(dtype), 1)
    t.is_contiguous = True
    t.scale = scale_ptr
    t.zero_point = None
    return t


def _torch_dt(t):
    import torch
    return {torch.float32: DataType.FLOAT32, torch.float16: DataType.FLOAT16,
            torch.bfloat16: DataType.BFLOAT16, torch.float8_e4m3fn: DataType.FP8_E4M3,
            torch.int8: DataType.INT8, torch.int32: DataType.INT32,
            torch.uint8: DataType.UINT8}[t.dtype]


def _torch_stream(stream, device):
    if stream is not None:
        return int(getattr(stream, "cuda_stream", stream))
    import torch
    return int(torch.cuda.current_stream(device).cuda_stream)


# ------------------------------------------------------- GEMM + bias + GELU
def fused_gemm_bias_gelu(input, weight, bias, output=None, stream=None, *, scales=None,
                         out_dtype=None, int8_mode=None):
    """output = gelu(input @ weight + bias)  (tanh-form GELU).

    input [M,K] or [batch,seq,K]; weight [K,N]; bias [N].  numpy operands run
    through the host-buffer operator, torch CUDA tensors in place.

    INT8 operands: ``scales=(sA, sB)`` (floats, or for CUDA tensors one-element
    float32 CUDA tensors).  ``int8_mode`` is INT8_LEGACY (default for FP32
    output: the reference's convention), INT8_DEQUANT (default for FP16 output)
    or INT8_RAW (INT32 accumulators).  Without ``scales`` the reference
    binding's guess 127/max|q| is used (core_bindings.cpp:467-491).
    """
    if _is_torch(input):
        if input.is_cuda:
            return _gemm_torch_cuda(input, weight, bias, output, stream, scales, out_dtype, int8_mode)
        import torch
        res = fused_gemm_bias_gelu(input.detach().numpy(), weight.detach().cpu().numpy(),
                                   bias.detach().cpu().numpy(),
                                   None if output is None else output.detach().numpy(), None,
                                   scales=scales, out_dtype=out_dtype, int8_mode=int8_mode)
        return output if output is not None else torch.from_numpy(res)

    A = np.ascontiguousarray(input)
    W = np.ascontiguousarray(weight)
    b = np.ascontiguousarray(bias)
    if A.ndim not in (2, 3) or W.ndim != 2 or b.ndim != 1:
        raise RuntimeError("fused_gemm_bias_gelu failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
    K, N = W.shape
    if A.shape[-1] != K or b.shape[0] != N:
        raise RuntimeError("fused_gemm_bias_gelu failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
    M = int(np.prod(A.shape[:-1]))
    in_dt = _NP_TO_DT.get(A.dtype)
    if in_dt is None or W.dtype != A.dtype:
        raise RuntimeError("fused_gemm_bias_gelu failed: " + get_error_string(Status.INVALID_ARGUMENT))

    sA = sB = 1.0
    mode = 0
    if in_dt == DataType.INT8:
        if output is not None and out_dtype is None:
            out_dtype = output.dtype
        odt = np.dtype(out_dtype) if out_dtype is not None else np.dtype(np.float32)
        if int8_mode is None:
            int8_mode = {np.dtype(np.float32): INT8_LEGACY, np.dtype(np.float16): INT8_DEQUANT,
                         np.dtype(np.int32): INT8_RAW}.get(odt, INT8_LEGACY)
        mode = int(int8_mode)
        if scales is None:
            sA = 127.0 / max(float(np.max(np.abs(A.astype(np.int32)))), 1.0)
            sB = 127.0 / max(float(np.max(np.abs(W.astype(np.int32)))), 1.0)
        else:
            sA, sB = float(scales[0]), float(scales[1])
        if mode == INT8_LEGACY:
            b = np.ascontiguousarray(b, dtype=np.float32)
    else:
        odt = A.dtype
        b = np.ascontiguousarray(b, dtype=A.dtype)
    out_shape = A.shape[:-1] + (N,)
    if output is None:
        output = np.empty(out_shape, dtype=odt)
    if tuple(output.shape) != tuple(out_shape) or not output.flags["C_CONTIGUOUS"] or output.dtype != odt:
        raise RuntimeError("fused_gemm_bias_gelu failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
    st = _auto_init(_L.tensorfuse_b200_gemm_bias_gelu_host, _np_ptr(A), _np_ptr(W), _np_ptr(b),
                    _np_ptr(output), M, N, K, int(in_dt), int(_NP_TO_DT[b.dtype]),
                    int(_NP_TO_DT[np.dtype(odt)]), mode, sA, sB)
    _check("fused_gemm_bias_gelu", st)
    return output


def _check_cuda_out(op: str, t, shape, dtype, device):
    """A caller-supplied CUDA result tensor is written through its raw pointer:
    refuse anything but the exact dense tensor the operator is about to fill."""
    if (not _is_torch(t) or not t.is_cuda or t.device != device or tuple(t.shape) != tuple(shape) or
            not t.is_contiguous() or (dtype is not None and t.dtype != dtype)):
        raise RuntimeError(f"{op} failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))


def _gemm_torch_cuda(x, w, b, out, stream, scales, out_dtype, int8_mode):
    import torch
    x = x.contiguous(); w = w.contiguous(); b = b.contiguous()
    if w.dim() != 2 or x.dim() < 1 or x.shape[-1] != w.shape[0] or b.numel() != w.shape[1] or \
            w.device != x.device or b.device != x.device:
        raise RuntimeError("fused_gemm_bias_gelu failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
    K, N = w.shape
    M = x.numel() // max(1, x.shape[-1])
    if out is not None:
        _check_cuda_out("fused_gemm_bias_gelu", out, tuple(x.shape[:-1]) + (N,), out_dtype, x.device)
    in_dt = _torch_dt(x)
    s = _torch_stream(stream, x.device)
    with torch.cuda.device(x.device):
        if in_dt == DataType.INT8:
            if out is not None and out_dtype is None:
                out_dtype = out.dtype
            odt = out_dtype if out_dtype is not None else torch.float32
            if int8_mode is None:
                int8_mode = {torch.float32: INT8_LEGACY, torch.float16: INT8_DEQUANT,
                             torch.int32: INT8_RAW}[odt]
            if out is None:
                out = torch.empty(tuple(x.shape[:-1]) + (N,), dtype=odt, device=x.device)
            if scales is not None and _is_torch(scales[1]) and scales[1].numel() == N and N > 1:
                # per-column weight scales (and a device-resident activation scale)
                sa = scales[0] if _is_torch(scales[0]) else torch.tensor([float(scales[0])], device=x.device)
                st = _auto_init(_L.tensorfuse_b200_gemm_int8_channelwise, x.data_ptr(), w.data_ptr(), b.data_ptr(),
                                out.data_ptr(), M, N, K, sa.data_ptr(), scales[1].contiguous().data_ptr(),
                                int(_torch_dt(b)), int(_torch_dt(out)), s)
            elif scales is not None and _is_torch(scales[0]):
                # device-resident scales: struct ABI, no host synchronisation
                ti = _c_tensor(x.data_ptr(), (M, x.shape[-1]), in_dt, scales[0].data_ptr())
                tw = _c_tensor(w.data_ptr(), (K, N), in_dt, scales[1].data_ptr())
                tb = _c_tensor(b.data_ptr(), (N,), _torch_dt(b))
                to = _c_tensor(out.data_ptr(), (M, N), _torch_dt(out))
                st = _auto_init(_L.tensorfuse_fused_gemm_bias_gelu, C.byref(ti), C.byref(tw),
                                C.byref(tb), C.byref(to), s)
            else:
                sA, sB = (1.0, 1.0) if scales is None else (float(scales[0]), float(scales[1]))
                st = _L.tensorfuse_b200_gemm_int8(x.data_ptr(), w.data_ptr(), b.data_ptr(),
                                                  out.data_ptr(), M, N, K, sA, sB, int(_torch_dt(b)),
                                                  int(_torch_dt(out)), int(int8_mode), s)
        elif in_dt == DataType.FP8_E4M3:
            # E4M3 operands, per-tensor dequantisation factors (floats or one-element CUDA tensors)
            odt = out_dtype if out_dtype is not None else (out.dtype if out is not None else torch.float16)
            if out is None:
                out = torch.empty(tuple(x.shape[:-1]) + (N,), dtype=odt, device=x.device)
            if scales is not None and _is_torch(scales[0]):
                ti = _c_tensor(x.data_ptr(), (M, x.shape[-1]), in_dt, scales[0].data_ptr())
                tw = _c_tensor(w.data_ptr(), (K, N), in_dt, scales[1].data_ptr())
                tb = _c_tensor(b.data_ptr(), (N,), _torch_dt(b))
                to = _c_tensor(out.data_ptr(), (M, N), _torch_dt(out))
                st = _auto_init(_L.tensorfuse_fused_gemm_bias_gelu, C.byref(ti), C.byref(tw),
                                C.byref(tb), C.byref(to), s)
            else:
                sA, sB = (1.0, 1.0) if scales is None else (float(scales[0]), float(scales[1]))
                st = _auto_init(_L.tensorfuse_b200_gemm_fp8, x.data_ptr(), w.data_ptr(), b.data_ptr(), out.data_ptr(),
                                M, N, K, sA, sB, int(_torch_dt(b)), int(_torch_dt(out)), s)
        else:
            if out is None:
                out = torch.empty(tuple(x.shape[:-1]) + (N,), dtype=x.dtype, device=x.device)
            ti = _c_tensor(x.data_ptr(), tuple(x.shape), in_dt)
            tw = _c_tensor(w.data_ptr(), (K, N), _torch_dt(w))
            tb = _c_tensor(b.data_ptr(), (N,), _torch_dt(b))
            to = _c_tensor(out.data_ptr(), tuple(out.shape), _torch_dt(out))
            st = _auto_init(_L.tensorfuse_fused_gemm_bias_gelu, C.byref(ti), C.byref(tw),
                            C.byref(tb), C.byref(to), s)
    _check("fused_gemm_bias_gelu", st)
    return out


# ------------------------------------------------------- softmax + dropout
def fused_softmax_dropout(input, output=None, dropout_mask=None, dropout_prob=0.0, stream=None, *,
                          seed=None):
    """output = dropout(softmax(input, axis=-1), p); dropout_mask[...] = 1 where kept.

    Reference signature: fused_softmax_dropout(input, output, dropout_mask,
    dropout_prob, stream) on 4-D arrays (core_bindings.cpp:635-771).  Returns
    ``(output, dropout_mask)``; both are allocated when not passed.  ``seed``
    fixes the Philox key of this call; otherwise the library's seed source
    (set_random_seed) supplies one.
    """
    if _is_torch(input):
        if input.is_cuda:
            return _softmax_torch_cuda(input, output, dropout_mask, dropout_prob, stream, seed)
        import torch
        o, m = fused_softmax_dropout(input.detach().numpy(),
                                     None if output is None else output.detach().numpy(),
                                     None if dropout_mask is None else dropout_mask.detach().numpy(),
                                     dropout_prob, None, seed=seed)
        return (output if output is not None else torch.from_numpy(o),
                dropout_mask if dropout_mask is not None else torch.from_numpy(m))

    x = np.ascontiguousarray(input)
    if x.ndim != 4:
        raise RuntimeError("fused_softmax_dropout failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
    dt = _NP_TO_DT.get(x.dtype)
    if dt not in (DataType.FLOAT16, DataType.FLOAT32):
        raise RuntimeError("fused_softmax_dropout failed: " + get_error_string(Status.UNSUPPORTED_OPERATION))
    if output is None:
        output = np.empty_like(x)
    if dropout_mask is None:
        dropout_mask = np.empty(x.shape, dtype=np.uint8)
    if (output.shape != x.shape or output.dtype != x.dtype or dropout_mask.shape != x.shape or
            dropout_mask.dtype != np.uint8 or not output.flags["C_CONTIGUOUS"] or
            not dropout_mask.flags["C_CONTIGUOUS"]):
        raise RuntimeError("fused_softmax_dropout failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
    if seed is None:
        seed = _next_host_seed()
    L = x.shape[-1]
    st = _auto_init(_L.tensorfuse_b200_softmax_dropout_host, _np_ptr(x), _np_ptr(output),
                    _np_ptr(dropout_mask), x.size // max(L, 1), L, int(dt), float(dropout_prob),
                    int(seed) & 0xFFFFFFFFFFFFFFFF)
    _check("fused_softmax_dropout", st)
    return output, dropout_mask


def fused_softmax_dropout_masked(input, scale=1.0, kv_lengths=None, dropout_prob=0.0, output=None,
                                 dropout_mask=None, stream=None, *, seed=None):
    """dropout(softmax(scale * input, axis=-1)) with the key positions >=
    kv_lengths[b] of batch item b masked inside the kernel.  ``input`` is a torch
    CUDA tensor [batch, ..., L] (FP16 or FP32); ``kv_lengths`` one int per batch
    item (tensor, array or None).  Returns ``(output, dropout_mask)``.  Extension
    (tensorfuse_b200_softmax_dropout_masked): the reference's operator has neither
    a scale nor a mask argument, callers add -inf to the scores beforehand."""
    import torch
    x = input.contiguous()
    if output is None:
        output = torch.empty_like(x)
    if dropout_mask is None:
        dropout_mask = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    _check_cuda_out("fused_softmax_dropout_masked", output, x.shape, x.dtype, x.device)
    _check_cuda_out("fused_softmax_dropout_masked", dropout_mask, x.shape, torch.uint8, x.device)
    lens_ptr = None
    if kv_lengths is not None:
        kv_lengths = torch.as_tensor(kv_lengths, dtype=torch.int32, device=x.device).contiguous()
        if kv_lengths.numel() != x.shape[0]:
            raise RuntimeError("fused_softmax_dropout_masked failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
        lens_ptr = kv_lengths.data_ptr()
    if seed is None:
        seed = _next_host_seed()
    L = x.shape[-1]
    batch = x.shape[0]
    rows_per_item = x.numel() // max(1, batch * L)
    with torch.cuda.device(x.device):
        st = _auto_init(_L.tensorfuse_b200_softmax_dropout_masked, x.data_ptr(), output.data_ptr(),
                        dropout_mask.data_ptr(), batch, rows_per_item, L, int(_torch_dt(x)), float(scale), lens_ptr,
                        float(dropout_prob), int(seed) & 0xFFFFFFFFFFFFFFFF, _torch_stream(stream, x.device))
    _check("fused_softmax_dropout_masked", st)
    return output, dropout_mask


def _softmax_torch_cuda(x, out, mask, p, stream, seed):
    import torch
    x = x.contiguous()
    if x.dim() != 4:
        raise RuntimeError("fused_softmax_dropout failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
    if out is None:
        out = torch.empty_like(x)
    if mask is None:
        mask = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    _check_cuda_out("fused_softmax_dropout", out, x.shape, x.dtype, x.device)
    _check_cuda_out("fused_softmax_dropout", mask, x.shape, torch.uint8, x.device)
    s = _torch_stream(stream, x.device)
    dt = _torch_dt(x)
    with torch.cuda.device(x.device):
        if seed is None:
            ti = _c_tensor(x.data_ptr(), tuple(x.shape), dt)
            to = _c_tensor(out.data_ptr(), tuple(out.shape), _torch_dt(out))
            st = _auto_init(_L.tensorfuse_fused_softmax_dropout, C.byref(ti), C.byref(to),
                            mask.data_ptr(), float(p), s)
        else:
            L = x.shape[-1]
            st = _L.tensorfuse_b200_softmax_dropout_rows(x.data_ptr(), out.data_ptr(), mask.data_ptr(),
                                                         x.numel() // max(L, 1), L, int(dt), float(p),
                                                         int(seed) & 0xFFFFFFFFFFFFFFFF, 0, s)
    _check("fused_softmax_dropout", st)
    return out, mask


def fused_multi_head_attention(query, key, value, output=None, num_heads=1, dropout_prob=0.0, stream=None, *,
                               seed=None, kv_lengths=None, scale=None):
    """output = dropout(softmax(scale * Q K^T)) V per head; query/output
    [batch, seq_q, hidden], key/value [batch, seq_kv, hidden], heads split hidden.

    Reference signature: fused_multi_head_attention(query, key, value, output,
    num_heads, dropout_prob, stream) (core_bindings.cpp:773-795), whose C entry
    only validates (src/tensorfuse_c_api.cpp:288-311); this one computes.  torch
    CUDA tensors run in place (last dimension contiguous; a view into a fused
    QKV buffer is fine); numpy arrays are staged through the device.  ``seed``
    fixes the dropout decisions, ``kv_lengths`` (one int per batch item) masks
    the keys from that position on, ``scale`` defaults to 1/sqrt(head width).
    """
    import torch
    if not _is_torch(query):
        if not torch.cuda.is_available():
            raise RuntimeError("fused_multi_head_attention failed: " + get_error_string(Status.CUDA_ERROR))
        q, k, v = (torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (query, key, value))
        lens = None if kv_lengths is None else torch.as_tensor(np.asarray(kv_lengths, np.int32)).cuda()
        o = fused_multi_head_attention(q, k, v, None, num_heads, dropout_prob, None, seed=seed,
                                       kv_lengths=lens, scale=scale)
        res = o.cpu().numpy()
        if output is not None:
            output[...] = res
            return output
        return res
    q, k, v = query, key, value
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3 or num_heads <= 0 or q.shape[2] % max(num_heads, 1):
        raise RuntimeError("fused_multi_head_attention failed: " + get_error_string(
            Status.INVALID_ARGUMENT if num_heads <= 0 else Status.INVALID_TENSOR_SHAPE))
    if k.shape != v.shape or k.shape[0] != q.shape[0] or k.shape[2] != q.shape[2]:
        raise RuntimeError("fused_multi_head_attention failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
    q, k, v = (t if t.stride(-1) == 1 else t.contiguous() for t in (q, k, v))
    if output is None:
        output = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    if output.shape != q.shape or output.stride(-1) != 1 or output.dtype != q.dtype:
        raise RuntimeError("fused_multi_head_attention failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise RuntimeError("fused_multi_head_attention failed: " + get_error_string(Status.INVALID_ARGUMENT))
    dt = _torch_dt(q)
    if dt not in (DataType.FLOAT16, DataType.BFLOAT16, DataType.FLOAT32):
        raise RuntimeError("fused_multi_head_attention failed: " + get_error_string(Status.UNSUPPORTED_OPERATION))
    lens_ptr = None
    if kv_lengths is not None:
        kv_lengths = torch.as_tensor(kv_lengths, dtype=torch.int32, device=q.device).contiguous()
        lens_ptr = kv_lengths.data_ptr()
    if seed is None:
        seed = _next_host_seed()
    B, Sq, H = q.shape
    hd = H // num_heads
    with torch.cuda.device(q.device):
        st = _auto_init(_L.tensorfuse_b200_attention, q.data_ptr(), k.data_ptr(), v.data_ptr(), output.data_ptr(),
                        B, Sq, k.shape[1], int(num_heads), hd, q.stride(1), k.stride(1), v.stride(1), output.stride(1),
                        0, 0, 0, 0, q.stride(0), k.stride(0), v.stride(0), output.stride(0), int(dt),
                        float(scale or 0.0), float(dropout_prob), int(seed) & 0xFFFFFFFFFFFFFFFF, lens_ptr,
                        _torch_stream(stream, q.device))
    _check("fused_multi_head_attention", st)
    return output


_LAYER_KEYS = ("query_weight", "key_weight", "value_weight", "output_weight", "query_bias", "key_bias",
               "value_bias", "output_bias", "ffn_weight1", "ffn_weight2", "ffn_bias1", "ffn_bias2",
               "ln1_weight", "ln1_bias", "ln2_weight", "ln2_bias")


def fused_transformer_layer(input, weights, num_heads, dropout_prob=0.0, layer_norm_eps=1e-12, output=None,
                            activation="gelu", use_bias=True, stream=None):
    """One post-LN encoder layer inside the library (tensorfuse_fused_transformer_layer):
    ``input``/``output`` [batch, seq, hidden] torch CUDA tensors (FP16 or FP32),
    ``weights`` a dict with the TensorFuseTransformerParams field names
    (matrices [in, out], vectors [out]).  The reference's entry point is a
    placeholder (src/tensorfuse_c_api.cpp:313-329); this one computes."""
    import torch
    from ._lib import TransformerParams
    x = input.contiguous()
    if output is None:
        output = torch.empty_like(x)
    _check_cuda_out("fused_transformer_layer", output, x.shape, x.dtype, x.device)
    dt = _torch_dt(x)
    params = TransformerParams()
    keep = []
    for name in _LAYER_KEYS:
        t = weights.get(name)
        if t is None:
            continue
        t = t.contiguous()
        ct = _c_tensor(t.data_ptr(), tuple(t.shape), _torch_dt(t))
        keep.append((t, ct))
        setattr(params, name, C.pointer(ct))
    params.num_heads = int(num_heads)
    params.dropout_prob = float(dropout_prob)
    params.ffn_activation = {"gelu": 2, "none": 0, "relu": 1}[activation]
    params.layer_norm_eps = float(layer_norm_eps)
    params.use_bias = bool(use_bias)
    params.use_flash_attention = True
    ti = _c_tensor(x.data_ptr(), tuple(x.shape), dt)
    to = _c_tensor(output.data_ptr(), tuple(output.shape), _torch_dt(output))
    with torch.cuda.device(x.device):
        st = _auto_init(_L.tensorfuse_fused_transformer_layer, C.byref(ti), C.byref(to), C.byref(params),
                        _torch_stream(stream, x.device))
    _check("fused_transformer_layer", st)
    return output


def add_layernorm(x, residual, gamma, beta, eps=1e-12, output=None, stream=None):
    """LayerNorm(x + residual) * gamma + beta over the last dimension (torch CUDA
    tensors, FP16 or FP32; residual may be None)."""
    import torch
    x = x.contiguous()
    if output is None:
        output = torch.empty_like(x)
    _check_cuda_out("add_layernorm", output, x.shape, x.dtype, x.device)
    H = x.shape[-1]
    if gamma.numel() != H or beta.numel() != H or (residual is not None and residual.shape != x.shape):
        raise RuntimeError("add_layernorm failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
    with torch.cuda.device(x.device):
        st = _auto_init(_L.tensorfuse_b200_add_layernorm, x.data_ptr(),
                        None if residual is None else residual.contiguous().data_ptr(), gamma.data_ptr(),
                        beta.data_ptr(), output.data_ptr(), x.numel() // H, H, int(_torch_dt(x)), float(eps),
                        _torch_stream(stream, x.device))
    _check("add_layernorm", st)
    return output


def quantize_int8(x, stream=None, *, per_column=False):
    """Symmetric INT8 quantisation of a torch CUDA tensor (FP16 or FP32) on the
    device: returns ``(q, scale)`` with ``q`` int8 of x's shape and ``scale`` a
    one-element FP32 CUDA tensor (= max|x|/127), or, with ``per_column=True`` for
    a weight matrix [K, N], N scales (one per output column).  Either is ready to
    be passed as a device scale to the INT8 GEMM.  No host synchronisation."""
    import torch
    if not (_is_torch(x) and x.is_cuda):
        raise RuntimeError("quantize_int8 failed: " + get_error_string(Status.INVALID_ARGUMENT))
    x = x.contiguous()
    dt = _torch_dt(x)
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    if per_column:
        if x.dim() != 2:
            raise RuntimeError("quantize_int8 failed: " + get_error_string(Status.INVALID_TENSOR_SHAPE))
        scales = torch.empty(x.shape[1], dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            st = _auto_init(_L.tensorfuse_b200_quantize_int8_columns, x.data_ptr(), int(dt), x.shape[0], x.shape[1],
                            q.data_ptr(), scales.data_ptr(), _torch_stream(stream, x.device))
        _check("quantize_int8", st)
        return q, scales
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        st = _auto_init(_L.tensorfuse_b200_quantize_int8, x.data_ptr(), int(dt), x.numel(), q.data_ptr(),
                        scale.data_ptr(), _torch_stream(stream, x.device))
    _check("quantize_int8", st)
    return q, scale


def is_gpu_supported() -> bool:
    """True on a device this build targets (compute capability 10.x)."""
    try:
        import torch
        return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10
    except Exception:
        return False


__all__ = ["Status", "DataType", "Config", "TensorFuseStatus", "TensorFuseDataType",
           "TensorFuseConfig", "init", "shutdown", "cleanup", "get_version", "get_error_string",
           "fused_gemm_bias_gelu", "fused_softmax_dropout", "fused_softmax_dropout_masked", "fused_multi_head_attention", "fused_transformer_layer", "add_layernorm", "quantize_int8",
           "set_random_seed", "device_ids", "watchdog_status", "launch_count", "softmax_schedule", "softmax_schedule_ex",
           "plan_shards", "pinned_empty", "register_weights", "invalidate_weights", "is_gpu_supported", "INT8_DEQUANT", "INT8_LEGACY",
           "INT8_RAW", "TENSORFUSE_MAX_DIMS"]
