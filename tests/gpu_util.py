"""Helpers for the GPU tests: device buffers come from torch (plumbing only),
every operator call goes through the C ABI of libtensorfuse.so."""
import ctypes as C

import numpy as np
import torch

import tensorfuse_b200 as tfm
from tensorfuse_b200._lib import lib as L

DT = tfm.DataType


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def stream() -> int:
    return int(torch.cuda.current_stream().cuda_stream)


def check_watchdog():
    torch.cuda.synchronize()
    code = L.tensorfuse_b200_watchdog_status()
    L.tensorfuse_b200_watchdog_reset()      # keep later tests independent of this one
    assert code == 0, f"device-side bounded wait expired (code {code})"


def gemm_wrapper(name, A, B, bias, out_dtype, alpha=1.0, beta=1.0, scales=None):
    """Call one of the flat *_wrapper symbols on device copies; returns host result."""
    M, K = A.shape
    N = B.shape[1]
    dA, dB, db = dev(A), dev(B), dev(bias)
    dC = torch.full((M, N), -7, dtype=out_dtype, device="cuda")
    fn = getattr(L, name)
    if scales is None:
        st = fn(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dC.data_ptr(), M, N, K, alpha, beta, stream())
    else:
        st = fn(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dC.data_ptr(), M, N, K, alpha, beta,
                scales[0], scales[1], stream())
    check_watchdog()
    return st, host(dC)


def gemm_int8(A, B, bias, scales, bias_dt, out_torch_dtype, epilogue):
    M, K = A.shape
    N = B.shape[1]
    dA, dB, db = dev(A), dev(B), dev(bias)
    dC = torch.zeros((M, N), dtype=out_torch_dtype, device="cuda")
    out_dt = {torch.float16: DT.FLOAT16, torch.float32: DT.FLOAT32, torch.int32: DT.INT32}[out_torch_dtype]
    st = L.tensorfuse_b200_gemm_int8(dA.data_ptr(), dB.data_ptr(), db.data_ptr(), dC.data_ptr(), M, N, K,
                                     scales[0], scales[1], int(bias_dt), int(out_dt), epilogue, stream())
    check_watchdog()
    return st, host(dC)


def softmax_rows(x: np.ndarray, p=0.0, seed=0, first_row=0):
    """tensorfuse_b200_softmax_dropout_rows on a device copy of x (last axis = row)."""
    Lr = x.shape[-1]
    rows = x.size // Lr if Lr else 0
    dx = dev(x)
    dout = torch.empty_like(dx)
    dmask = torch.full(x.shape, 9, dtype=torch.uint8, device="cuda")
    dt = DT.FLOAT16 if x.dtype == np.float16 else DT.FLOAT32
    st = L.tensorfuse_b200_softmax_dropout_rows(dx.data_ptr(), dout.data_ptr(), dmask.data_ptr(), rows, Lr,
                                                int(dt), float(p), int(seed), int(first_row), stream())
    torch.cuda.synchronize()
    return st, host(dout), host(dmask)


def c_tensor(t: torch.Tensor, shape=None, scale: torch.Tensor | None = None):
    dt = {torch.float32: DT.FLOAT32, torch.float16: DT.FLOAT16, torch.int8: DT.INT8,
          torch.int32: DT.INT32, torch.uint8: DT.UINT8}[t.dtype]
    return tfm._c_tensor(t.data_ptr(), tuple(shape if shape is not None else t.shape), dt,
                         None if scale is None else scale.data_ptr())


def byref(x):
    return C.byref(x)
