"""The allocation-free softmax+dropout entry point against the allocating one.

Some callers of the host-buffer operators cannot let a library allocate device
memory: their process has given all of it to another allocator, or they run
where the synchronisation hidden in cudaMalloc / cudaFree is not acceptable.
tensorfuse_b200_softmax_dropout_host_noalloc stages its operands in a fixed
16 MiB area inside the library image instead.  This test calls it through the C
ABI twice in a row -- the second call on a smaller, different tensor, so that
anything left in the shared staging area by the first call would show -- and
requires the bytes of tensorfuse_b200_softmax_dropout_host (the tolerance of the
softmax tests is bit-exactness).  It is collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(fn, x, p, seed, *extra):
    out = np.full_like(x, 7)
    mask = np.full(x.shape, 9, np.uint8)
    L = x.shape[-1]
    st = fn(x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), mask.ctypes.data_as(C.c_void_p),
            x.size // L, L, 1 if x.dtype == np.float16 else 0, p, seed, *extra)
    return st, out, mask


def test_noalloc_matches_allocating_entry_point_twice(tf):
    from tensorfuse_b200._lib import lib as L
    r = np.random.default_rng(123)
    first = r.standard_normal((2, 4, 128, 512)).astype(np.float16)     # 2.6 MB of staging
    second = (r.standard_normal((1, 3, 40, 264)) * 2).astype(np.float32)  # smaller, other dtype
    second[0, 1, 5, 100:] = -np.inf
    for x, p, seed in ((first, 0.1, 11), (second, 0.25, 12)):
        st_ref, out_ref, mask_ref = _run(L.tensorfuse_b200_softmax_dropout_host, x, p, seed)
        st_new, out_new, mask_new = _run(L.tensorfuse_b200_softmax_dropout_host_noalloc, x, p, seed, None)
        assert st_ref == 0 and st_new == 0
        assert np.array_equal(out_new.view(np.uint8), out_ref.view(np.uint8))
        assert np.array_equal(mask_new, mask_ref)
        assert set(np.unique(mask_new)) <= {0, 1}


def test_noalloc_rejects_what_does_not_fit(tf):
    from tensorfuse_b200._lib import lib as L
    big = np.zeros((4, 16, 512, 512), np.float16)       # 16 Mi elements: 80 MiB of staging
    st, out, mask = _run(L.tensorfuse_b200_softmax_dropout_host_noalloc, big, 0.0, 1, None)
    assert st == 3 and tf.get_error_string(st) == "Out of memory"
    assert out[0, 0, 0, 0] == 7 and mask[0, 0, 0, 0] == 9   # nothing was written
    st, _, _ = _run(L.tensorfuse_b200_softmax_dropout_host_noalloc, big[:1, :1, :8], 1.5, 1, None)
    assert st == 1
