"""Softmax+dropout on long rows and on the streaming kernel, against the CPU oracle.

Three kernels beyond the warp-per-row one are exercised here, all bit-exact
against oracle.softmax_dropout_exact evaluated with the schedule the library
reports (tensorfuse_b200_softmax_schedule_ex):
  * the streaming kernel (copy-engine fed ring of row tiles) that large
    problems with rows of at most 4 KB take,
  * the shared-memory resident CTA-per-row kernel for rows up to 200 KiB
    (replaces the reference's three global sweeps per row,
    src/kernels/fused_softmax_dropout.cu:39-158),
  * the online kernel (running maximum, rescaled partial sums) beyond that.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _exact(oracle, tf, x, **kw):
    vec, warps, online = tf.softmax_schedule_ex(x.shape[-1], x.dtype, True)
    return oracle.softmax_dropout_exact(x, vec=vec, warps=warps, online=bool(online), **kw), (vec, warps, online)


def _bits(a):
    return a.view(np.uint16 if a.dtype == np.float16 else np.uint32)


@pytest.mark.parametrize("dtype,rows,L", [
    (np.float16, 5000, 512),      # streaming kernel, 2 rows per warp and tile, ragged last tile (5000 % 16 = 8)
    (np.float16, 4100, 256),      # 4 rows per warp and tile
    (np.float16, 4099, 1024),     # 1 row per warp and tile, odd row count
    (np.float16, 4200, 2048),     # widest streaming row (4 KB)
    (np.float16, 4500, 48),       # short rows: most lanes idle
    (np.float32, 4300, 512),
    (np.float32, 4100, 1024),     # widest FP32 streaming row
])
@pytest.mark.parametrize("p", [0.0, 0.1])
def test_streaming_kernel_bit_exact(tf, oracle, dtype, rows, L, p):
    from gpu_util import check_watchdog, softmax_rows
    r = np.random.default_rng(rows + L)
    x = r.uniform(-3, 3, (rows, L)).astype(dtype)
    x[7, L // 2:] = -np.inf
    x[11, :] = -np.inf
    st, out, mask = softmax_rows(x, p=p, seed=77, first_row=123)
    check_watchdog()
    assert st == 0
    (want, wmask), sched = _exact(oracle, tf, x, p=p, seed=77, first_row=123)
    assert sched == (8, 1, 0)
    assert np.array_equal(mask, wmask)
    bad = np.argwhere(_bits(out) != _bits(want))
    if len(bad):                                   # say which rows, and whose data they hold
        rows_bad = np.unique(bad[:, 0])
        base = oracle.np_softmax(np.where(np.isfinite(x[:]), x, -1e30).astype(np.float64))
        src = []
        for rb in rows_bad[:6]:
            kept = mask[rb] == 1
            got = out[rb].astype(np.float64)[kept] * (1 - p)
            err = np.abs(base[:, kept] - got).sum(-1)
            o = out[rb].astype(np.float64); w = want[rb].astype(np.float64)
            nz = (o != 0) & (w != 0)
            ratio = o[nz] / w[nz]
            src.append((int(rb), int(np.argmin(err)), float(err.min()), "ratio min/max", float(ratio.min()), float(ratio.max()),
                        "kept-but-zero", int(((o == 0) & (w != 0)).sum()), "dropped-but-nonzero", int(((o != 0) & (w == 0)).sum()),
                        "first/last bad col", int(bad[bad[:, 0] == rb][0, 1]), int(bad[bad[:, 0] == rb][-1, 1])))
        raise AssertionError(f"{len(bad)} mismatches in rows {rows_bad.tolist()[:40]}; (row, best matching source row, "
                             f"L1 distance): {src}")
    assert np.all(out[11] == 0)


@pytest.mark.parametrize("dtype,rows,L", [
    (np.float16, 2300, 4096),     # two row buffers per CTA, more rows than resident CTAs
    (np.float16, 37, 8192),
    (np.float16, 9, 8200),        # not a multiple of 128 bytes
    (np.float32, 300, 4096),
    (np.float16, 700, 32768),     # 64 KB rows: one buffer per CTA, several rows per CTA
    (np.float32, 12, 51200),      # 200 KiB: the largest shared-memory resident row
])
@pytest.mark.parametrize("p", [0.0, 0.1])
def test_smem_resident_rows_bit_exact(tf, oracle, dtype, rows, L, p):
    from gpu_util import check_watchdog, softmax_rows
    r = np.random.default_rng(L)
    x = r.uniform(-4, 4, (rows, L)).astype(dtype)
    x[1, L - 1000:] = -np.inf
    x[2, :] = -np.inf
    st, out, mask = softmax_rows(x, p=p, seed=5)
    check_watchdog()
    assert st == 0
    (want, wmask), sched = _exact(oracle, tf, x, p=p, seed=5)
    assert sched == (8, 8, 0)
    assert np.array_equal(mask, wmask)
    assert np.array_equal(_bits(out), _bits(want))
    if p == 0.0:
        live = np.isfinite(x).any(-1)                      # a fully masked row is defined as zeros
        np.testing.assert_allclose(out[live].astype(np.float64), oracle.np_softmax(x[live].astype(np.float64)),
                                   rtol=2e-3 if dtype == np.float16 else 1e-4, atol=1e-6)
        assert np.all(out[~live] == 0)


@pytest.mark.parametrize("dtype,rows,L", [(np.float16, 6, 106496), (np.float32, 5, 53248), (np.float16, 300, 102408)])
@pytest.mark.parametrize("p", [0.0, 0.1])
def test_online_rows_bit_exact(tf, oracle, dtype, rows, L, p):
    from gpu_util import check_watchdog, softmax_rows
    r = np.random.default_rng(L + 1)
    x = r.uniform(-4, 4, (rows, L)).astype(dtype)
    # a late maximum forces rescaling of the partial sums; masked stretches and a masked row
    x[0, L - 5] = 9.0
    x[1, : L // 2] = -np.inf
    x[2, :] = -np.inf
    x[3, 1000:] = -np.inf
    st, out, mask = softmax_rows(x, p=p, seed=9)
    check_watchdog()
    assert st == 0
    (want, wmask), sched = _exact(oracle, tf, x, p=p, seed=9)
    assert sched == (8, 8, 1)
    assert np.array_equal(mask, wmask)
    assert np.array_equal(_bits(out), _bits(want))
    if p == 0.0:
        live = np.isfinite(x).any(-1)
        np.testing.assert_allclose(out[live].astype(np.float64), oracle.np_softmax(x[live].astype(np.float64)),
                                   rtol=2e-3 if dtype == np.float16 else 1e-4, atol=1e-7)
        assert np.all(out[2] == 0)


def test_long_rows_full_size_properties(tf, oracle):
    """[4, 16, 512, 8192] FP16 (268 M elements): sampled rows against the oracle,
    and size-independent properties on the whole tensor."""
    import torch
    from gpu_util import L as lib, stream
    rows, Lr = 4 * 16 * 512, 8192
    g = torch.Generator(device="cuda"); g.manual_seed(8)
    x = (torch.randn((rows, Lr), generator=g, device="cuda") * 2).half()
    out = torch.empty_like(x); mask = torch.empty((rows, Lr), dtype=torch.uint8, device="cuda")
    assert lib.tensorfuse_b200_softmax_dropout_rows(x.data_ptr(), out.data_ptr(), mask.data_ptr(), rows, Lr, 1, 0.1,
                                                    21, 0, stream()) == 0
    torch.cuda.synchronize()
    assert tf.watchdog_status() == 0
    keep = mask.float().mean().item()
    assert abs(keep - 0.9) < 1e-3
    assert bool((out[mask == 0] == 0).all())               # (kept probabilities may underflow to 0 in FP16 too)
    sums = out.float().sum(-1)
    assert abs(sums.mean().item() - 1.0) < 2e-3            # E[kept/(1-p)] = 1
    idx = torch.tensor([0, 1, 777, 16383, 16384, rows - 1], device="cuda")
    xs = x[idx].cpu().numpy()
    for k, r in enumerate(idx.tolist()):
        (want, wmask), _ = _exact(oracle, tf, xs[k:k + 1], p=0.1, seed=21, first_row=r)
        assert np.array_equal(mask[r].cpu().numpy(), wmask[0])
        assert np.array_equal(out[r].cpu().numpy().view(np.uint16), want[0].view(np.uint16))
    # idempotent launch: same seed, same bytes
    out2 = torch.empty_like(x); mask2 = torch.empty_like(mask)
    assert lib.tensorfuse_b200_softmax_dropout_rows(x.data_ptr(), out2.data_ptr(), mask2.data_ptr(), rows, Lr, 1, 0.1,
                                                    21, 0, stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, out2) and torch.equal(mask, mask2)


def test_forced_streaming_form_in_a_child_process():
    """By default small problems stay on the warp-per-row kernel; with
    TENSORFUSE_B200_SOFTMAX_FORM=stream (read once per process) every eligible
    shape takes the streaming kernel, dropout-generator warps included.  The
    whole bit-exact softmax suite must pass that way as well."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, TENSORFUSE_B200_SOFTMAX_FORM="stream")
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider",
                        os.path.join(here, "test_softmax_gpu.py"), os.path.join(here, "test_softmax_masked_gpu.py"),
                        os.path.join(here, "test_softmax_long_gpu.py") + "::test_streaming_kernel_bit_exact"],
                       env=env, capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
