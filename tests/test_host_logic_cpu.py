"""Host-side logic that needs no GPU: the shard planner, the softmax schedule,
and (two gloo ranks on CPU) that a row split over ranks reproduces the
unsharded result, dropout mask included."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("rows,parts,align", [(16384, 8, 128), (16384, 3, 128), (5000, 4, 128), (100, 8, 128),
                                              (0, 2, 16), (7, 3, 1), (262144, 7, 16), (129, 2, 128)])
def test_plan_shards(rows, parts, align):
    import tensorfuse_b200 as t
    b, c = t.plan_shards(rows, parts, align)
    assert sum(c) == rows and b[0] == 0
    for i in range(parts):
        assert c[i] >= 0 and b[i] % align == 0 or c[i] == 0
        if i + 1 < parts:
            assert b[i + 1] == b[i] + c[i]
    nz = [x for x in c if x]
    if nz:
        assert max(nz) - min(nz) <= 2 * align          # balanced to one aligned block (plus the tail)


def test_softmax_schedule():
    import tensorfuse_b200 as t
    assert t.softmax_schedule(512) == (8, 1) and t.softmax_schedule(2048) == (8, 1)
    assert t.softmax_schedule(4096) == (8, 8)
    assert t.softmax_schedule(100) == (1, 1) and t.softmax_schedule(1500) == (1, 8)
    assert t.softmax_schedule(512, aligned16=False) == (1, 1)


_RANK_PROG = r'''
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from oracle import oracle as o
import tensorfuse_b200 as t
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
x = np.random.default_rng(0).standard_normal((96, 256)).astype(np.float16)       # same on both ranks
A = np.random.default_rng(1).standard_normal((96 * 4, 64)).astype(np.float16)
B = (np.random.default_rng(2).standard_normal((64, 32)) / 8).astype(np.float16)
bias = np.zeros(32, np.float16)
b, c = t.plan_shards(96, 2, 16)
r0, n = b[rank], c[rank]
part, pmask = o.softmax_dropout_exact(x[r0:r0 + n], p=0.1, seed=7, first_row=r0)
gb, gc = t.plan_shards(A.shape[0], 2, 128)
gpart = o.gemm_bias_gelu_f16(A[gb[rank]:gb[rank] + gc[rank]], B, bias)
gathered = [None, None]
dist.all_gather_object(gathered, (part, pmask, gpart))        # test-side gather only; the data path has no collective
if rank == 0:
    whole, wmask = o.softmax_dropout_exact(x, p=0.1, seed=7)
    assert np.array_equal(np.concatenate([g[0] for g in gathered]).view(np.uint16), whole.view(np.uint16))
    assert np.array_equal(np.concatenate([g[1] for g in gathered]), wmask)
    assert np.array_equal(np.concatenate([g[2] for g in gathered]).view(np.uint16),
                          o.gemm_bias_gelu_f16(A, B, bias).view(np.uint16))
dist.barrier()
dist.destroy_process_group()
'''


def test_two_rank_row_sharding_on_gloo(tmp_path):
    prog = tmp_path / "rank.py"
    prog.write_text(_RANK_PROG)
    port = str(29500 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(prog), ROOT, port, str(r)], cwd=ROOT) for r in range(2)]
    codes = [p.wait(timeout=300) for p in procs]
    assert codes == [0, 0]
