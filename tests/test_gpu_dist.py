"""GPU: the reference's collective API (tc_dist_init / tc_allreduce / tc_broadcast / tc_allgather /
tc_barrier, include/tensorcore/distributed.h:51-87) on device buffers.  One rank always; two
ranks - one process per GPU over NCCL, rendezvous on 127.0.0.1 - when the box has two GPUs."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_single_rank_collectives(tc, ctx):
    d = tc.DistContext(ctx, tc.TC_DIST_SINGLE, 1, 0)
    assert d.world_size() == 1 and d.rank() == 0
    x = np.arange(1000, dtype=np.float32)
    bx, by = ctx.buffer_from_array(x), ctx.buffer(x.nbytes)
    d.allreduce(bx, x.size, "f32", "sum")
    d.broadcast(bx, x.size, "f32", 0)
    d.allgather(bx, by, x.size, "f32")
    d.barrier()
    assert np.array_equal(bx.to_numpy(x.shape, np.float32), x)
    assert np.array_equal(by.to_numpy(x.shape, np.float32), x)
    with pytest.raises(tc.TensorcoreError):
        d.allreduce(bx, x.size, tc.TC_DTYPE_BF16, "sum")          # only fp16 and fp32 are carried
    with pytest.raises(tc.TensorcoreError):
        tc.DistContext(ctx, tc.TC_DIST_SINGLE, 2, 0)
    d.close()
    bx.close(); by.close()


RANK_SCRIPT = r"""
import os, sys
sys.path.insert(0, os.environ["TCB_ROOT"])
import numpy as np
import tensorcore_b200 as tc
rank, world, url = int(os.environ["TCB_RANK"]), int(os.environ["TCB_WORLD"]), os.environ["TCB_URL"]
ctx = tc.Context()
d = tc.DistContext(ctx, tc.TC_DIST_RING, world, rank, url)
assert d.world_size() == world and d.rank() == rank
n = 4096 + 3
x = (np.arange(n, dtype=np.float32) + 1000 * rank)
b = ctx.buffer_from_array(x)
d.allreduce(b, n, "f32", "sum")
want = sum(np.arange(n, dtype=np.float32) + 1000 * r for r in range(world))
assert np.array_equal(b.to_numpy((n,), np.float32), want)
h = (np.ones(n) * (rank + 1)).astype(np.float16)
bh = ctx.buffer_from_array(h)
d.allreduce(bh, n, "f16", "max")
assert np.all(bh.to_numpy((n,), np.float16) == world)
d.allreduce(bh, n, "f16", "avg")
assert np.all(bh.to_numpy((n,), np.float16) == world)
g_in = ctx.buffer_from_array(np.full(100, rank, np.float16))
g_out = ctx.buffer(100 * world * 2)
d.allgather(g_in, g_out, 100, "f16")
got = g_out.to_numpy((world, 100), np.float16)
assert all(np.all(got[r] == r) for r in range(world))
bb = ctx.buffer_from_array(np.full(64, float(rank), np.float32))
d.broadcast(bb, 64, "f32", world - 1)
assert np.all(bb.to_numpy((64,), np.float32) == world - 1)
d.barrier()
d.close()
ctx.close()
print("rank", rank, "ok")
"""


def test_two_rank_collectives_over_nccl(tc, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    procs = []
    for r in range(2):
        env = dict(os.environ, TCB_ROOT=ROOT, TCB_RANK=str(r), TCB_WORLD="2", TCB_URL="nccl+tcp://127.0.0.1:29741",
                   TC_CUDA_DEVICE=str(r), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in o, o
