"""CPU: the tensor-parallel decode driver (tensorcore_b200/tp.py) on two and four gloo ranks.
The compute back end here is the CPU checker (oracle); what is under test is the host-side
logic the CUDA ranks share: shard arithmetic, which slice each rank quantises, and the order of
GEMVs, all-gathers and all-reduces of one token."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

from tensorcore_b200 import tp
from tensorcore_b200.decode import LlamaShape


def test_row_and_k_ranges_cover_everything():
    for N, P in ((4096, 8), (11008, 8), (32000, 4), (10, 3), (128256, 8)):
        parts = [tp.row_range(N, P, r) for r in range(P)]
        assert parts[0][0] == 0 and parts[-1][1] == N
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        assert max(b - a for a, b in parts) - min(b - a for a, b in parts) <= 1
    for K, P in ((4096, 8), (11008, 8), (11008, 2), (28672, 8), (8192, 4), (512, 8), (96, 2)):
        parts = tp.k_ranges(K, P)
        assert parts[0][0] == 0 and parts[-1][1] == K
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        align = 256 if K % 256 == 0 and K // 256 >= P else 32
        assert all(a % align == 0 and b % align == 0 and b > a for a, b in parts)
    # 11008 = 43 groups of 256 over 8 ranks: five or six groups each
    assert sorted({b - a for a, b in tp.k_ranges(11008, 8)}) == [1280, 1536]


def test_plan_rejects_unsplittable_shapes():
    bad = LlamaShape("bad", 1, 256, 512, 4, 4, 1001)
    with pytest.raises(ValueError):
        tp.TPPlan(bad, 2, 0).check()


class CpuBackend:
    """numpy vectors, oracle GEMVs, gloo collectives (none when world == 1)."""

    def __init__(self, shape, world):
        import oracle as O
        self.O, self.shape, self.world = O, shape, world
        self.log = []

    def weight(self, which, seed, rows, cols):
        N, K = self.shape.proj_shape(which)
        rng = np.random.default_rng(seed)
        w = (rng.standard_normal((N, K)) * (1.0 / np.sqrt(K))).astype(np.float32).astype(np.float16)
        if rows is not None:
            w = w[rows[0]:rows[1]]
        if cols is not None:
            w = w[:, cols[0]:cols[1]]
        return self.O.quantize_weights(np.ascontiguousarray(w), 0)

    def gamma(self, seed):
        rng = np.random.default_rng(seed)
        return (1.0 + 0.1 * rng.standard_normal(self.shape.d_model)).astype(np.float32)

    def empty(self, n, dtype):
        return np.zeros(n, dtype=np.float16 if dtype == "f16" else np.float32)

    def view(self, vec, a, b):
        return vec[a:b]

    def gemv(self, x, w, y, N, K, gamma=None, layout=0):
        assert x.shape == (K,) and y.shape == (N,) and w.size == N * (K // 32) * 18
        xf = x.astype(np.float32).reshape(1, K)
        if gamma is None:
            out = self.O.gemv_quantized_f32(xf, w, 0, N)[0]
        else:
            out = self.O.fused_rmsnorm_gemv_quantized_f32(xf, gamma, w, 0, N, 1e-5)[0]
        y[:] = out.astype(y.dtype)
        self.log.append(("gemv", N, K, gamma is not None))

    def all_gather(self, dst, src):
        if self.world == 1:
            dst[:] = src
        else:
            t = torch.from_numpy(dst)
            dist.all_gather_into_tensor(t, torch.from_numpy(src.copy()))
        self.log.append(("ag", dst.size))

    def all_reduce(self, vec):
        if self.world > 1:
            dist.all_reduce(torch.from_numpy(vec))
        self.log.append(("ar", vec.size))


SHAPE = LlamaShape("tiny-tp", 2, 1024, 2048, 8, 4, 1000)


def _single_process_logits():
    be = CpuBackend(SHAPE, 1)
    dec = tp.TPDecoder(tp.TPPlan(SHAPE, 1, 0), be)
    dec.x_in[:] = np.random.default_rng(1).standard_normal(SHAPE.d_model).astype(np.float32)
    dec.token()
    return dec.logits.copy(), be.log


def _rank_main(rank, world, port, ret, flow):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        be = CpuBackend(SHAPE, world)
        plan = tp.TPPlan(SHAPE, world, rank, flow)
        dec = tp.TPDecoder(plan, be)
        dec.x_in[:] = np.random.default_rng(1).standard_normal(SHAPE.d_model).astype(np.float32)
        dec.token()
        ret[rank] = (dec.logits.copy(), be.log, plan.weight_bytes_local(0))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("flow", ["local", "gathered"])
@pytest.mark.parametrize("world", [2, 4])
def test_tp_decode_matches_single_rank(world, flow, oracle):
    want, log1 = _single_process_logits()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, _free_port(), ret, flow), nprocs=world, join=True)
    per_layer = 7 if flow == "gathered" else 2
    assert sorted(ret.keys()) == list(range(world))
    total_bytes = 0
    for r in range(world):
        logits, log, nbytes = ret[r]
        total_bytes += nbytes
        # every rank ends with the same full logits
        assert np.array_equal(logits.view(np.uint16), ret[0][0].view(np.uint16))
        # same sequence of operations on every rank: 7 GEMVs per layer + lm_head; collectives:
        # two all-reduces per layer ("local") or all seven outputs ("gathered"), + the logits
        assert [e[0] for e in log] == [e[0] for e in ret[0][1]]
        assert sum(e[0] == "gemv" for e in log) == 7 * SHAPE.n_layers + 1
        assert sum(e[0] in ("ag", "ar") for e in log) == per_layer * SHAPE.n_layers + 1
    # the shards partition the model: no weight byte is held twice
    assert total_bytes == SHAPE.weight_bytes(0)
    # split-K partial sums are added in a different order and intermediate fp16 roundings may
    # flip: the bar is the fp16-activation tolerance
    assert oracle.scaled_rms(ret[0][0], want) <= 2e-3
