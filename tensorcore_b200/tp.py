"""Tensor-parallel decode of a Llama-shaped Q4_0 model: one process per GPU.

Sharding (the partition BASELINE's north_star prescribes):
  * q/k/v, gate/up and lm_head are split by output rows (a contiguous byte range of the block
    array); each rank computes its slice;
  * o_proj and down_proj are split along K into 256-aligned ranges (so that every shard keeps
    the kernels' fast path: whole 8-block groups, 16-byte aligned rows); each rank computes an
    fp32 partial product over its K range and the partials are all-reduced (sum).
Two data flows.  "local" (default): the row slices of q and of gate ARE the K ranges of o_proj and
down_proj, so a rank's slice feeds its own K-shard directly and k/v/up stay sharded, as they do
in a head-parallel attention / sharded SwiGLU: two all-reduces per layer plus one all-gather of
the logits (65 collectives per 7B token).  "gathered": every row-split output is all-gathered to
all ranks first (225 collectives per token), which needs equal row slices.
Norm weights and hidden states are replicated.

The arithmetic per rank is the library's own kernels (raw device-pointer launches on the
collective's stream); the plumbing - process group, collectives, graph capture - is
torch.distributed over NCCL.  A whole token (GEMVs and collectives) is captured into one CUDA
graph and replayed.

`TPPlan` and `TPDecoder` are backend-agnostic: the compute/collective back end is passed in, so
the host-side logic (shard arithmetic, data flow) is exercised on CPU ranks over gloo by the
tests with a CPU checker as the compute back end.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass

import numpy as np

from tensorcore_b200.decode import (LM_HEAD_SEED, PROJ, X_SEED, LlamaShape, gamma_fp16,
                                    tensor_seed)

K_ALIGN = 256   # K-shards keep whole 8-block groups


def row_range(N: int, P: int, r: int) -> tuple[int, int]:
    """Output-row slice of rank r: as even as possible, contiguous, in rank order."""
    base, extra = divmod(N, P)
    n0 = r * base + min(r, extra)
    return n0, n0 + base + (1 if r < extra else 0)


def k_ranges(K: int, P: int) -> list[tuple[int, int]]:
    """K slices of all ranks, each a multiple of K_ALIGN where K allows it (else of 32)."""
    align = K_ALIGN if K % K_ALIGN == 0 and K // K_ALIGN >= P else 32
    units = K // align
    out = []
    for r in range(P):
        u0, u1 = row_range(units, P, r)
        out.append((u0 * align, u1 * align))
    return out


# row-split projection -> the K-split projection its output feeds in the "local" data flow
FEEDS = {"attn_q": "attn_output", "attn_k": "attn_output", "attn_v": "attn_output",
         "ffn_gate": "ffn_down", "ffn_up": "ffn_down"}


@dataclass
class TPPlan:
    shape: LlamaShape
    world: int
    rank: int
    flow: str = "local"     # "local" | "gathered"

    def col(self, which: str) -> tuple[int, int]:
        N, _ = self.shape.proj_shape(which)
        if self.flow == "local" and which in FEEDS:
            # the consumer's K range, scaled when the producer has fewer rows (grouped-query k/v)
            Kc = self.shape.proj_shape(FEEDS[which])[1]
            k0, k1 = k_ranges(Kc, self.world)[self.rank]
            if N == Kc:
                return k0, k1
        return row_range(N, self.world, self.rank)

    def kslice(self, which: str) -> tuple[int, int]:
        _, K = self.shape.proj_shape(which)
        return k_ranges(K, self.world)[self.rank]

    def equal_cols(self, which: str) -> bool:
        N, _ = self.shape.proj_shape(which)
        return N % self.world == 0

    def check(self) -> None:
        gathered = ("attn_q", "attn_k", "attn_v", "ffn_gate", "ffn_up", "output")
        for p in (gathered if self.flow == "gathered" else ("output",)):
            if not self.equal_cols(p):
                raise ValueError(f"{p}: {self.shape.proj_shape(p)[0]} rows do not divide by "
                                 f"{self.world} ranks (all-gather needs equal slices)")
        for p in ("attn_output", "ffn_down"):
            k0, k1 = self.kslice(p)
            if k1 <= k0:
                raise ValueError(f"{p}: empty K shard on rank {self.rank}")

    def weight_bytes_local(self, fmt: int = 0) -> int:
        bb = 18 if fmt == 0 else 34
        total = 0
        for p in PROJ:
            N, K = self.shape.proj_shape(p)
            if p in ("attn_output", "ffn_down"):
                k0, k1 = self.kslice(p)
                total += N * ((k1 - k0) // 32) * bb * self.shape.n_layers
            else:
                n0, n1 = self.col(p)
                total += (n1 - n0) * (K // 32) * bb * self.shape.n_layers
        n0, n1 = self.col("output")
        total += (n1 - n0) * (self.shape.d_model // 32) * bb
        return total


class TPDecoder:
    """Data flow of one decode token on one rank.  `be` supplies:
         be.weight(which, layer, rows=(n0,n1) | None, cols=(k0,k1) | None) -> weight handle
         be.gamma(seed) -> gamma handle (fp32)
         be.empty(n, dtype) -> activation vector ("f16" | "f32")
         be.gemv(x, w, y, N, K, gamma=None)       # dtype taken from the vectors
         be.all_gather(dst_full, src_local); be.all_reduce(vec)
         be.view(vec, a, b) -> sub-vector
    """

    def __init__(self, plan: TPPlan, be, fmt: int = 0):
        plan.check()
        self.plan, self.be, self.fmt = plan, be, fmt
        s, P = plan.shape, plan.world
        self.w = []
        for l in range(s.n_layers):
            lw = {}
            for t, p in enumerate(PROJ):
                if p in ("attn_output", "ffn_down"):
                    lw[p] = be.weight(p, tensor_seed(l, t), None, plan.kslice(p))
                else:
                    lw[p] = be.weight(p, tensor_seed(l, t), plan.col(p), None)
            lw["attn_norm"] = be.gamma(0x7CB000 + l)
            lw["ffn_norm"] = be.gamma(0x7CC000 + l)
            self.w.append(lw)
        self.out_norm = be.gamma(0x7CD000)
        self.lm_head = be.weight("output", LM_HEAD_SEED, plan.col("output"), None)
        d, f, kv, V = s.d_model, s.d_ff, s.d_kv, s.vocab
        self.x_in = be.empty(d, "f32")
        self.h = [be.empty(d, "f32"), be.empty(d, "f32")]
        self.o = be.empty(d, "f32")
        def loc(which):
            n0, n1 = plan.col(which)
            return be.empty(n1 - n0, "f16")
        self.q_loc, self.k_loc, self.v_loc = loc("attn_q"), loc("attn_k"), loc("attn_v")
        self.g_loc, self.u_loc = loc("ffn_gate"), loc("ffn_up")
        self.l_loc, self.logits = be.empty(V // P, "f16"), be.empty(V, "f16")
        if plan.flow == "gathered":
            self.q, self.k, self.v = be.empty(d, "f16"), be.empty(kv, "f16"), be.empty(kv, "f16")
            self.g, self.u = be.empty(f, "f16"), be.empty(f, "f16")

    def token(self) -> None:
        """x_in -> logits.  Same stand-ins as the single-GPU harness: q feeds o_proj, gate
        feeds down_proj; hidden states are fp32 (the all-reduced partial sums)."""
        be, s, plan = self.be, self.plan.shape, self.plan
        d = s.d_model
        gathered = plan.flow == "gathered"
        cur = self.x_in
        for l, lw in enumerate(self.w):
            nxt = self.h[l & 1]
            for p, y in (("attn_q", self.q_loc), ("attn_k", self.k_loc), ("attn_v", self.v_loc)):
                n0, n1 = plan.col(p)
                be.gemv(cur, lw[p], y, n1 - n0, d, gamma=lw["attn_norm"])
            k0, k1 = plan.kslice("attn_output")
            if gathered:
                be.all_gather(self.q, self.q_loc)
                be.all_gather(self.k, self.k_loc)
                be.all_gather(self.v, self.v_loc)
                q_in = be.view(self.q, k0, k1)
            else:
                q_in = self.q_loc                    # this rank's q rows are its o_proj K range
            be.gemv(q_in, lw["attn_output"], self.o, d, k1 - k0)
            be.all_reduce(self.o)
            for p, y in (("ffn_gate", self.g_loc), ("ffn_up", self.u_loc)):
                n0, n1 = plan.col(p)
                be.gemv(self.o, lw[p], y, n1 - n0, d, gamma=lw["ffn_norm"])
            k0, k1 = plan.kslice("ffn_down")
            if gathered:
                be.all_gather(self.g, self.g_loc)
                be.all_gather(self.u, self.u_loc)
                g_in = be.view(self.g, k0, k1)
            else:
                g_in = self.g_loc
            be.gemv(g_in, lw["ffn_down"], nxt, d, k1 - k0)
            be.all_reduce(nxt)
            cur = nxt
        n0, n1 = plan.col("output")
        be.gemv(cur, self.lm_head, self.l_loc, n1 - n0, d, gamma=self.out_norm)
        be.all_gather(self.logits, self.l_loc)

    def gemvs_per_token(self) -> int:
        return 7 * self.plan.shape.n_layers + 1

    def collectives_per_token(self) -> int:
        return (7 if self.plan.flow == "gathered" else 2) * self.plan.shape.n_layers + 1


# ---------------------------------------------------------------------------------------
# CUDA / NCCL back end
# ---------------------------------------------------------------------------------------
class CudaBackend:
    def __init__(self, ctx, shape: LlamaShape, fmt: int, device):
        import torch
        import torch.distributed as dist

        import tensorcore_b200 as tc
        self.torch, self.dist, self.tc = torch, dist, tc
        self.ctx, self.shape, self.fmt, self.device = ctx, shape, fmt, device
        self.keep = []
        self.launches = 0
        self.collectives = 0

    def weight(self, which, seed, rows, cols):
        from tensorcore_b200.decode import device_weights_fp16, quantize_into
        N, K = self.shape.proj_shape(which)
        w = device_weights_fp16(N, K, seed, self.device)
        if rows is not None:
            w = w[rows[0]:rows[1]].contiguous()
        if cols is not None:
            w = w[:, cols[0]:cols[1]].contiguous()
        buf = quantize_into(self.ctx, w, self.fmt)
        self.keep.append(buf)
        del w
        return buf.device_ptr()

    def gamma(self, seed):
        g = self.torch.from_numpy(gamma_fp16(self.shape.d_model, seed).astype(np.float32)).to(self.device)
        self.keep.append(g)
        return g

    def empty(self, n, dtype):
        t = self.torch.zeros(n, dtype=self.torch.float16 if dtype == "f16" else self.torch.float32,
                             device=self.device)
        self.keep.append(t)
        return t

    def view(self, vec, a, b):
        return vec[a:b]

    def gemv(self, x, w, y, N, K, gamma=None):
        tc, torch = self.tc, self.torch
        xd = "f32" if x.dtype == torch.float32 else "f16"
        yd = "f32" if y.dtype == torch.float32 else "f16"
        st = torch.cuda.current_stream().cuda_stream
        if gamma is None:
            tc.raw_gemv_quantized(self.ctx, x.data_ptr(), w, y.data_ptr(), self.fmt, 1, N, K, xd, yd, st)
        else:
            assert gamma.dtype == x.dtype
            tc.raw_fused_rmsnorm_gemv_quantized(self.ctx, x.data_ptr(), gamma.data_ptr(), w,
                                                y.data_ptr(), self.fmt, 1, N, K, 1e-5, xd, yd, st)
        self.launches += 1

    def all_gather(self, dst, src):
        self.dist.all_gather_into_tensor(dst, src)
        self.collectives += 1

    def all_reduce(self, vec):
        self.dist.all_reduce(vec)
        self.collectives += 1


def run_bench(args):
    """bench.py's N>1 leg: launched under torch.distributed.run, one rank per GPU."""
    import torch
    import torch.distributed as dist

    import tensorcore_b200 as tc
    from bench import (METRIC, UNIT, ClockSampler, algorithmic_bytes_per_token, measured_peaks)
    from tensorcore_b200 import decode as D

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if "MASTER_ADDR" not in os.environ:
        raise SystemExit("bench.py --gpus N>1 must be launched with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    ctx = tc.Context()          # binds the device that is current in this thread
    shape = D.LLAMA_7B
    plan = TPPlan(shape, world, rank)
    be = CudaBackend(ctx, shape, 0, device)
    dec = TPDecoder(plan, be, 0)
    rng = np.random.default_rng(X_SEED)
    x = rng.standard_normal(shape.d_model).astype(np.float32)
    hx = torch.from_numpy(x.copy()).pin_memory()
    hl = torch.empty(shape.vocab, dtype=torch.float16).pin_memory()
    dec.x_in.copy_(hx, non_blocking=False)

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for _ in range(3):                      # warm-up outside capture (NCCL setup)
            dec.token()
        stream.synchronize()
        be.launches = be.collectives = 0
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            dec.token()
        per_token_launches = be.launches
        for _ in range(max(3, args.warmup)):
            graph.replay()
        stream.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        gpu_ms = float(ms.item())

        # end to end: input from pinned host memory in, logits out, every step
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            dec.x_in.copy_(hx, non_blocking=True)
            graph.replay()
            hl.copy_(dec.logits, non_blocking=True)
            stream.synchronize()
        dist.barrier()
        wall = torch.tensor([time.perf_counter() - t0], device=device)
        dist.all_reduce(wall, op=dist.ReduceOp.MAX)
        e2e_s = float(wall.item())
    finite = bool(torch.isfinite(dec.logits.float()).all().item())
    err = tc.take_device_error(ctx)
    dist.barrier()
    out = None
    if rank == 0:
        if not finite or err:
            raise SystemExit(f"invalid run: finite={finite} device_error={err}")
        total_b, weight_b = algorithmic_bytes_per_token(shape)
        ms_per_step = gpu_ms / args.steps
        peak, peak_kind = measured_peaks()
        achieved = total_b / (ms_per_step * 1e-3) / 1e9
        out = {
            "metric": METRIC, "value": 1e3 / ms_per_step, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "s16 x u4 -> s32 (dp2a), f32 scales", "data": "synthetic",
            "config": {
                "workload": "llama-7b-shape Q4_0 decode weight stream, batch 1, tensor parallel: "
                            "q/k/v/gate/up split by rows feeding this rank's K-shard of o/down "
                            "(split along K + all-reduce), lm_head split by rows + all-gather; one "
                            "CUDA graph per token",
                "parallelism": f"tp{world}", "gemvs_per_token": dec.gemvs_per_token(),
                "collectives_per_token": dec.collectives_per_token(),
                "weight_bytes_per_token": weight_b,
                "weight_bytes_per_rank": plan.weight_bytes_local(0),
                "l2": f"{plan.weight_bytes_local(0) / 1e6:.0f} MB of weights per rank per step "
                      "(126 MB L2): no flush needed",
            },
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak * world, "unit": "GB/s",
                         "frac": achieved / (peak * world), "traffic": None, "peak_kind": peak_kind,
                         "note": "aggregate algorithmic bytes over all ranks / step time; at batch 1 "
                                 "the step is bound by collective latency, not HBM"},
            "e2e": {"value": args.steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": shape.d_model * 4,
                    "d2h_bytes_per_step": shape.vocab * 2},
            "gpu_launches": per_token_launches * args.steps,
            "clocks": clocks,
        }
    # Tear-down order matters: a CUDA graph that holds captured NCCL kernels must be released
    # before the communicator is destroyed (destroying first blocks forever).
    del graph
    torch.cuda.synchronize()
    dist.barrier()
    return out


def shutdown() -> None:
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()
