#!/usr/bin/env python
"""Benchmark of the quantized-decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): synthetic Llama-7B-shape decode weight stream, batch 1, all Q4_0 - 32 layers of
q/k/v/o 4096x4096, gate/up 11008x4096, down 4096x11008 plus lm_head 32000x4096, seeded
N(0, 0.02^2) weights packed into a GGUF v3 file and loaded with tc_gguf_load_supported_tensors.
A step is one decode token: 225 quantized GEMVs (RMSNorm fused into q/k/v, gate/up and lm_head)
recorded on a tc_stream and synchronised once.  Metric: tokens per second (whole job).

Prints one JSON line.  `value` is measured with the model and activations resident in HBM;
`e2e` runs the same steps with the step input copied from pinned host memory and the logits
copied back every step.  `--impl reference` times the reference's own CPU implementation of
the same GEMV sequence on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "synthetic 7B Q4_0 decode tok/s"
TRAFFIC_RATIO = 1.0087   # DRAM bytes / algorithmic bytes of the persistent decode kernel (ncu, see profiles/)
UNIT = "tok/s"


def measured_peaks() -> tuple[float, str]:
    """HBM GB/s denominator: the driver-measured copy bandwidth, else the stated fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 50 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(np.max(mx)) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def algorithmic_bytes_per_token(shape, fmt: int = 0) -> tuple[int, int]:
    """(total, weights only).  Per GEMV: N*(K/32)*18 weight bytes + K*2 activation bytes read +
    N*2 result bytes written (+ K*2 gamma bytes where the RMSNorm prologue is fused)."""
    from tensorcore_b200.decode import PROJ
    total = 0
    fused = {"attn_q", "attn_k", "attn_v", "ffn_gate", "ffn_up", "output"}
    items = [(p, shape.n_layers) for p in PROJ] + [("output", 1)]
    for p, count in items:
        n, k = shape.proj_shape(p)
        per = n * (k // 32) * (18 if fmt == 0 else 34) + k * 2 + n * 2
        if p in fused:
            per += k * 2
        total += per * count
    return total, shape.weight_bytes(fmt)


# ---------------------------------------------------------------------------------------
# Reference arm / CPU baseline: the reference's CPU code on the host cores
# ---------------------------------------------------------------------------------------
class CpuDecode:
    """The same GEMV sequence on the host, through the reference's portable-CPU library
    (oracle/_ref, kind "reference") or, when that was not built, the oracle port (kind "port").
    Every GEMV is split by output rows over `threads` host threads; the reference code itself
    is single-threaded scalar C++ (lib/ops/quantized_cpu.cpp has no threading)."""

    def __init__(self, shape, layers: int, threads: int):
        import oracle as O
        self.O, self.shape, self.layers, self.threads = O, shape, layers, threads
        self.kind = "reference" if O.ref_available() else "port"
        rng = np.random.default_rng(0x7C0000)
        from tensorcore_b200.decode import PROJ
        self.w = {}
        # one set of weights per projection kind, reused for every layer of the sample: the CPU
        # loops are compute-bound (0.3 GB/s per core), so cache residency does not help them.
        for p in list(PROJ) + ["output"]:
            n, k = shape.proj_shape(p)
            self.w[p] = rng.integers(0, 256, n * (k // 32) * 18, dtype=np.uint8)
            blocks = self.w[p].reshape(-1, 18)
            blocks[:, 0:2] = np.frombuffer(np.float16(0.005).tobytes(), dtype=np.uint8)
        self.x = rng.standard_normal((1, shape.d_model)).astype(np.float16)
        self.xff = rng.standard_normal((1, shape.d_ff)).astype(np.float16)
        self.ref = O.RefLib() if self.kind == "reference" else None
        from concurrent.futures import ThreadPoolExecutor
        self.pool = ThreadPoolExecutor(max_workers=threads)
        self._bufs = {}
        if self.ref is not None:
            self._prepare_ref()

    def _prepare_ref(self):
        """Row-sliced tc_buffers over the numpy arrays (tc_buffer_from_ptr, zero copy)."""
        import ctypes
        L, ctx = self.ref.L, self.ref.ctx
        L.tc_buffer_from_ptr.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                         ctypes.POINTER(ctypes.c_void_p)]

        def wrap(ptr, nbytes):
            h = ctypes.c_void_p()
            assert L.tc_buffer_from_ptr(ctx, ctypes.c_void_p(int(ptr)), int(nbytes), ctypes.byref(h)) == 0
            return h
        self.y = {}
        for p, w in self.w.items():
            n, k = self.shape.proj_shape(p)
            row = (k // 32) * 18
            self.y[p] = np.zeros((1, n), dtype=np.float16)
            xin = self.xff if k == self.shape.d_ff else self.x
            xb = wrap(xin.ctypes.data, xin.nbytes)
            cuts = np.linspace(0, n, self.threads + 1).astype(int)
            parts = []
            for a, b in zip(cuts[:-1], cuts[1:]):
                if b > a:
                    parts.append((xb, wrap(w.ctypes.data + a * row, (b - a) * row),
                                  wrap(self.y[p].ctypes.data + a * 2, (b - a) * 2), b - a, k))
            self._bufs[p] = parts

    def gemv(self, p):
        n, k = self.shape.proj_shape(p)
        if self.ref is not None:
            L, ctx = self.ref.L, self.ref.ctx

            def run(part):
                xb, wb, yb, rows, kk = part
                st = L.tc_gemv_quantized(ctx, xb, wb, yb, 0, 1, int(rows), int(kk))
                assert st == 0, st
            list(self.pool.map(run, self._bufs[p]))
        else:
            O = self.O
            xin = self.xff if k == self.shape.d_ff else self.x
            y = np.zeros((1, n), dtype=np.uint16)
            cuts = np.linspace(0, n, self.threads + 1).astype(int)
            list(self.pool.map(lambda ab: O.gemv_quantized_rows(xin, self.w[p], y, 0, n, int(ab[0]), int(ab[1])),
                               [(a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]))

    def step(self, with_lm_head: bool):
        from tensorcore_b200.decode import PROJ
        for _ in range(self.layers):
            for p in PROJ:
                self.gemv(p)
        if with_lm_head:
            self.gemv("output")

    def seconds_per_token(self, steps: int, warmup: int) -> tuple[float, float]:
        """Times `steps` samples (self.layers layers + lm_head each) and scales to one full token
        by weight bytes.  Returns (seconds per token, seconds per sample)."""
        from tensorcore_b200.decode import PROJ
        for _ in range(warmup):
            self.step(True)
        t0 = time.perf_counter()
        for _ in range(steps):
            self.step(True)
        dt = (time.perf_counter() - t0) / steps
        layer_bytes = sum(self.w[p].nbytes for p in PROJ)
        sample_bytes = self.layers * layer_bytes + self.w["output"].nbytes
        full_bytes = self.shape.n_layers * layer_bytes + self.w["output"].nbytes
        return dt * full_bytes / sample_bytes, dt


def workload_text(shape) -> str:
    return (f"llama-7b-shape Q4_0 decode weight stream, batch 1: {shape.n_layers} layers x "
            "(q,k,v,o 4096x4096; gate,up 11008x4096; down 4096x11008) + lm_head "
            "32000x4096, RMSNorm fused into q/k/v, gate/up and lm_head")


def run_reference_arm(args) -> dict:
    from tensorcore_b200.decode import LLAMA_7B
    shape = LLAMA_7B
    cores = os.cpu_count() or 1
    # size the sample so that one step is a few seconds of host work at most
    probe = CpuDecode(shape, layers=1, threads=cores)
    t0 = time.perf_counter()
    probe.step(False)
    t_layer = time.perf_counter() - t0
    per_step_budget = 120.0 / max(1, args.steps + args.warmup)   # whole run within ~2 minutes
    layers = int(max(1, min(shape.n_layers, per_step_budget / max(t_layer, 1e-3))))
    probe.layers = layers
    spt, per_sample = probe.seconds_per_token(args.steps, args.warmup)
    value = 1.0 / spt
    total_b, weight_b = algorithmic_bytes_per_token(shape)
    sample = (f"{layers} of {shape.n_layers} layers + lm_head per step, scaled to a full token by "
              f"weight bytes; {probe.kind} CPU code, every GEMV split by rows over {cores} threads")
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": spt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_text(shape),
                   "gemvs_per_token": shape.gemvs_per_token(), "weight_bytes_per_token": weight_b,
                   "api": "the reference's CPU kernels called through the reference library's tc_* ABI"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": probe.kind,
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "weight_gbs": weight_b / spt / 1e9,
    }


def cpu_baseline_leg(shape) -> dict:
    """The reference CPU code as shipped (one thread) on one whole token (about 10 s of host
    work for the 7B shape)."""
    cpu = CpuDecode(shape, layers=shape.n_layers, threads=1)
    spt, per_sample = cpu.seconds_per_token(steps=1, warmup=0)
    return {"value": 1.0 / spt, "unit": UNIT, "cores": 1, "kind": cpu.kind,
            "sample": f"one token: {shape.n_layers} of {shape.n_layers} layers + lm_head on one thread "
                      f"({per_sample:.1f} s)"}


# ---------------------------------------------------------------------------------------
# Single operations (BASELINE configs 1, 2 and 4, and the dense fused operations)
# ---------------------------------------------------------------------------------------
def gemv_cases(ctx, quick: bool = False) -> list[dict]:
    """Per case: microseconds per GEMV with the weights streamed from HBM (the calls rotate over
    enough distinct copies of the matrix to exceed twice the L2), algorithmic GB/s and its
    fraction of the measured HBM peak.  Two ways of issuing the same calls:
      stream  - recorded on a tc_stream, one tc_stream_sync (Q4_0, M = 1 lists run as one
                persistent kernel; everything else replays a CUDA graph of per-operation kernels);
      per_op  - the same with the persistent kernel switched off: one kernel per GEMV.
    Algorithmic bytes per call: N*(K/32)*B + M*K*sx + M*N*sy (+ K*sx of gamma when fused)."""
    import tensorcore_b200 as tc
    from tensorcore_b200 import decode as D
    peak, _ = measured_peaks()
    out = []

    def weights_copies(fmt, N, K):
        nbytes = tc.quantized_size(fmt, N, K)
        copies = max(2, min(64, int(2 * 126e6 // nbytes) + 1))
        w16 = D.device_weights_fp16(N, K, 0xC0FFEE + N + K)
        return [D.quantize_into(ctx, w16, fmt) for _ in range(copies)], nbytes

    def quant_case(config, fmt, M, N, K, xd, yd, fused, iters):
        ws, nbytes = weights_copies(fmt, N, K)
        xs, ys = (4 if xd == "f32" else 2), (4 if yd == "f32" else 2)
        rng = np.random.default_rng(M + N + K)
        xdt = np.float32 if xd == "f32" else np.float16
        x = ctx.buffer_from_array(rng.standard_normal((M, K)).astype(np.float32).astype(xdt))
        g = ctx.buffer_from_array((1 + 0.1 * rng.standard_normal(K)).astype(np.float32).astype(xdt)) if fused else None
        y = ctx.buffer(M * N * ys)
        alg = nbytes + M * K * xs + M * N * ys + (K * xs if fused else 0)
        rec = {"config": config, "fmt": "q4_0" if fmt == 0 else "q8_0", "M": M, "N": N, "K": K, "x": xd, "y": yd,
               "fused_rmsnorm": bool(fused), "weight_copies": len(ws), "bytes": alg}
        for mode in ("stream", "per_op"):
            ms = D.gemv_bench(ctx, ws, x, y, fmt, M, N, K, iters, xd, yd, g, persistent=(mode == "stream"))
            us = ms / iters * 1e3
            rec[mode] = {"us": round(us, 3), "GBs": round(alg / us / 1e3, 1), "frac": round(alg / us / 1e3 / peak, 4),
                         "kernel": tc.cuda_last_kernel_name()}
            if mode == "stream" and "persistent" not in rec[mode]["kernel"]:
                rec["per_op"] = rec["stream"]          # nothing to switch off: same launches
                break
        best = min(rec["stream"]["us"], rec["per_op"]["us"])
        rec["tflops"] = round(2.0 * M * N * K / best / 1e6, 2)
        for b in ws + [x, y] + ([g] if g else []):
            b.close()
        out.append(rec)

    def dense_case(name, layernorm, M, N, K, iters):
        import torch
        nbytes = K * N * 2
        copies = max(2, int(2 * 126e6 // nbytes) + 1)
        gen = torch.Generator(device="cuda"); gen.manual_seed(0xD0 + N)
        rng = np.random.default_rng(N + K)
        ws = []
        for _ in range(copies):
            w = (torch.randn((K, N), generator=gen, device="cuda") * 0.02).to(torch.float16)
            b = ctx.buffer(nbytes)
            b.upload(w.cpu().numpy())
            ws.append(b)
        x = ctx.buffer_from_array(rng.standard_normal((M, K)).astype(np.float16))
        g = ctx.buffer_from_array((1 + 0.1 * rng.standard_normal(K)).astype(np.float16))
        bt = ctx.buffer_from_array((0.1 * rng.standard_normal(K)).astype(np.float16)) if layernorm else None
        y = ctx.buffer(M * N * 2)
        alg = nbytes + M * K * 2 + M * N * 2 + K * 2 * (2 if layernorm else 1)
        ms = D.dense_bench(ctx, ws, x, g, bt, y, M, N, K, iters)
        us = ms / iters * 1e3
        out.append({"config": name, "fmt": "f16 W[K,N]", "M": M, "N": N, "K": K, "x": "f16", "y": "f16",
                    "weight_copies": copies, "bytes": alg,
                    "per_op": {"us": round(us, 3), "GBs": round(alg / us / 1e3, 1), "frac": round(alg / us / 1e3 / peak, 4),
                               "kernel": tc.cuda_last_kernel_name()}})
        for b in ws + [x, g, y] + ([bt] if bt else []):
            b.close()

    def attention_case(name, B, H, Hkv, Sk, Dh, iters):
        """Decode attention: one query row per head over a K/V cache of Sk positions.  Algorithmic
        bytes: K and V of every kv head once (2 * B * Hkv * Sk * Dh * 2) + Q and O."""
        kv_bytes = B * Hkv * Sk * Dh * 2
        copies = max(2, int(2 * 126e6 // (2 * kv_bytes)) + 1)
        rng = np.random.default_rng(Sk + Dh)
        ks = [ctx.buffer_from_array(rng.standard_normal((B, Hkv, Sk, Dh)).astype(np.float16)) for _ in range(copies)]
        vs = [ctx.buffer_from_array(rng.standard_normal((B, Hkv, Sk, Dh)).astype(np.float16)) for _ in range(copies)]
        q = ctx.buffer_from_array(rng.standard_normal((B, H, 1, Dh)).astype(np.float16))
        o = ctx.buffer(B * H * Dh * 2)
        alg = 2 * kv_bytes + 2 * B * H * Dh * 2
        ms = D.attention_bench(ctx, q, ks, vs, o, B, H, Hkv, Sk, Dh, iters)
        us = ms / iters * 1e3
        out.append({"config": name, "fmt": "f16 K/V", "batch": B, "heads": H, "kv_heads": Hkv, "seq_kv": Sk, "head_dim": Dh,
                    "kv_copies": copies, "bytes": alg,
                    "per_op": {"us": round(us, 3), "GBs": round(alg / us / 1e3, 1), "frac": round(alg / us / 1e3 / peak, 4),
                               "kernel": tc.cuda_last_kernel_name()}})
        for b in ks + vs + [q, o]:
            b.close()

    def gemm_case(name, M, N, K, iters):
        """tc_gemm, fp16 in and out, fp32 accumulation, through the buffer API (each call returns
        after the device is done, as the reference's does): host clock around the calls, against the
        measured dense bf16 peak."""
        rng = np.random.default_rng(M + N + K)
        a = ctx.buffer_from_array(rng.standard_normal((M, K)).astype(np.float16))
        b = ctx.buffer_from_array((rng.standard_normal((K, N)) * 0.05).astype(np.float16))
        c = ctx.buffer(M * N * 2)
        for _ in range(3):
            tc.gemm(ctx, a, b, c, M, N, K)
        t0 = time.perf_counter()
        for _ in range(iters):
            tc.gemm(ctx, a, b, c, M, N, K)
        us = (time.perf_counter() - t0) / iters * 1e6
        tflops = 2.0 * M * N * K / us / 1e6
        tpeak = None
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                tpeak = float(json.load(f)["bf16_tflops"])
        except Exception:
            tpeak = 1590.0
        out.append({"config": name, "fmt": "f16", "M": M, "N": N, "K": K,
                    "per_op": {"us": round(us, 2), "tflops": round(tflops, 1), "frac_tensor": round(tflops / tpeak, 4),
                               "kernel": tc.cuda_last_kernel_name()}})
        for x in (a, b, c):
            x.close()

    it = 100 if quick else 200
    quant_case("config 1: Q4_0 4096x4096, fp32 x -> fp32 y", 0, 1, 4096, 4096, "f32", "f32", False, it)
    quant_case("config 1 through the fp16 ABI", 0, 1, 4096, 4096, "f16", "f16", False, it)
    for xd in ("f32", "f16"):
        quant_case(f"config 2: Q8_0 11008x4096, {xd} x", 1, 1, 11008, 4096, xd, xd, False, it)
        quant_case(f"config 2: fused RMSNorm + Q8_0 11008x4096, {xd} x", 1, 1, 11008, 4096, xd, xd, True, it)
    for M in (1, 4, 8, 16, 32):
        quant_case(f"config 4: Q4_0 14336x4096, M={M}, fp16 x -> fp32 y", 0, M, 14336, 4096, "f16", "f32", False, it // 2)
    quant_case("config 2 batched: Q8_0 11008x4096, M=16, fp16 x -> fp16 y (weights dequantised once, then the tcgen05 "
               "GEMM)", 1, 16, 11008, 4096, "f16", "f16", False, 20)
    for fmt, tag in ((0, "Q4_0"), (1, "Q8_0")):
        quant_case(f"prefill block: {tag} 14336x4096, M=512, fp16 x -> fp16 y (weights dequantised once, then the "
                   "tcgen05 GEMM)", fmt, 512, 14336, 4096, "f16", "f16", False, 20)
    dense_case("tc_fused_rmsnorm_gemv, fp16 W 4096x11008", False, 1, 11008, 4096, it // 2)
    dense_case("tc_fused_layernorm_gemv, fp16 W 4096x11008", True, 1, 11008, 4096, it // 2)
    attention_case("tc_attention_forward, decode row: 32 heads x 128, 4096 keys (7B shape)", 1, 32, 32, 4096, 128, it // 2)
    attention_case("tc_attention_forward, decode row: 64 heads / 8 kv heads x 128, 8192 keys (70B shape)", 1, 64, 8, 8192, 128, it // 2)
    gemm_case("tc_gemm fp16 4096 x 4096 x 4096", 4096, 4096, 4096, 20)
    gemm_case("tc_gemm fp16 512 x 11008 x 4096 (a prefill block against a 7B projection)", 512, 11008, 4096, 20)
    return out


def cpu_single_gemv_baselines() -> list[dict]:
    """The reference's CPU code as shipped (one thread) on configs 1 and 2: median of 3 calls."""
    import oracle as O
    if not O.ref_available():
        return []
    R = O.RefLib()
    rng = np.random.default_rng(12)
    res = []
    for config, fmt, N, K in (("config 1: Q4_0 4096x4096", 0, 4096, 4096), ("config 2: Q8_0 11008x4096", 1, 11008, 4096)):
        bb = 18 if fmt == 0 else 34
        Wq = rng.integers(0, 256, N * (K // 32) * bb, dtype=np.uint8)
        Wq.reshape(-1, bb)[:, 0:2] = np.frombuffer(np.float16(0.005).tobytes(), dtype=np.uint8)
        X = rng.standard_normal((1, K)).astype(np.float16)
        ts = []
        for _ in range(3):
            t0 = time.perf_counter()
            R.gemv_quantized(X, Wq, fmt, N)
            ts.append(time.perf_counter() - t0)
        t = float(np.median(ts))
        res.append({"config": config, "ms": round(t * 1e3, 2), "GBs": round(Wq.nbytes / t / 1e9, 3), "cores": 1,
                    "kind": "reference", "sample": "whole call through the reference library's tc_gemv_quantized "
                                                   "(includes its buffer set-up), median of 3"})
    return res


def llama70b_record(ctx, steps: int) -> dict:
    """BASELINE config 5 on one GPU: the 70B-shape model (39.1 GB of Q4_0) quantised on the device,
    decoded at batch 1 (one persistent launch per token) and batch 8 (tcgen05 kernels, CUDA graph)."""
    import tensorcore_b200 as tc
    from tensorcore_b200 import decode as D
    shape = D.LLAMA_70B
    peak, _ = measured_peaks()
    t0 = time.perf_counter()
    model = D.synthetic_model_on_device(ctx, shape, 0)
    build_s = time.perf_counter() - t0
    rec = {"workload": "llama-70b-shape Q4_0 decode weight stream: 80 layers x (q,o 8192x8192; k,v 1024x8192; "
                       "gate,up 28672x8192; down 8192x28672) + lm_head 128256x8192, RMSNorm fused",
           "weight_bytes_per_token": shape.weight_bytes(0), "build_s": round(build_s, 1)}
    for M in (1, 8):
        sess = D.DecodeSession(ctx, model, M=M)
        rng = np.random.default_rng(D.X_SEED + M)
        sess.x.upload(rng.standard_normal((M, shape.d_model)).astype(np.float16))
        sess.run(3, fused_norms=True)
        gpu_ms, _ = sess.run(steps, fused_norms=True)
        logits = sess.logits.to_numpy((M, shape.vocab), np.float16)
        if not np.all(np.isfinite(logits)) or tc.take_device_error(ctx) != 0:
            raise SystemExit("70B run: non-finite logits or device error")
        ms = gpu_ms / steps
        wb = shape.weight_bytes(0)
        rec[f"batch{M}"] = {"ms_per_step": round(ms, 4), "tok_s": round(M * 1e3 / ms, 2),
                            "weight_GBs": round(wb / ms / 1e6, 1), "frac": round(wb / ms / 1e6 / peak, 4),
                            "kernel": tc.cuda_last_kernel_name()}
        sess.close()
    for b in model.owner.values():
        b.close()
    return rec


def run_single_gpu(args) -> dict:
    import torch

    import tensorcore_b200 as tc
    from tensorcore_b200 import decode as D

    shape = D.LLAMA_7B
    if getattr(args, "layers", 0):
        import dataclasses
        shape = dataclasses.replace(shape, name=f"{shape.name}-first{args.layers}layers", n_layers=args.layers)
    if not os.path.exists(tc.LIB_PATH):
        raise SystemExit("libtensorcore.so is not built: run `python -m tensorcore_b200.build`")
    torch.cuda.set_device(0)
    ctx = tc.Context()
    tmpdir = tempfile.mkdtemp(prefix="tcb_bench_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
    path = os.path.join(tmpdir, "synthetic-llama-7b-q4_0.gguf")
    t0 = time.perf_counter()
    D.build_synthetic_gguf(path, shape, ctx, fmt=0)
    t_build = time.perf_counter() - t0
    t0 = time.perf_counter()
    model = D.model_from_gguf(ctx, path, shape, fmt=0)
    t_load = time.perf_counter() - t0
    os.remove(path)
    os.rmdir(tmpdir)

    sess = D.DecodeSession(ctx, model, M=1)
    rng = np.random.default_rng(D.X_SEED)
    x = rng.standard_normal((1, shape.d_model)).astype(np.float32).astype(np.float16)
    sess.x.upload(x)

    # resident-in-HBM measurement
    sess.run(max(3, args.warmup), fused_norms=True)
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = tc.launch_count()
    gpu_ms, wall_ms = sess.run(args.steps, fused_norms=True)
    launches = tc.launch_count() - launches0
    clocks = sampler.stop()
    logits = sess.logits.to_numpy((1, shape.vocab), np.float16)
    if not np.all(np.isfinite(logits)):
        raise SystemExit("non-finite logits")
    if tc.take_device_error(ctx) != 0:
        raise SystemExit("device-side error word set")

    # end-to-end: step input from pinned host memory in, logits out, every step
    hx = torch.from_numpy(x.copy()).pin_memory()
    hl = torch.empty((1, shape.vocab), dtype=torch.float16).pin_memory()
    sess.run(3, fused_norms=True, host_x=hx.data_ptr(), host_logits=hl.data_ptr())
    _, e2e_wall_ms = sess.run(args.steps, fused_norms=True, host_x=hx.data_ptr(),
                              host_logits=hl.data_ptr())
    # same input, same kernels: the e2e path must reproduce the resident path's logits, up to
    # the summation order of the shared-memory accumulators (fp16 rounding flips)
    a, b = hl.numpy().astype(np.float64), logits.astype(np.float64)
    drift = float(np.sqrt(np.mean((a - b) ** 2)) / max(np.sqrt(np.mean(b ** 2)), 1e-30))
    if not drift <= 2e-2:   # 225 chained fp16 GEMVs: the accumulation order differs run to run and rounding flips compound
        raise SystemExit(f"e2e logits differ from resident-run logits (scaled rms {drift})")

    total_b, weight_b = algorithmic_bytes_per_token(shape)
    ms_per_step = gpu_ms / args.steps
    value = 1e3 / ms_per_step
    peak, peak_kind = measured_peaks()
    n_gemv = shape.gemvs_per_token()
    achieved = total_b / (ms_per_step * 1e-3) / 1e9
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "s16 x u4 -> s32 (dp2a), f32 scales", "data": "synthetic",
        "config": {
            "workload": workload_text(shape),
            "gemvs_per_token": n_gemv, "weight_bytes_per_token": weight_b,
            "model": "GGUF v3 file loaded with tc_gguf_load_supported_tensors",
            "l2": "3.7 GB of weights are streamed per step (126 MB L2): no flush needed",
            "api": "tc_gemv_quantized_async / tcx_fused_rmsnorm_gemv_quantized_ex on a tc_stream, "
                   "one tc_stream_sync per token",
            "gguf_build_s": round(t_build, 2), "gguf_load_s": round(t_load, 2),
        },
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak,
                     # DRAM bytes per launch, modelled: ncu (dram__bytes_read + write) on an 8-layer
                     # launch of this kernel, as a ratio to its algorithmic bytes, scaled by bytes
                     "traffic": TRAFFIC_RATIO * total_b / (launches / args.steps),
                     "traffic_kind": f"modelled: algorithmic bytes x {TRAFFIC_RATIO} (ncu capture of an 8-layer launch)",
                     "traffic_source": "profiles/bench_decode_7b_q4_0_persistent_launch.md",
                     "peak_kind": peak_kind,
                     # one persistent launch per token when the stream takes that path, else
                     # one launch per GEMV
                     "launches_per_step": launches / args.steps,
                     "bytes_per_launch": total_b / (launches / args.steps),
                     "us_per_launch": ms_per_step * 1e3 / (launches / args.steps),
                     "weight_gbs": weight_b / (ms_per_step * 1e-3) / 1e9},
        "e2e": {"value": 1e3 / (e2e_wall_ms / args.steps), "unit": UNIT,
                "h2d_bytes_per_step": shape.d_model * 2, "d2h_bytes_per_step": shape.vocab * 2,
                "timing": "host clock around the loop (copies are synchronous calls)"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "wall_ms_per_step": wall_ms / args.steps,
        "kernel": tc.cuda_last_kernel_name(),
    }
    sess.close()
    model.owner.close()
    if not args.no_gemv:
        out["gemv"] = gemv_cases(ctx, quick=args.steps < 50)
    if not args.no_70b and not getattr(args, "layers", 0):
        out["llama70b"] = llama70b_record(ctx, steps=max(5, min(30, args.steps // 5)))
    if not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline_leg(shape)
        out["cpu_baseline"]["single_gemv"] = cpu_single_gemv_baselines()
    ctx.close()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gemv", action="store_true", help="skip the single-operation cases (configs 1, 2, 4)")
    ap.add_argument("--no-70b", action="store_true", help="skip the 70B-shape record (config 5)")
    ap.add_argument("--layers", type=int, default=0,
                    help="profiling aid: run the same step on the first LAYERS layers + lm_head (a smaller "
                         "device footprint for ncu captures); the JSON line then names the reduced workload")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference_arm(args)), flush=True)
        return
    if args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # stdout carries the one JSON line and nothing else: libraries that print to it while the ranks
        # set up (NCCL's version banner) are pointed at stderr until the line is ready.
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            from tensorcore_b200 import tp
            out = tp.run_bench(args)
        finally:
            sys.stdout.flush()
            try:
                import ctypes
                ctypes.CDLL(None).fflush(None)       # whatever C code left in stdio's buffer goes to stderr too
            except Exception:
                pass
            os.dup2(saved, 1)
            os.close(saved)
        if rank == 0 and out is not None:
            print(json.dumps(out), flush=True)
        sys.stdout.flush()
        tp.shutdown()
        return
    print(json.dumps(run_single_gpu(args)), flush=True)


if __name__ == "__main__":
    main()
