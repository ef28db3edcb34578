"""Synthetic Llama-shaped decode workloads on top of the C ABI.

* `LlamaShape` - the projection shapes of the 7B and 70B configurations;
* `build_synthetic_gguf` - seeded N(0, 0.02^2) weights, quantised on the device by the library's
  own quantiser and written to a GGUF v3 file (the file is then loaded with
  tc_gguf_load_supported_tensors like any other model);
* `synthetic_model_on_device` - the same weights quantised straight into device buffers, for
  models too large to round-trip through a file;
* `DecodeSession` - the GEMV sequence of one decode step, recorded on a tc_stream and
  synchronised once per token by the compiled harness (csrc/harness/decode_harness.cpp).

torch is used here for seeded random numbers on the device and pinned host memory only.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_double, c_float, c_int, c_void_p
from dataclasses import dataclass

import numpy as np

import tensorcore_b200 as tc
from tensorcore_b200 import gguf_writer as gw

HARNESS_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libtc_harness.so")
BLOCK_BYTES = {0: 18, 1: 34}
PROJ = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")


@dataclass(frozen=True)
class LlamaShape:
    name: str
    n_layers: int
    d_model: int
    d_ff: int
    n_heads: int
    n_kv_heads: int
    vocab: int

    @property
    def d_kv(self) -> int:
        return self.d_model // self.n_heads * self.n_kv_heads

    def proj_shape(self, which: str) -> tuple[int, int]:
        """(N, K) of a projection: N output rows, K input columns."""
        d, f, kv = self.d_model, self.d_ff, self.d_kv
        return {"attn_q": (d, d), "attn_k": (kv, d), "attn_v": (kv, d), "attn_output": (d, d),
                "ffn_gate": (f, d), "ffn_up": (f, d), "ffn_down": (d, f),
                "output": (self.vocab, d)}[which]

    def weight_bytes(self, fmt: int = 0, lm_head: bool = True) -> int:
        bb = BLOCK_BYTES[fmt]
        per_layer = sum(n * (k // 32) * bb for n, k in (self.proj_shape(p) for p in PROJ))
        total = self.n_layers * per_layer
        if lm_head:
            n, k = self.proj_shape("output")
            total += n * (k // 32) * bb
        return total

    def gemvs_per_token(self, lm_head: bool = True) -> int:
        return 7 * self.n_layers + (1 if lm_head else 0)


LLAMA_7B = LlamaShape("llama-7b", 32, 4096, 11008, 32, 32, 32000)
LLAMA_70B = LlamaShape("llama-70b", 80, 8192, 28672, 64, 8, 128256)


def tiny_shape(n_layers=2, d_model=1024, d_ff=2048, n_heads=8, n_kv_heads=4, vocab=1000):
    return LlamaShape("tiny", n_layers, d_model, d_ff, n_heads, n_kv_heads, vocab)


def tensor_seed(layer: int, t: int) -> int:
    return 0x7C0000 + 16 * layer + t


LM_HEAD_SEED = 0x7CFFFF
X_SEED = 0x7CA000


def _torch():
    import torch
    return torch


def device_weights_fp16(N: int, K: int, seed: int, device="cuda"):
    """fp32 N(0, 0.02^2) from a seeded device generator, rounded to fp16."""
    torch = _torch()
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.empty((N, K), dtype=torch.float32, device=device)
    w.normal_(0.0, 0.02, generator=g)
    return w.to(torch.float16)


def quantize_into(ctx: tc.Context, w16, fmt: int) -> tc.Buffer:
    """Quantises a device fp16 [N,K] torch tensor into a new device buffer with the library's
    quantiser (raw launch on torch's current stream)."""
    torch = _torch()
    N, K = w16.shape
    buf = ctx.buffer(tc.quantized_size(fmt, N, K))
    tc.raw_quantize_weights(ctx, w16.data_ptr(), buf.device_ptr(), fmt, N, K,
                            torch.cuda.current_stream().cuda_stream)
    torch.cuda.current_stream().synchronize()
    return buf


def gamma_fp16(K: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32).astype(np.float16)


def build_synthetic_gguf(path: str, shape: LlamaShape, ctx: tc.Context, fmt: int = 0) -> int:
    """Writes the synthetic model to `path`; returns the number of weight bytes written."""
    ggml = gw.GGML_Q4_0 if fmt == 0 else gw.GGML_Q8_0
    specs, total = [], 0

    def qspec(name, which, seed):
        nonlocal total
        N, K = shape.proj_shape(which)
        nbytes = tc.quantized_size(fmt, N, K)
        total += nbytes

        def write(f, N=N, K=K, seed=seed, nbytes=nbytes):
            buf = quantize_into(ctx, device_weights_fp16(N, K, seed), fmt)
            f.write(buf.to_numpy((nbytes,), np.uint8).tobytes())
            buf.close()
        return gw.TensorSpec(name, [K, N], ggml, nbytes, writer=write)

    def nspec(name, seed):
        g = gamma_fp16(shape.d_model, seed)
        return gw.TensorSpec(name, [shape.d_model], gw.GGML_F16, g.nbytes, data=g)

    for l in range(shape.n_layers):
        for t, p in enumerate(PROJ):
            specs.append(qspec(f"blk.{l}.{p}.weight", p, tensor_seed(l, t)))
        specs.append(nspec(f"blk.{l}.attn_norm.weight", 0x7CB000 + l))
        specs.append(nspec(f"blk.{l}.ffn_norm.weight", 0x7CC000 + l))
    specs.append(nspec("output_norm.weight", 0x7CD000))
    specs.append(qspec("output.weight", "output", LM_HEAD_SEED))
    meta = gw.llama_metadata(shape.d_model, shape.d_ff, shape.n_layers, shape.n_heads,
                             shape.n_kv_heads, shape.vocab)
    gw.write_gguf(path, meta, specs)
    return total


class _ModelDesc(Structure):
    _fields_ = [("n_layers", c_int), ("d_model", c_int), ("d_ff", c_int), ("d_kv", c_int),
                ("vocab", c_int), ("M", c_int), ("fmt", c_int)] + \
               [(n, POINTER(c_void_p)) for n in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown",
                                                 "attn_norm", "ffn_norm")] + \
               [("out_norm", c_void_p), ("lm_head", c_void_p)]


_harness = None


def harness() -> ctypes.CDLL:
    global _harness
    if _harness is None:
        tc.lib()
        if not os.path.exists(HARNESS_PATH):
            raise RuntimeError(f"{HARNESS_PATH} not found: run `python -m tensorcore_b200.build`")
        H = ctypes.CDLL(HARNESS_PATH)
        H.tch_session_create.argtypes = [c_void_p, POINTER(_ModelDesc), POINTER(c_void_p)]
        H.tch_session_create.restype = c_int
        H.tch_session_destroy.argtypes = [c_void_p]
        H.tch_session_destroy.restype = None
        for n in ("tch_session_x", "tch_session_logits"):
            getattr(H, n).argtypes = [c_void_p]
            getattr(H, n).restype = c_void_p
        H.tch_session_hidden.argtypes = [c_void_p, c_int]
        H.tch_session_hidden.restype = c_void_p
        H.tch_session_run.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                      POINTER(c_float), POINTER(c_double)]
        H.tch_session_run.restype = c_int
        H.tch_gemv_bench.argtypes = [c_void_p, POINTER(c_void_p), c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_int, POINTER(c_float)]
        H.tch_gemv_bench.restype = c_int
        H.tch_dense_bench.argtypes = [c_void_p, POINTER(c_void_p), c_int, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int, c_int, c_int, c_int, POINTER(c_float)]
        H.tch_dense_bench.restype = c_int
        H.tch_attention_bench.argtypes = [c_void_p, c_void_p, POINTER(c_void_p), POINTER(c_void_p), c_int, c_void_p,
                                          c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_float)]
        H.tch_attention_bench.restype = c_int
        _harness = H
    return _harness


class Model:
    """Handles of a Llama-shaped model's projection and norm buffers (one device)."""

    def __init__(self, shape: LlamaShape, fmt: int, get, owner=None):
        """`get(name)` returns the tc_buffer handle (int / c_void_p) of a tensor name."""
        self.shape, self.fmt, self.owner = shape, fmt, owner
        L = shape.n_layers
        self.lists = {}
        for field, p in zip(("wq", "wk", "wv", "wo", "wgate", "wup", "wdown"), PROJ):
            self.lists[field] = [get(f"blk.{l}.{p}.weight") for l in range(L)]
        self.lists["attn_norm"] = [get(f"blk.{l}.attn_norm.weight") for l in range(L)]
        self.lists["ffn_norm"] = [get(f"blk.{l}.ffn_norm.weight") for l in range(L)]
        self.out_norm = get("output_norm.weight")
        self.lm_head = get("output.weight")


def model_from_gguf(ctx: tc.Context, path: str, shape: LlamaShape, fmt: int = 0) -> Model:
    g = tc.GgufFile(path)
    loaded = g.load_supported_tensors(ctx)
    g.close()
    return Model(shape, fmt, lambda n: loaded.get_tensor(n)["buffer"], owner=loaded)


def synthetic_model_on_device(ctx: tc.Context, shape: LlamaShape, fmt: int = 0) -> Model:
    """Quantises every projection straight into device buffers (no file)."""
    bufs: dict[str, tc.Buffer] = {}
    for l in range(shape.n_layers):
        for t, p in enumerate(PROJ):
            N, K = shape.proj_shape(p)
            bufs[f"blk.{l}.{p}.weight"] = quantize_into(
                ctx, device_weights_fp16(N, K, tensor_seed(l, t)), fmt)
        bufs[f"blk.{l}.attn_norm.weight"] = ctx.buffer_from_array(gamma_fp16(shape.d_model, 0x7CB000 + l))
        bufs[f"blk.{l}.ffn_norm.weight"] = ctx.buffer_from_array(gamma_fp16(shape.d_model, 0x7CC000 + l))
    bufs["output_norm.weight"] = ctx.buffer_from_array(gamma_fp16(shape.d_model, 0x7CD000))
    N, K = shape.proj_shape("output")
    bufs["output.weight"] = quantize_into(ctx, device_weights_fp16(N, K, LM_HEAD_SEED), fmt)
    return Model(shape, fmt, lambda n: bufs[n].handle.value, owner=bufs)


class DecodeSession:
    """One stream, one set of activation buffers, M sequences decoded together."""

    def __init__(self, ctx: tc.Context, model: Model, M: int = 1):
        self.ctx, self.model, self.M = ctx, model, M
        s = model.shape
        d = _ModelDesc()
        d.n_layers, d.d_model, d.d_ff, d.d_kv, d.vocab = s.n_layers, s.d_model, s.d_ff, s.d_kv, s.vocab
        d.M, d.fmt = M, model.fmt
        self._keep = []
        for field, handles in model.lists.items():
            arr = (c_void_p * len(handles))(*[c_void_p(int(getattr(h, "value", h))) for h in handles])
            self._keep.append(arr)
            setattr(d, field, ctypes.cast(arr, POINTER(c_void_p)))
        d.out_norm = c_void_p(int(getattr(model.out_norm, "value", model.out_norm)))
        d.lm_head = c_void_p(int(getattr(model.lm_head, "value", model.lm_head)))
        self.handle = c_void_p()
        st = harness().tch_session_create(ctx.handle, byref(d), byref(self.handle))
        if st != tc.TC_OK:
            raise tc.TensorcoreError(st)
        self.x = tc.Buffer(ctx, handle=c_void_p(harness().tch_session_x(self.handle)), owned=False)
        self.logits = tc.Buffer(ctx, handle=c_void_p(harness().tch_session_logits(self.handle)),
                                owned=False)

    def hidden(self, which: int) -> tc.Buffer:
        return tc.Buffer(self.ctx, handle=c_void_p(harness().tch_session_hidden(self.handle, which)),
                         owned=False)

    def run(self, tokens: int, fused_norms: bool = True, host_x: int = 0, host_logits: int = 0):
        """Returns (gpu_ms, wall_ms) over `tokens` decode steps.  With host_x / host_logits
        (addresses of pinned host arrays) every step copies its input in and its logits out."""
        gpu, wall = c_float(), c_double()
        e2e = 1 if host_x and host_logits else 0
        st = harness().tch_session_run(self.handle, tokens, 1 if fused_norms else 0, e2e,
                                       c_void_p(host_x), c_void_p(host_logits), byref(gpu),
                                       byref(wall))
        if st != tc.TC_OK:
            raise tc.TensorcoreError(st)
        return gpu.value, wall.value

    def close(self):
        if self.handle:
            harness().tch_session_destroy(self.handle)
            self.handle = None


def gemv_bench(ctx: tc.Context, weights: list[tc.Buffer], x: tc.Buffer, y: tc.Buffer, fmt: int,
               M: int, N: int, K: int, iters: int, x_dtype="f16", y_dtype="f16",
               gamma: tc.Buffer | None = None, persistent: bool = True) -> float:
    """Milliseconds (CUDA events) for `iters` back-to-back GEMVs rotating over `weights`,
    recorded on one tc_stream.  persistent=False keeps one kernel per operation."""
    arr = (c_void_p * len(weights))(*[w.handle for w in weights])
    ms = c_float()
    st = harness().tch_gemv_bench(ctx.handle, ctypes.cast(arr, POINTER(c_void_p)), len(weights),
                                  x.handle, gamma.handle if gamma else None, y.handle, fmt, M, N,
                                  K, tc._dtype(x_dtype), tc._dtype(y_dtype), 1 if gamma else 0,
                                  iters, 1 if persistent else 0, byref(ms))
    if st != tc.TC_OK:
        raise tc.TensorcoreError(st)
    return ms.value


def dense_bench(ctx: tc.Context, weights: list[tc.Buffer], x: tc.Buffer, gamma: tc.Buffer,
                beta: tc.Buffer | None, y: tc.Buffer, M: int, N: int, K: int, iters: int) -> float:
    """Milliseconds for `iters` back-to-back fused norm + dense fp16 GEMV launches."""
    arr = (c_void_p * len(weights))(*[w.handle for w in weights])
    ms = c_float()
    st = harness().tch_dense_bench(ctx.handle, ctypes.cast(arr, POINTER(c_void_p)), len(weights), x.handle,
                                   gamma.handle, beta.handle if beta else None, y.handle, M, N, K, iters,
                                   byref(ms))
    if st != tc.TC_OK:
        raise tc.TensorcoreError(st)
    return ms.value


def attention_bench(ctx: tc.Context, q: tc.Buffer, ks: list[tc.Buffer], vs: list[tc.Buffer], o: tc.Buffer, batch: int,
                    heads: int, kv_heads: int, seq_kv: int, head_dim: int, iters: int) -> float:
    """Milliseconds for `iters` back-to-back decode-attention launches (one query row per head)."""
    ka = (c_void_p * len(ks))(*[b.handle for b in ks])
    va = (c_void_p * len(vs))(*[b.handle for b in vs])
    ms = c_float()
    st = harness().tch_attention_bench(ctx.handle, q.handle, ctypes.cast(ka, POINTER(c_void_p)),
                                       ctypes.cast(va, POINTER(c_void_p)), len(ks), o.handle, batch, heads, kv_heads,
                                       seq_kv, head_dim, iters, byref(ms))
    if st != tc.TC_OK:
        raise tc.TensorcoreError(st)
    return ms.value
