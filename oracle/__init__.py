"""TEST INFRASTRUCTURE - not part of the product.

ctypes access to the two CPU checkers:

* ``liboracle.so``  - the plain-C restatement in ``tc_oracle.c`` (always available after
  ``make -C oracle``);
* ``_ref/libtensorcore_ref.so`` - the reference's own portable-CPU backend compiled from its
  sources (available when it was built where a reference checkout exists; the built file
  travels with the repository tree, the sources do not).

Only the test suite, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this module.  The product package never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_float, c_int, c_size_t, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libtensorcore_ref.so")

Q4_0, Q8_0 = 0, 1
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34}


def build(ref_root: str | None = None) -> None:
    """Compile liboracle.so and, when a reference checkout is present, _ref/."""
    args = ["make", "-C", _HERE, "all"]
    if ref_root:
        args.append(f"REF={ref_root}")
    subprocess.run(args, check=True, stdout=subprocess.DEVNULL)


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build()
        L = ctypes.CDLL(ORACLE_SO)
        L.orc_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.orc_f16_to_f32.restype = c_float
        L.orc_f32_to_f16.argtypes = [c_float]
        L.orc_f32_to_f16.restype = ctypes.c_uint16
        L.orc_quantized_size.argtypes = [c_int, c_int, c_int]
        L.orc_quantized_size.restype = c_size_t
        for name in ("orc_f32_to_f16_array", "orc_f16_to_f32_array"):
            getattr(L, name).argtypes = [c_void_p, c_void_p, c_size_t]
            getattr(L, name).restype = None
        _lib = L
    return _lib


def _p(a: np.ndarray) -> c_void_p:
    assert a.flags["C_CONTIGUOUS"]
    return c_void_p(a.ctypes.data)


def _call(fn, *args):
    fn.restype = c_int
    rc = fn(*args)
    if rc != 0:
        raise ValueError(f"oracle rejected the arguments (rc={rc})")


def f32_to_f16_bits(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_f32_to_f16_array(_p(a), _p(out), a.size)
    return out


def f16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().orc_f16_to_f32_array(_p(a), _p(out), a.size)
    return out


def quantized_size(fmt: int, N: int, K: int) -> int:
    return int(lib().orc_quantized_size(fmt, N, K))


def quantize_weights(W_f16: np.ndarray, fmt: int) -> np.ndarray:
    """W_f16: [N,K] float16 (or uint16 bit patterns) -> packed blocks as uint8."""
    W = np.ascontiguousarray(W_f16).view(np.uint16)
    N, K = W.shape
    out = np.empty(quantized_size(fmt, N, K), dtype=np.uint8)
    _call(lib().orc_quantize_weights, _p(W), _p(out), c_int(fmt), c_int(N), c_int(K))
    return out


def gemv_quantized(X_f16: np.ndarray, Wq: np.ndarray, fmt: int, N: int) -> np.ndarray:
    X = np.ascontiguousarray(X_f16).view(np.uint16)
    M, K = X.shape
    Y = np.empty((M, N), dtype=np.uint16)
    _call(lib().orc_gemv_quantized, _p(X), _p(Wq), _p(Y), c_int(fmt), c_int(M), c_int(N), c_int(K))
    return Y.view(np.float16)


def gemv_quantized_rows(X_f16, Wq, Y_bits, fmt, N, n_begin, n_end) -> None:
    """Rows [n_begin, n_end) of gemv_quantized, written into Y_bits ([M,N] uint16)."""
    X = np.ascontiguousarray(X_f16).view(np.uint16)
    M, K = X.shape
    _call(lib().orc_gemv_quantized_rows, _p(X), _p(Wq), _p(Y_bits), c_int(fmt), c_int(M),
          c_int(N), c_int(K), c_int(n_begin), c_int(n_end))


def gemv_quantized_f32(X: np.ndarray, Wq: np.ndarray, fmt: int, N: int) -> np.ndarray:
    X = np.ascontiguousarray(X, dtype=np.float32)
    M, K = X.shape
    Y = np.empty((M, N), dtype=np.float32)
    _call(lib().orc_gemv_quantized_f32, _p(X), _p(Wq), _p(Y), c_int(fmt), c_int(M), c_int(N),
          c_int(K))
    return Y


def fused_rmsnorm_gemv_quantized(X_f16, gamma_f16, Wq, fmt, N, eps=1e-5) -> np.ndarray:
    X = np.ascontiguousarray(X_f16).view(np.uint16)
    g = np.ascontiguousarray(gamma_f16).view(np.uint16)
    M, K = X.shape
    Y = np.empty((M, N), dtype=np.uint16)
    _call(lib().orc_fused_rmsnorm_gemv_quantized, _p(X), _p(g), _p(Wq), _p(Y), c_int(fmt),
          c_int(M), c_int(N), c_int(K), c_float(eps))
    return Y.view(np.float16)


def fused_rmsnorm_gemv_quantized_f32(X, gamma, Wq, fmt, N, eps=1e-5) -> np.ndarray:
    X = np.ascontiguousarray(X, dtype=np.float32)
    g = np.ascontiguousarray(gamma, dtype=np.float32)
    M, K = X.shape
    Y = np.empty((M, N), dtype=np.float32)
    _call(lib().orc_fused_rmsnorm_gemv_quantized_f32, _p(X), _p(g), _p(Wq), _p(Y), c_int(fmt),
          c_int(M), c_int(N), c_int(K), c_float(eps))
    return Y


def fused_rmsnorm_gemv(X_f16, gamma_f16, W_f16, eps=1e-5) -> np.ndarray:
    X = np.ascontiguousarray(X_f16).view(np.uint16)
    g = np.ascontiguousarray(gamma_f16).view(np.uint16)
    W = np.ascontiguousarray(W_f16).view(np.uint16)
    M, K = X.shape
    N = W.shape[1]
    Y = np.empty((M, N), dtype=np.uint16)
    _call(lib().orc_fused_rmsnorm_gemv, _p(X), _p(g), _p(W), _p(Y), c_int(M), c_int(N), c_int(K),
          c_float(eps))
    return Y.view(np.float16)


def gemm_f16(A_f16, B_f16, transpose_b=False, alpha=1.0, beta=0.0, C_f16=None, ref_narrowing=False,
             transpose_a=False) -> np.ndarray:
    """alpha * A . op(B) + beta * C in the reference's order (lib/ops/gemm_cpu.cpp:544-568), stored with
    IEEE round-to-nearest-even or, ref_narrowing, with the reference GEMM's own narrowing (:142-160)."""
    A = np.ascontiguousarray(A_f16).view(np.uint16)
    B = np.ascontiguousarray(B_f16).view(np.uint16)
    K, M = A.shape if transpose_a else A.shape[::-1]
    N = B.shape[0] if transpose_b else B.shape[1]
    C = (np.zeros((M, N), dtype=np.uint16) if C_f16 is None
         else np.ascontiguousarray(C_f16).view(np.uint16).copy())
    _call(lib().orc_gemm_f16, _p(A), _p(B), _p(C), c_int(M), c_int(N), c_int(K), c_int(A.shape[1]),
          c_int(B.shape[1]), c_int(N), c_int(1 if transpose_a else 0), c_int(1 if transpose_b else 0),
          c_float(alpha), c_float(beta), c_int(1 if ref_narrowing else 0))
    return C.view(np.float16)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def gemm_bf16(A_bits, B_bits, transpose_b=False, alpha=1.0, beta=0.0, C_bits=None, transpose_a=False) -> np.ndarray:
    """The bfloat16 case of gemm_f16 (lib/ops/gemm_cpu.cpp:544-568, conversions :217-230); operands and
    result are bfloat16 bit patterns (uint16)."""
    A = np.ascontiguousarray(A_bits, dtype=np.uint16)
    B = np.ascontiguousarray(B_bits, dtype=np.uint16)
    K, M = A.shape if transpose_a else A.shape[::-1]
    N = B.shape[0] if transpose_b else B.shape[1]
    C = np.zeros((M, N), dtype=np.uint16) if C_bits is None else np.ascontiguousarray(C_bits, dtype=np.uint16).copy()
    _call(lib().orc_gemm_bf16, _p(A), _p(B), _p(C), c_int(M), c_int(N), c_int(K), c_int(A.shape[1]),
          c_int(B.shape[1]), c_int(N), c_int(1 if transpose_a else 0), c_int(1 if transpose_b else 0),
          c_float(alpha), c_float(beta))
    return C


def fused_layernorm_gemv(X_f16, gamma_f16, beta_f16, W_f16, eps=1e-5) -> np.ndarray:
    X = np.ascontiguousarray(X_f16).view(np.uint16)
    g = np.ascontiguousarray(gamma_f16).view(np.uint16)
    b = np.ascontiguousarray(beta_f16).view(np.uint16)
    W = np.ascontiguousarray(W_f16).view(np.uint16)
    M, K = X.shape
    N = W.shape[1]
    Y = np.empty((M, N), dtype=np.uint16)
    _call(lib().orc_fused_layernorm_gemv, _p(X), _p(g), _p(b), _p(W), _p(Y), c_int(M), c_int(N),
          c_int(K), c_float(eps))
    return Y.view(np.float16)


def rmsnorm_forward(X_f16, gamma_f16, eps=1e-5):
    """Returns (Y fp16 [N,D], rstd fp32 [N])."""
    X = np.ascontiguousarray(X_f16).view(np.uint16)
    g = np.ascontiguousarray(gamma_f16).view(np.uint16)
    N, D = X.shape
    Y, r = np.empty((N, D), np.uint16), np.empty(N, np.float32)
    _call(lib().orc_rmsnorm_forward, _p(X), _p(g), _p(Y), _p(r), c_int(N), c_int(D), c_float(eps))
    return Y.view(np.float16), r


def layernorm_forward(X_f16, gamma_f16, beta_f16, eps=1e-5):
    """Returns (Y fp16 [N,D], mean fp32 [N], rstd fp32 [N])."""
    X = np.ascontiguousarray(X_f16).view(np.uint16)
    g = np.ascontiguousarray(gamma_f16).view(np.uint16)
    b = np.ascontiguousarray(beta_f16).view(np.uint16)
    N, D = X.shape
    Y, m, r = np.empty((N, D), np.uint16), np.empty(N, np.float32), np.empty(N, np.float32)
    _call(lib().orc_layernorm_forward, _p(X), _p(g), _p(b), _p(Y), _p(m), _p(r), c_int(N), c_int(D),
          c_float(eps))
    return Y.view(np.float16), m, r


def swiglu_forward(gate_f16, up_f16):
    g = np.ascontiguousarray(gate_f16).view(np.uint16).ravel()
    u = np.ascontiguousarray(up_f16).view(np.uint16).ravel()
    out = np.empty(g.size, np.uint16)
    _call(lib().orc_swiglu_forward, _p(g), _p(u), _p(out), c_int(g.size))
    return out.view(np.float16)


def rope_forward(X_f16, cos_t, sin_t):
    """X [B,H,S,D] fp16 (a rotated copy is returned), tables [S, D/2] fp32."""
    X = np.ascontiguousarray(X_f16).view(np.uint16).copy()
    B, H, S, D = X.shape
    c = np.ascontiguousarray(cos_t, dtype=np.float32)
    s = np.ascontiguousarray(sin_t, dtype=np.float32)
    _call(lib().orc_rope_forward, _p(X), _p(c), _p(s), c_int(B), c_int(H), c_int(S), c_int(D))
    return X.view(np.float16)


def attention_forward(Q_f16, K_f16, V_f16, softmax_scale=0.0, causal=True, window=0, alibi_slopes=None,
                      return_lse=False, dot_order=1):
    """Q [B,Hq,Sq,D], K/V [B,Hkv,Sk,D] fp16 -> O [B,Hq,Sq,D] fp16 (and LSE [B,Hq,Sq] fp32).
    dot_order 1 is the order of the reference's AVX2 dot product, 0 that of its scalar one."""
    Q = np.ascontiguousarray(Q_f16).view(np.uint16)
    K = np.ascontiguousarray(K_f16).view(np.uint16)
    V = np.ascontiguousarray(V_f16).view(np.uint16)
    B, Hq, Sq, D = Q.shape
    _, Hkv, Sk, _ = K.shape
    O = np.empty((B, Hq, Sq, D), np.uint16)
    L = np.empty((B, Hq, Sq), np.float32) if return_lse else None
    sl = None if alibi_slopes is None else np.ascontiguousarray(alibi_slopes, dtype=np.float32)
    _call(lib().orc_attention_forward, _p(Q), _p(K), _p(V), _p(O), _p(L) if L is not None else None,
          c_int(B), c_int(Hq), c_int(Hkv), c_int(Sq), c_int(Sk), c_int(D), c_float(softmax_scale),
          c_int(1 if causal else 0), c_int(window), _p(sl) if sl is not None else None, c_int(dot_order))
    return (O.view(np.float16), L) if return_lse else O.view(np.float16)


def dequant_dot_f64(X: np.ndarray, Wq: np.ndarray, fmt: int, N: int) -> np.ndarray:
    X = np.ascontiguousarray(X, dtype=np.float64)
    M, K = X.shape
    Y = np.empty((M, N), dtype=np.float64)
    _call(lib().orc_dequant_dot_f64, _p(X), _p(Wq), _p(Y), c_int(fmt), c_int(M), c_int(N),
          c_int(K))
    return Y


def dequantize(Wq: np.ndarray, fmt: int, N: int, K: int) -> np.ndarray:
    out = np.empty((N, K), dtype=np.float32)
    _call(lib().orc_dequantize, _p(Wq), _p(out), c_int(fmt), c_int(N), c_int(K))
    return out


def scaled_rms(got: np.ndarray, want: np.ndarray) -> float:
    """rms(got - want) / rms(want), the reference's error measure (docs/numerics.md:10-28)."""
    g = np.asarray(got, dtype=np.float64).ravel()
    w = np.asarray(want, dtype=np.float64).ravel()
    den = np.sqrt(np.mean(w * w))
    num = np.sqrt(np.mean((g - w) ** 2))
    return float(num / den) if den > 0 else float(num)


# --------------------------------------------------------------------------------------
# The reference's own CPU backend (oracle/_ref), driven through its public tc_* C ABI.
# --------------------------------------------------------------------------------------
class RefLib:
    """Minimal ctypes driver for a libtensorcore-compatible shared library, used on the
    reference's CPU build.  Buffers are filled and read through tc_buffer_map exactly as the
    reference's tests do (tests/test_quantized.c:114-138)."""

    def __init__(self, path: str = REF_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        L = ctypes.CDLL(path)
        self.L = L
        vp = c_void_p
        L.tc_init.argtypes = [POINTER(vp)]
        L.tc_buffer_alloc.argtypes = [vp, c_size_t, POINTER(vp)]
        L.tc_buffer_free.argtypes = [vp, vp]
        L.tc_buffer_map.argtypes = [vp, POINTER(vp)]
        L.tc_quantized_size.argtypes = [c_int, c_int, c_int]
        L.tc_quantized_size.restype = c_size_t
        L.tc_quantize_weights.argtypes = [vp, vp, vp, c_int, c_int, c_int]
        L.tc_gemv_quantized.argtypes = [vp, vp, vp, vp, c_int, c_int, c_int, c_int]
        L.tc_fused_rmsnorm_gemv_quantized.argtypes = [vp, vp, vp, vp, vp, c_int, c_int, c_int,
                                                      c_int, c_float]
        L.tc_fused_rmsnorm_gemv.argtypes = [vp, vp, vp, vp, vp, c_int, c_int, c_int, c_float]
        L.tc_fused_layernorm_gemv.argtypes = [vp, vp, vp, vp, vp, vp, c_int, c_int, c_int,
                                              c_float]
        ctx = vp()
        st = L.tc_init(ctypes.byref(ctx))
        if st not in (0, -2):
            raise RuntimeError(f"tc_init -> {st}")
        self.ctx = ctx

    def _buf(self, data: np.ndarray | int):
        nbytes = data if isinstance(data, int) else data.nbytes
        h = c_void_p()
        st = self.L.tc_buffer_alloc(self.ctx, nbytes, ctypes.byref(h))
        assert st == 0, st
        p = c_void_p()
        assert self.L.tc_buffer_map(h, ctypes.byref(p)) == 0
        if not isinstance(data, int):
            ctypes.memmove(p, data.ctypes.data, nbytes)
        return h, p, nbytes

    def _read(self, p, nbytes, dtype):
        out = np.empty(nbytes // np.dtype(dtype).itemsize, dtype=dtype)
        ctypes.memmove(out.ctypes.data, p, nbytes)
        return out

    def _free(self, *hs):
        for h in hs:
            self.L.tc_buffer_free(self.ctx, h)

    def quantize_weights(self, W_f16: np.ndarray, fmt: int) -> np.ndarray:
        W = np.ascontiguousarray(W_f16).view(np.uint16)
        N, K = W.shape
        hw, _, _ = self._buf(W)
        hq, pq, nq = self._buf(int(self.L.tc_quantized_size(fmt, N, K)))
        st = self.L.tc_quantize_weights(self.ctx, hw, hq, fmt, N, K)
        assert st == 0, st
        out = self._read(pq, nq, np.uint8)
        self._free(hw, hq)
        return out

    def gemm_f16(self, A_f16, B_f16, transpose_b=False, alpha=1.0, beta=0.0, C_f16=None, dtype=0,
                 transpose_a=False) -> np.ndarray:
        """tc_gemm of the reference's CPU backend (include/tensorcore/gemm.h:16-50), fp16 in and out."""
        class Desc(ctypes.Structure):
            _fields_ = [("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32), ("a", c_int), ("b", c_int),
                        ("c", c_int), ("acc", c_int), ("ta", ctypes.c_bool), ("tb", ctypes.c_bool), ("alpha", c_float),
                        ("beta", c_float), ("lda", ctypes.c_int32), ("ldb", ctypes.c_int32), ("ldc", ctypes.c_int32)]
        A = np.ascontiguousarray(A_f16).view(np.uint16)
        B = np.ascontiguousarray(B_f16).view(np.uint16)
        K, M = A.shape if transpose_a else A.shape[::-1]
        N = B.shape[0] if transpose_b else B.shape[1]
        C = np.zeros((M, N), dtype=np.uint16) if C_f16 is None else np.ascontiguousarray(C_f16).view(np.uint16)
        ha, _, _ = self._buf(A)
        hb, _, _ = self._buf(B)
        hc, pc, nc = self._buf(C)
        d = Desc(M, N, K, dtype, dtype, dtype, 2, bool(transpose_a), bool(transpose_b), float(alpha), float(beta), 0, 0, 0)   # F16 = 0, BF16 = 1, F32 = 2
        self.L.tc_gemm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        st = self.L.tc_gemm(self.ctx, ctypes.byref(d), ha, hb, hc)
        assert st == 0, st
        out = self._read(pc, nc, np.uint16).reshape(M, N).view(np.float16)
        self._free(ha, hb, hc)
        return out

    def gemv_quantized(self, X_f16, Wq, fmt, N) -> np.ndarray:
        X = np.ascontiguousarray(X_f16).view(np.uint16)
        M, K = X.shape
        hx, _, _ = self._buf(X)
        hw, _, _ = self._buf(np.ascontiguousarray(Wq))
        hy, py, ny = self._buf(M * N * 2)
        st = self.L.tc_gemv_quantized(self.ctx, hx, hw, hy, fmt, M, N, K)
        assert st == 0, st
        out = self._read(py, ny, np.uint16).reshape(M, N).view(np.float16)
        self._free(hx, hw, hy)
        return out

    def fused_rmsnorm_gemv_quantized(self, X_f16, gamma_f16, Wq, fmt, N, eps=1e-5):
        X = np.ascontiguousarray(X_f16).view(np.uint16)
        M, K = X.shape
        hx, _, _ = self._buf(X)
        hg, _, _ = self._buf(np.ascontiguousarray(gamma_f16).view(np.uint16))
        hw, _, _ = self._buf(np.ascontiguousarray(Wq))
        hy, py, ny = self._buf(M * N * 2)
        st = self.L.tc_fused_rmsnorm_gemv_quantized(self.ctx, hx, hg, hw, hy, fmt, M, N, K,
                                                    c_float(eps))
        assert st == 0, st
        out = self._read(py, ny, np.uint16).reshape(M, N).view(np.float16)
        self._free(hx, hg, hw, hy)
        return out

    def fused_rmsnorm_gemv(self, X_f16, gamma_f16, W_f16, eps=1e-5):
        X = np.ascontiguousarray(X_f16).view(np.uint16)
        W = np.ascontiguousarray(W_f16).view(np.uint16)
        M, K = X.shape
        N = W.shape[1]
        hx, _, _ = self._buf(X)
        hg, _, _ = self._buf(np.ascontiguousarray(gamma_f16).view(np.uint16))
        hw, _, _ = self._buf(W)
        hy, py, ny = self._buf(M * N * 2)
        st = self.L.tc_fused_rmsnorm_gemv(self.ctx, hx, hg, hw, hy, M, N, K, c_float(eps))
        assert st == 0, st
        out = self._read(py, ny, np.uint16).reshape(M, N).view(np.float16)
        self._free(hx, hg, hw, hy)
        return out

    def fused_layernorm_gemv(self, X_f16, gamma_f16, beta_f16, W_f16, eps=1e-5):
        X = np.ascontiguousarray(X_f16).view(np.uint16)
        W = np.ascontiguousarray(W_f16).view(np.uint16)
        M, K = X.shape
        N = W.shape[1]
        hx, _, _ = self._buf(X)
        hg, _, _ = self._buf(np.ascontiguousarray(gamma_f16).view(np.uint16))
        hb, _, _ = self._buf(np.ascontiguousarray(beta_f16).view(np.uint16))
        hw, _, _ = self._buf(W)
        hy, py, ny = self._buf(M * N * 2)
        st = self.L.tc_fused_layernorm_gemv(self.ctx, hx, hg, hb, hw, hy, M, N, K, c_float(eps))
        assert st == 0, st
        out = self._read(py, ny, np.uint16).reshape(M, N).view(np.float16)
        self._free(hx, hg, hb, hw, hy)
        return out


    # --- the operations between the GEMVs of a decode step ---
    def rmsnorm_forward(self, X_f16, gamma_f16, eps=1e-5):
        X = np.ascontiguousarray(X_f16).view(np.uint16)
        N, D = X.shape
        self.L.tc_rmsnorm_forward.argtypes = [c_void_p] * 5 + [c_int, c_int, c_float]
        hx, _, _ = self._buf(X)
        hg, _, _ = self._buf(np.ascontiguousarray(gamma_f16).view(np.uint16))
        hy, py, ny = self._buf(N * D * 2)
        hr, pr, nr = self._buf(N * 4)
        st = self.L.tc_rmsnorm_forward(self.ctx, hx, hg, hy, hr, N, D, c_float(eps))
        assert st == 0, st
        out = self._read(py, ny, np.uint16).reshape(N, D).view(np.float16), self._read(pr, nr, np.float32)
        self._free(hx, hg, hy, hr)
        return out

    def layernorm_forward(self, X_f16, gamma_f16, beta_f16, eps=1e-5):
        X = np.ascontiguousarray(X_f16).view(np.uint16)
        N, D = X.shape
        self.L.tc_layernorm_forward.argtypes = [c_void_p] * 7 + [c_int, c_int, c_float]
        hx, _, _ = self._buf(X)
        hg, _, _ = self._buf(np.ascontiguousarray(gamma_f16).view(np.uint16))
        hb, _, _ = self._buf(np.ascontiguousarray(beta_f16).view(np.uint16))
        hy, py, ny = self._buf(N * D * 2)
        hm, pm, nm = self._buf(N * 4)
        hr, pr, nr = self._buf(N * 4)
        st = self.L.tc_layernorm_forward(self.ctx, hx, hg, hb, hy, hm, hr, N, D, c_float(eps))
        assert st == 0, st
        out = (self._read(py, ny, np.uint16).reshape(N, D).view(np.float16), self._read(pm, nm, np.float32),
               self._read(pr, nr, np.float32))
        self._free(hx, hg, hb, hy, hm, hr)
        return out

    def swiglu_forward(self, gate_f16, up_f16):
        g = np.ascontiguousarray(gate_f16).view(np.uint16).ravel()
        self.L.tc_swiglu_forward.argtypes = [c_void_p] * 4 + [c_int]
        hg, _, _ = self._buf(g)
        hu, _, _ = self._buf(np.ascontiguousarray(up_f16).view(np.uint16).ravel())
        ho, po, no = self._buf(g.size * 2)
        st = self.L.tc_swiglu_forward(self.ctx, hg, hu, ho, g.size)
        assert st == 0, st
        out = self._read(po, no, np.uint16).view(np.float16)
        self._free(hg, hu, ho)
        return out

    def rope_forward(self, X_f16, cos_t, sin_t):
        X = np.ascontiguousarray(X_f16).view(np.uint16)
        B, H, S, D = X.shape
        self.L.tc_rope_forward.argtypes = [c_void_p] * 4 + [c_int] * 4
        hx, px, nx = self._buf(X)
        hc, _, _ = self._buf(np.ascontiguousarray(cos_t, dtype=np.float32))
        hs, _, _ = self._buf(np.ascontiguousarray(sin_t, dtype=np.float32))
        st = self.L.tc_rope_forward(self.ctx, hx, hc, hs, B, H, S, D)
        assert st == 0, st
        out = self._read(px, nx, np.uint16).reshape(B, H, S, D).view(np.float16)
        self._free(hx, hc, hs)
        return out


    def attention_forward(self, Q_f16, K_f16, V_f16, softmax_scale=0.0, causal=True, window=0,
                          alibi_slopes=None, return_lse=False):
        import ctypes

        class Desc(ctypes.Structure):     # include/tensorcore/attention.h:24-52
            _fields_ = [("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("seq_q", ctypes.c_int32),
                        ("seq_kv", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("io_dtype", ctypes.c_int),
                        ("accum_dtype", ctypes.c_int), ("softmax_scale", ctypes.c_float), ("causal", ctypes.c_bool),
                        ("return_lse", ctypes.c_bool), ("kv_heads", ctypes.c_int32), ("window_size", ctypes.c_int32),
                        ("alibi_slopes", ctypes.c_void_p)]

        Q = np.ascontiguousarray(Q_f16).view(np.uint16)
        K = np.ascontiguousarray(K_f16).view(np.uint16)
        V = np.ascontiguousarray(V_f16).view(np.uint16)
        B, Hq, Sq, D = Q.shape
        _, Hkv, Sk, _ = K.shape
        sl = None if alibi_slopes is None else np.ascontiguousarray(alibi_slopes, dtype=np.float32)
        d = Desc(B, Hq, Sq, Sk, D, 0, 2, softmax_scale, bool(causal), bool(return_lse), Hkv, window,
                 sl.ctypes.data if sl is not None else None)
        self.L.tc_attention_forward.argtypes = [c_void_p] * 7
        hq, _, _ = self._buf(Q)
        hk, _, _ = self._buf(K)
        hv, _, _ = self._buf(V)
        ho, po, no = self._buf(Q.size * 2)
        hl, pl, nl = self._buf(B * Hq * Sq * 4) if return_lse else (None, None, 0)
        st = self.L.tc_attention_forward(self.ctx, ctypes.byref(d), hq, hk, hv, ho, hl)
        assert st == 0, st
        out = self._read(po, no, np.uint16).reshape(B, Hq, Sq, D).view(np.float16)
        lse = self._read(pl, nl, np.float32).reshape(B, Hq, Sq) if return_lse else None
        self._free(hq, hk, hv, ho, *( [hl] if hl else []))
        return (out, lse) if return_lse else out


def ref_available() -> bool:
    return os.path.exists(REF_SO)
