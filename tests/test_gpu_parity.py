"""GPU: parity of the CUDA path, called through the C ABI, against the oracle.

Bars: quantiser bytes identical; fp32 activations and outputs within scaled-RMS 1e-4 of an fp64
dequantise-and-dot and of the oracle's fp32 path (the bound stated for fp32 activations;
observed 2-3e-5: the kernels stage activations as int16 with one scale per 32-element block and
take exact integer dot products, so the error is the 2^-16-of-block-maximum quantisation of x);
fp16-ABI GEMV / fused outputs within 3e-4 of the oracle's fp16 outputs (both sides rounded to
fp16, so the difference is fp16 rounding flips: observed 1.0-1.9e-4; the bound stated for fp16
activations is 2e-3) and within 2.5e-4 of fp64 (the fp16 output rounding floor is 2.1e-4).  Batched
calls (Q4_0, fp16 activations, five rows or more, or four rows of a large matrix: `batched_rows`
below) run on the tcgen05 kernel, which rounds dequantised weights
to fp16 (observed 1.8e-4): for those the bar is the 2e-3 that applies to fp16 activations.
"""
import os

import numpy as np
import pytest

from conftest import GOLDEN

pytestmark = pytest.mark.gpu

Q = {"q4_0": 0, "q8_0": 1}
TOL_VS_ORACLE_F16 = 3e-4
TOL_VS_F64_F16OUT = 2.5e-4
TOL_F32 = 1e-4
TOL_F16_ACT = 2e-3


def batched_rows(M, N, K):
    """The dispatcher's rule for the batched tensor-core kernel (csrc/kernels.h batched_tc_rows)."""
    return M >= 5 or (M == 4 and (K >= 8192 or N > 4096))


def tol_f16(tc):
    """Bar against the oracle's fp16 output for the kernel that ran last."""
    return TOL_F16_ACT if "tcgen05" in tc.cuda_last_kernel_name() else TOL_VS_ORACLE_F16


def make_weights(rng, N, K):
    return (rng.standard_normal((N, K)) * 0.02).astype(np.float32).astype(np.float16)


def dev(ctx, arr):
    return ctx.buffer_from_array(np.ascontiguousarray(arr))


def gpu_quantize(tc, ctx, W16, fmt):
    N, K = W16.shape
    with dev(ctx, W16.view(np.uint16)) as bw, ctx.buffer(tc.quantized_size(fmt, N, K)) as bq:
        ctx.quantize_weights(bw, bq, fmt, N, K)
        return bq.to_numpy((tc.quantized_size(fmt, N, K),), np.uint8)


def gpu_gemv(tc, ctx, X, Wq, fmt, N, y_f32=False, gamma=None, eps=1e-5, stream=None):
    """X: float16 or float32 [M,K].  Uses the reference entry points when both types are
    fp16 and no stream is given, else the additive *_ex forms."""
    M, K = X.shape
    x_f32 = X.dtype == np.float32
    ydt = np.float32 if y_f32 else np.float16
    bx, bw = dev(ctx, X), dev(ctx, Wq)
    by = ctx.buffer(M * N * np.dtype(ydt).itemsize)
    bg = dev(ctx, gamma) if gamma is not None else None
    try:
        plain = not x_f32 and not y_f32 and stream is None
        if gamma is None:
            if plain:
                ctx.gemv_quantized(bx, bw, by, fmt, M, N, K)
            else:
                tc.gemv_quantized_ex(ctx, bx, bw, by, fmt, M, N, K, "f32" if x_f32 else "f16",
                                     "f32" if y_f32 else "f16", stream)
        else:
            if plain:
                ctx.fused_rmsnorm_gemv_quantized(bx, bg, bw, by, fmt, M, N, K, eps)
            else:
                tc.fused_rmsnorm_gemv_quantized_ex(ctx, bx, bg, bw, by, fmt, M, N, K, eps,
                                                   "f32" if x_f32 else "f16",
                                                   "f32" if y_f32 else "f16", stream)
        if stream is not None:
            stream.sync()
        return by.to_numpy((M, N), ydt)
    finally:
        for b in (bx, bw, by, bg):
            if b is not None:
                b.close()


# ---------------------------------------------------------------------------------------
# Quantiser: bit-exact
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["q4_0", "q8_0"])
@pytest.mark.parametrize("shape", [(1, 32), (8, 32), (130, 256), (97, 512), (33, 4096),
                                   (1024, 4096)])
def test_quantiser_bytes_match_oracle(tc, ctx, oracle, tag, shape):
    rng = np.random.default_rng(Q[tag] * 100003 + shape[0] * 31 + shape[1])
    W = make_weights(rng, *shape)
    W[0, :32] = 0
    if shape[0] > 1:
        W[1, :32] = np.float16(-0.25)
    got = gpu_quantize(tc, ctx, W, Q[tag])
    assert np.array_equal(got, oracle.quantize_weights(W, Q[tag]))
    assert tc.last_backend() == tc.TC_BACKEND_CUDA
    assert "quantize" in tc.cuda_last_kernel_name()


@pytest.mark.parametrize("tag", ["q4_0", "q8_0"])
def test_quantiser_matches_reference_golden_bytes(tc, ctx, tag):
    g = np.load(os.path.join(GOLDEN, "quantized_path.npz"))
    for key in sorted({k.rsplit("_", 1)[0] for k in g.files if k.startswith(tag)}):
        W = g[key + "_W"].view(np.float16)
        assert np.array_equal(gpu_quantize(tc, ctx, W, Q[tag]), g[key + "_Wq"]), key


def test_quantiser_extreme_values(tc, ctx, oracle):
    """Subnormal inputs, the largest finite fp16, mixed signs, exact ties."""
    rng = np.random.default_rng(77)
    W = np.zeros((8, 64), dtype=np.float16)
    W[0, :32] = np.float16(65504)
    W[1, :32] = np.array([5.96e-8 * (i + 1) for i in range(32)], dtype=np.float16)
    W[2, :32] = np.linspace(-8, 8, 32).astype(np.float16)           # ties at .5 after scaling
    W[3, :32] = (np.arange(32) - 16).astype(np.float16) * np.float16(0.5)
    W[4] = (rng.standard_normal(64) * 1e-4).astype(np.float16)
    W[5] = (rng.standard_normal(64) * 100).astype(np.float16)
    W[6, ::2] = np.float16(-1.0)
    W[7, 33] = np.float16(-6.1e-5)
    for fmt in (0, 1):
        assert np.array_equal(gpu_quantize(tc, ctx, W, fmt), oracle.quantize_weights(W, fmt))


# ---------------------------------------------------------------------------------------
# GEMV, fp16 ABI
# ---------------------------------------------------------------------------------------
SHAPES = [
    # (N, K, M) - streaming kernel (K % 256 == 0) and the generic path (other K)
    (128, 256, 1), (130, 256, 1), (129, 256, 2), (1, 256, 1), (97, 512, 3), (64, 1024, 4),
    (33, 4096, 2), (500, 2816, 1), (300, 768, 5), (64, 512, 9), (4100, 256, 4), (40, 8192, 4),
    (3, 32, 1), (8, 64, 2), (77, 96, 1), (40, 1376, 1),
]


@pytest.mark.parametrize("tag", ["q4_0", "q8_0"])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemv_fp16_abi(tc, ctx, oracle, tag, shape):
    N, K, M = shape
    fmt = Q[tag]
    rng = np.random.default_rng(N * 7919 + K + M)
    Wq = oracle.quantize_weights(make_weights(rng, N, K), fmt)
    X = rng.standard_normal((M, K)).astype(np.float32).astype(np.float16)
    got = gpu_gemv(tc, ctx, X, Wq, fmt, N)
    want16 = oracle.gemv_quantized(X, Wq, fmt, N)
    want64 = oracle.dequant_dot_f64(X.astype(np.float64), Wq, fmt, N)
    batched = "tcgen05" in tc.cuda_last_kernel_name()
    assert batched == (tag == "q4_0" and batched_rows(M, N, K) and K % 256 == 0)
    assert oracle.scaled_rms(got, want16) <= tol_f16(tc)
    if M * N >= 64:   # an RMS over a handful of fp16 roundings is not a statistic
        assert oracle.scaled_rms(got, want64) <= (TOL_F16_ACT if batched else TOL_VS_F64_F16OUT)
    assert tc.last_backend() == tc.TC_BACKEND_CUDA
    name = tc.cuda_last_kernel_name()
    assert ("generic" not in name) == (K % 256 == 0), name   # fast paths need K % 256 == 0


@pytest.mark.parametrize("tag", ["q4_0", "q8_0"])
def test_gemv_matches_reference_golden_outputs(tc, ctx, oracle, tag):
    g = np.load(os.path.join(GOLDEN, "quantized_path.npz"))
    for key in sorted({k.rsplit("_", 1)[0] for k in g.files if k.startswith(tag)}):
        N = int(key.split("_N")[1].split("_")[0])
        X = g[key + "_X"].view(np.float16)
        gam = g[key + "_gamma"].view(np.float16)
        Wq = g[key + "_Wq"]
        got = gpu_gemv(tc, ctx, X, Wq, Q[tag], N)
        assert oracle.scaled_rms(got, g[key + "_Y"].view(np.float16)) <= TOL_VS_ORACLE_F16, key
        gotf = gpu_gemv(tc, ctx, X, Wq, Q[tag], N, gamma=gam)
        assert oracle.scaled_rms(gotf, g[key + "_Yfused"].view(np.float16)) <= TOL_VS_ORACLE_F16, key


def test_gguf_known_answer_is_bit_exact(tc, ctx):
    # tests/test_gguf.c:119-122,267-279 -> 0x5100
    blk = np.array([0x00, 0x38] + [0xAB] * 16, dtype=np.uint8)
    x = np.full((1, 32), 0x3C00, dtype=np.uint16).view(np.float16)
    y = gpu_gemv(tc, ctx, x, blk, 0, 1)
    assert y.view(np.uint16)[0, 0] == 0x5100


# ---------------------------------------------------------------------------------------
# fp32 activations / outputs (additive entry points)
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["q4_0", "q8_0"])
@pytest.mark.parametrize("shape", [(130, 256, 1), (97, 512, 3), (256, 4096, 1), (8, 64, 2)])
def test_gemv_fp32(tc, ctx, oracle, tag, shape):
    N, K, M = shape
    fmt = Q[tag]
    rng = np.random.default_rng(N + K * 31 + M)
    Wq = oracle.quantize_weights(make_weights(rng, N, K), fmt)
    X = rng.standard_normal((M, K)).astype(np.float32)
    want64 = oracle.dequant_dot_f64(X.astype(np.float64), Wq, fmt, N)
    got = gpu_gemv(tc, ctx, X, Wq, fmt, N, y_f32=True)
    assert oracle.scaled_rms(got, want64) <= TOL_F32
    assert oracle.scaled_rms(got, oracle.gemv_quantized_f32(X, Wq, fmt, N)) <= TOL_F32
    # fp16 activations, fp32 output
    X16 = X.astype(np.float16)
    got16 = gpu_gemv(tc, ctx, X16, Wq, fmt, N, y_f32=True)
    assert oracle.scaled_rms(got16, want64) <= TOL_F16_ACT
    assert oracle.scaled_rms(
        got16, oracle.dequant_dot_f64(X16.astype(np.float64), Wq, fmt, N)) <= TOL_F32


# ---------------------------------------------------------------------------------------
# Fused RMSNorm + quantized GEMV
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["q4_0", "q8_0"])
@pytest.mark.parametrize("shape", [(97, 256, 1), (96, 256, 2), (130, 1024, 4), (64, 4096, 1),
                                   (12, 64, 1), (300, 768, 5)])
def test_fused_rmsnorm_gemv_quantized(tc, ctx, oracle, tag, shape):
    N, K, M = shape
    fmt = Q[tag]
    rng = np.random.default_rng(N * 3 + K * 5 + M)
    Wq = oracle.quantize_weights(make_weights(rng, N, K), fmt)
    X = rng.standard_normal((M, K)).astype(np.float32).astype(np.float16)
    gam = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32).astype(np.float16)
    got = gpu_gemv(tc, ctx, X, Wq, fmt, N, gamma=gam)
    want = oracle.fused_rmsnorm_gemv_quantized(X, gam, Wq, fmt, N, 1e-5)
    # Q4_0 with enough fp16 rows (batched_rows) runs on the tensor-core kernel (rows normalised to fp16, weights
    # dequantised to fp16): the 2e-3 bound of fp16 activations applies there, as in test_gpu_batched.py
    batched = fmt == 0 and batched_rows(M, N, K) and K % 256 == 0
    assert oracle.scaled_rms(got, want) <= (TOL_F16_ACT if batched else TOL_VS_ORACLE_F16)
    # fp32 form
    Xf = rng.standard_normal((M, K)).astype(np.float32)
    gf = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    gotf = gpu_gemv(tc, ctx, Xf, Wq, fmt, N, y_f32=True, gamma=gf)
    wantf = oracle.fused_rmsnorm_gemv_quantized_f32(Xf, gf, Wq, fmt, N, 1e-5)
    assert oracle.scaled_rms(gotf, wantf) <= TOL_F32


# ---------------------------------------------------------------------------------------
# Fused norm + dense fp16 GEMV
# ---------------------------------------------------------------------------------------
def gpu_dense(tc, ctx, X, gam, bet, W):
    M, K = X.shape
    N = W.shape[1]
    bufs = [dev(ctx, a.view(np.uint16)) for a in (X, gam, W)]
    bb = dev(ctx, bet.view(np.uint16)) if bet is not None else None
    by = ctx.buffer(M * N * 2)
    try:
        if bet is None:
            ctx.fused_rmsnorm_gemv(bufs[0], bufs[1], bufs[2], by, M, N, K, 1e-5)
        else:
            ctx.fused_layernorm_gemv(bufs[0], bufs[1], bb, bufs[2], by, M, N, K, 1e-5)
        return by.to_numpy((M, N), np.float16)
    finally:
        for b in bufs + [by] + ([bb] if bb else []):
            b.close()


@pytest.mark.parametrize("shape", [(1, 128, 256), (2, 96, 512), (4, 40, 1024), (1, 33, 64),
                                   (5, 1024, 4096), (1, 11008, 4096), (3, 77, 100)])
def test_dense_fused_norm_gemv(tc, ctx, oracle, shape):
    M, N, K = shape
    rng = np.random.default_rng(M + N * 3 + K * 7)
    X = rng.standard_normal((M, K)).astype(np.float16)
    gam = (1 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    bet = (0.1 * rng.standard_normal(K)).astype(np.float16)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float16)
    if N * K <= 1 << 22:
        want_r = oracle.fused_rmsnorm_gemv(X, gam, W, 1e-5)
        want_l = oracle.fused_layernorm_gemv(X, gam, bet, W, 1e-5)
        cols = slice(None)
    else:  # big case: check a slice of the columns against the oracle
        cols = slice(0, N, 37)
        Ws = np.ascontiguousarray(W[:, cols])
        want_r = oracle.fused_rmsnorm_gemv(X, gam, Ws, 1e-5)
        want_l = oracle.fused_layernorm_gemv(X, gam, bet, Ws, 1e-5)
    got_r = gpu_dense(tc, ctx, X, gam, None, W)[:, cols]
    got_l = gpu_dense(tc, ctx, X, gam, bet, W)[:, cols]
    assert oracle.scaled_rms(got_r, want_r) <= TOL_VS_ORACLE_F16
    assert oracle.scaled_rms(got_l, want_l) <= TOL_VS_ORACLE_F16


@pytest.mark.parametrize("shape", [(8, 1024, 4096), (32, 2048, 1024), (40, 264, 520), (7, 77, 100)])
def test_dense_fused_norm_gemv_batched(tc, ctx, oracle, shape):
    """Five rows or more: the rows are normalised once (fp16, as the reference rounds them before
    its GEMM) and multiplied on the tensor cores; shapes the tiled copies cannot describe (N not a
    multiple of 8) keep the four-rows-at-a-time kernels."""
    M, N, K = shape
    rng = np.random.default_rng(M * 5 + N + K)
    X = rng.standard_normal((M, K)).astype(np.float16)
    gam = (1 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    bet = (0.1 * rng.standard_normal(K)).astype(np.float16)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float16)
    got_r = gpu_dense(tc, ctx, X, gam, None, W)
    name_r = tc.cuda_last_kernel_name()
    got_l = gpu_dense(tc, ctx, X, gam, bet, W)
    name_l = tc.cuda_last_kernel_name()
    if N % 8 == 0:
        assert name_r == "rmsnorm_rows_gemm_tcgen05_sm100" and name_l == "layernorm_rows_gemm_tcgen05_sm100"
    else:
        assert "tcgen05" not in name_r and "tcgen05" not in name_l
    assert oracle.scaled_rms(got_r, oracle.fused_rmsnorm_gemv(X, gam, W, 1e-5)) <= TOL_VS_ORACLE_F16
    assert oracle.scaled_rms(got_l, oracle.fused_layernorm_gemv(X, gam, bet, W, 1e-5)) <= TOL_VS_ORACLE_F16
    assert tc.take_device_error(ctx) == 0


def test_dense_fused_matches_reference_golden(tc, ctx, oracle):
    g = np.load(os.path.join(GOLDEN, "dense_fused.npz"))
    for key in sorted({k.rsplit("_", 1)[0] for k in g.files}):
        X, gam, bet, W = (g[key + s].view(np.float16) for s in ("_X", "_gamma", "_beta", "_W"))
        assert oracle.scaled_rms(gpu_dense(tc, ctx, X, gam, None, W),
                                 g[key + "_Yrms"].view(np.float16)) <= TOL_VS_ORACLE_F16, key
        assert oracle.scaled_rms(gpu_dense(tc, ctx, X, gam, bet, W),
                                 g[key + "_Yln"].view(np.float16)) <= TOL_VS_ORACLE_F16, key


# ---------------------------------------------------------------------------------------
# Full BASELINE shapes
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", [("q4_0", 4096, 4096, 1), ("q8_0", 11008, 4096, 1),
                                  ("q4_0", 32000, 4096, 1), ("q4_0", 4096, 11008, 1),
                                  ("q4_0", 14336, 4096, 1), ("q4_0", 14336, 4096, 4),
                                  ("q4_0", 14336, 4096, 8), ("q4_0", 14336, 4096, 16),
                                  ("q4_0", 14336, 4096, 32),
                                  ("q4_0", 1024, 8192, 1), ("q4_0", 8192, 28672, 1)])
def test_full_size_shapes(tc, ctx, oracle, case):
    tag, N, K, M = case
    fmt = Q[tag]
    rng = np.random.default_rng(N ^ K ^ M)
    W = make_weights(rng, N, K)
    Wq = gpu_quantize(tc, ctx, W, fmt)
    # quantiser: sampled rows against the oracle (the whole matrix when it is small)
    rows = np.unique(np.concatenate([[0, N - 1], rng.integers(0, N, 64)]))
    bb = 18 if fmt == 0 else 34
    Wq_rows = Wq.reshape(N, K // 32 * bb)[rows]
    assert np.array_equal(Wq_rows.ravel(), oracle.quantize_weights(W[rows], fmt))
    X = rng.standard_normal((M, K)).astype(np.float32).astype(np.float16)
    got = gpu_gemv(tc, ctx, X, Wq, fmt, N)
    tol = tol_f16(tc)
    want = oracle.gemv_quantized(X[:1], Wq, fmt, N)          # oracle on the first row: < 1 s
    assert oracle.scaled_rms(got[:1], want) <= tol
    if M > 1:  # remaining rows: sampled output columns
        cols = rng.integers(0, N, 256)
        sub = np.ascontiguousarray(Wq.reshape(N, -1)[cols]).ravel()
        want_s = oracle.gemv_quantized(X, sub, fmt, len(cols))
        assert oracle.scaled_rms(got[:, cols], want_s) <= tol
    # size-independent property: linearity in the activations (fp32 entry point)
    Xa = rng.standard_normal((1, K)).astype(np.float32)
    Xb = rng.standard_normal((1, K)).astype(np.float32)
    ya = gpu_gemv(tc, ctx, Xa, Wq, fmt, N, y_f32=True)
    yb = gpu_gemv(tc, ctx, Xb, Wq, fmt, N, y_f32=True)
    yab = gpu_gemv(tc, ctx, Xa + 2 * Xb, Wq, fmt, N, y_f32=True)
    assert oracle.scaled_rms(yab, ya + 2 * yb) <= TOL_F32


@pytest.mark.parametrize("variant", ["simt", "stream"])
@pytest.mark.parametrize("tag", ["q4_0", "q8_0"])
def test_repeated_launches_on_cache_resident_weights(tc, ctx, oracle, variant, tag):
    # "simt" is the box kernel (what the dispatcher picks), "stream" the streaming kernel
    """Weights that stay in L2 make the copy engine refill ring slots as fast as it ever will:
    the timing in which a slot released before its loads were consumed would show stale data."""
    fmt, N, K, M = Q[tag], 2048, 4096, 1
    rng = np.random.default_rng(99)
    Wq = oracle.quantize_weights(make_weights(rng, N, K), fmt)
    X = rng.standard_normal((M, K)).astype(np.float32)
    want = oracle.dequant_dot_f64(X.astype(np.float64), Wq, fmt, N)
    bx, bw, by = dev(ctx, X), dev(ctx, Wq), ctx.buffer(M * N * 4)
    try:
        tc.set_gemv_variant(variant)
        for rep in range(60):
            tc.gemv_quantized_ex(ctx, bx, bw, by, fmt, M, N, K, "f32", "f32", None)
            got = by.to_numpy((M, N), np.float32)
            assert oracle.scaled_rms(got, want) <= TOL_F32, rep
    finally:
        tc.set_gemv_variant("auto")
        for b in (bx, bw, by):
            b.close()
    assert tc.take_device_error(ctx) == 0


@pytest.mark.parametrize("x_f32", [False, True])
def test_config2_fused_rmsnorm_q8_0_full_size(tc, ctx, oracle, x_f32):
    """Q8_0 11008 x 4096 with the RMSNorm prologue fused, fp16 and fp32 activations."""
    fmt, N, K = 1, 11008, 4096
    rng = np.random.default_rng(20404 + x_f32)
    Wq = gpu_quantize(tc, ctx, make_weights(rng, N, K), fmt)
    xdt = np.float32 if x_f32 else np.float16
    X = rng.standard_normal((1, K)).astype(np.float32).astype(xdt)
    gam = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32).astype(xdt)
    if x_f32:
        got = gpu_gemv(tc, ctx, X, Wq, fmt, N, y_f32=True, gamma=gam)
        assert oracle.scaled_rms(got, oracle.fused_rmsnorm_gemv_quantized_f32(X, gam, Wq, fmt, N, 1e-5)) <= TOL_F32
    else:
        got = gpu_gemv(tc, ctx, X, Wq, fmt, N, gamma=gam)
        assert oracle.scaled_rms(got, oracle.fused_rmsnorm_gemv_quantized(X, gam, Wq, fmt, N, 1e-5)) <= TOL_VS_ORACLE_F16
    plain = gpu_gemv(tc, ctx, X, Wq, fmt, N, y_f32=x_f32)
    want = oracle.gemv_quantized_f32(X, Wq, fmt, N) if x_f32 else oracle.gemv_quantized(X, Wq, fmt, N)
    assert oracle.scaled_rms(plain, want) <= (TOL_F32 if x_f32 else TOL_VS_ORACLE_F16)


@pytest.mark.parametrize("shape", [(28672, 8192), (128256, 8192)])
def test_llama70b_shapes_sampled_rows(tc, ctx, oracle, shape):
    """The 70B gate/up and lm_head matrices (up to 590 MB of Q4_0): weights are drawn and
    quantised on the device; quantiser bytes and GEMV results are checked on sampled rows."""
    from tensorcore_b200 import decode as D
    N, K = shape
    fmt, bb = 0, 18
    rng = np.random.default_rng(N + K)
    w16 = D.device_weights_fp16(N, K, 0x70B + N)
    bq = D.quantize_into(ctx, w16, fmt)
    rows = np.unique(np.concatenate([[0, 1, N - 1], rng.integers(0, N, 200)]))
    W_rows = w16[rows.tolist()].cpu().numpy()
    del w16
    row_bytes = K // 32 * bb
    Wq_rows = np.concatenate([bq.to_numpy((row_bytes,), np.uint8, offset=int(r) * row_bytes) for r in rows])
    assert np.array_equal(Wq_rows, oracle.quantize_weights(W_rows, fmt))
    X = rng.standard_normal((1, K)).astype(np.float16)
    with dev(ctx, X) as bx, ctx.buffer(N * 2) as by:
        ctx.gemv_quantized(bx, bq, by, fmt, 1, N, K)
        got = by.to_numpy((1, N), np.float16)
    want = oracle.gemv_quantized(X, Wq_rows, fmt, len(rows))
    assert oracle.scaled_rms(got[:, rows], want) <= TOL_VS_ORACLE_F16
    assert np.all(np.isfinite(got))
    bq.close()


# ---------------------------------------------------------------------------------------
# Activations that stress the int16 staging: outliers, heavy tails, empty blocks, non-finite values
# ---------------------------------------------------------------------------------------
def _stress_rows(rng, K):
    rows = {}
    x = rng.standard_normal(K)
    for f in (100.0, 1000.0):                      # one element f times its block-mates, in 16 blocks
        y = x.copy()
        for b in rng.choice(K // 32, 16, replace=False):
            y[32 * b + rng.integers(0, 32)] *= f
        rows[f"outlier{int(f)}"] = y
    rows["student_t2"] = rng.standard_t(2, K)
    z = x.copy()
    z[64:96] = 0.0
    z[K - 32:] = 0.0
    rows["zero_blocks"] = z
    rows["tiny"] = x * 1e-4
    return rows


@pytest.mark.parametrize("tag", ["q4_0", "q8_0"])
@pytest.mark.parametrize("variant", ["simt", "stream"])
def test_outlier_activations_single_operation(tc, ctx, oracle, tag, variant):
    fmt, N, K = Q[tag], 512, 4096
    rng = np.random.default_rng(4242 + fmt)
    Wq = oracle.quantize_weights(make_weights(rng, N, K), fmt)
    try:
        tc.set_gemv_variant(variant)
        for name, row in _stress_rows(rng, K).items():
            X32 = row.astype(np.float32)[None, :]
            want = oracle.dequant_dot_f64(X32.astype(np.float64), Wq, fmt, N)
            got = gpu_gemv(tc, ctx, X32, Wq, fmt, N, y_f32=True)
            assert oracle.scaled_rms(got, want) <= TOL_F32, name
            X16 = X32.astype(np.float16)
            if np.all(np.isfinite(X16)):
                want16 = oracle.dequant_dot_f64(X16.astype(np.float64), Wq, fmt, N)
                got16 = gpu_gemv(tc, ctx, X16, Wq, fmt, N, y_f32=True)
                assert oracle.scaled_rms(got16, want16) <= TOL_F32, name   # fp16 values are staged exactly enough
                assert oracle.scaled_rms(gpu_gemv(tc, ctx, X16, Wq, fmt, N), want16) <= TOL_F16_ACT, name
            gam = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
            wantf = oracle.fused_rmsnorm_gemv_quantized_f32(X32, gam, Wq, fmt, N, 1e-5)
            gotf = gpu_gemv(tc, ctx, X32, Wq, fmt, N, y_f32=True, gamma=gam)
            assert oracle.scaled_rms(gotf, wantf) <= TOL_F32, name
    finally:
        tc.set_gemv_variant("auto")


def test_outlier_activations_persistent_launch(tc, ctx, oracle):
    """The same rows through a recorded list (the persistent decode kernel), plain and fused."""
    fmt, N, K = 0, 512, 4096
    rng = np.random.default_rng(777)
    Wq = oracle.quantize_weights(make_weights(rng, N, K), fmt)
    gam = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    bw, bg = dev(ctx, Wq), dev(ctx, gam)
    y1, y2 = ctx.buffer(N * 4), ctx.buffer(N * 4)
    s = ctx.stream()
    for name, row in _stress_rows(rng, K).items():
        X32 = row.astype(np.float32)[None, :]
        bx = dev(ctx, X32)
        tc.gemv_quantized_ex(ctx, bx, bw, y1, fmt, 1, N, K, "f32", "f32", s)
        tc.fused_rmsnorm_gemv_quantized_ex(ctx, bx, bg, bw, y2, fmt, 1, N, K, 1e-5, "f32", "f32", s)
        s.sync()
        assert "persistent" in tc.cuda_last_kernel_name()
        want = oracle.dequant_dot_f64(X32.astype(np.float64), Wq, fmt, N)
        assert oracle.scaled_rms(y1.to_numpy((1, N), np.float32), want) <= TOL_F32, name
        wantf = oracle.fused_rmsnorm_gemv_quantized_f32(X32, gam, Wq, fmt, N, 1e-5)
        assert oracle.scaled_rms(y2.to_numpy((1, N), np.float32), wantf) <= TOL_F32, name
        bx.close()
    s.close()
    for b in (bw, bg, y1, y2):
        b.close()
    assert tc.take_device_error(ctx) == 0


@pytest.mark.parametrize("bad", [np.nan, np.inf, -np.inf])
def test_non_finite_activations_propagate(tc, ctx, oracle, bad):
    """The reference multiplies and accumulates in fp32, so a NaN or an infinity in x makes every
    result that uses it non-finite (lib/ops/quantized_cpu.cpp:193-228); the int16 staging must
    not turn it into a plausible finite number."""
    fmt, N, K = 0, 256, 1024
    rng = np.random.default_rng(99)
    Wq = oracle.quantize_weights(make_weights(rng, N, K), fmt)
    X = rng.standard_normal((1, K)).astype(np.float32)
    X[0, 517] = bad
    want = oracle.gemv_quantized_f32(X, Wq, fmt, N)
    assert not np.any(np.isfinite(want))
    for variant in ("simt", "stream"):
        try:
            tc.set_gemv_variant(variant)
            assert not np.any(np.isfinite(gpu_gemv(tc, ctx, X, Wq, fmt, N, y_f32=True))), variant
            if np.isnan(bad):
                X16 = X.astype(np.float16)
                assert not np.any(np.isfinite(gpu_gemv(tc, ctx, X16, Wq, fmt, N).astype(np.float32))), variant
        finally:
            tc.set_gemv_variant("auto")
    # recorded list -> persistent kernel; the second operation reads the first one's NaNs
    bx, bw = dev(ctx, X), dev(ctx, Wq)
    W2 = oracle.quantize_weights(make_weights(rng, 64, N), fmt)
    bw2, y1, y2 = dev(ctx, W2), ctx.buffer(N * 4), ctx.buffer(64 * 4)
    s = ctx.stream()
    tc.gemv_quantized_ex(ctx, bx, bw, y1, fmt, 1, N, K, "f32", "f32", s)
    tc.gemv_quantized_ex(ctx, y1, bw2, y2, fmt, 1, 64, N, "f32", "f32", s)
    s.sync()
    assert "persistent" in tc.cuda_last_kernel_name()
    assert not np.any(np.isfinite(y1.to_numpy((1, N), np.float32)))
    assert not np.any(np.isfinite(y2.to_numpy((1, 64), np.float32)))
    s.close()
    for b in (bx, bw, bw2, y1, y2):
        b.close()
    # a NaN must not linger in the kernel's scratch: the next list is clean
    X[0, 517] = 0.5
    got = gpu_gemv(tc, ctx, X, Wq, fmt, N, y_f32=True, stream=None)
    assert np.all(np.isfinite(got))


# ---------------------------------------------------------------------------------------
# The operations between the GEMVs of a decode step
# ---------------------------------------------------------------------------------------
def _ulps16(a, b):
    """Largest distance between two fp16 arrays in units in the last place (finite values)."""
    ia = a.view(np.int16).astype(np.int32); ib = b.view(np.int16).astype(np.int32)
    ia = np.where(ia < 0, -32768 - ia, ia); ib = np.where(ib < 0, -32768 - ib, ib)
    return int(np.abs(ia - ib).max())


@pytest.mark.parametrize("shape", [(1, 64), (3, 1000), (2, 4096), (1, 8192), (8, 4096)])
def test_norm_forward_matches_oracle(tc, ctx, oracle, shape):
    """fp32 arithmetic in the reference's order; the only freedom is the summation order of the
    double-precision statistics, so results agree to the last fp16 place or one off."""
    N, D = shape
    rng = np.random.default_rng(N * 100 + D)
    X = (rng.standard_normal((N, D)) * 1.5).astype(np.float16)
    gam = (1 + 0.1 * rng.standard_normal(D)).astype(np.float16)
    bet = (0.1 * rng.standard_normal(D)).astype(np.float16)
    bx, bg, bb = dev(ctx, X), dev(ctx, gam), dev(ctx, bet)
    by, bm, br = ctx.buffer(N * D * 2), ctx.buffer(N * 4), ctx.buffer(N * 4)
    tc.rmsnorm_forward(ctx, bx, bg, by, br, N, D, 1e-5)
    assert tc.last_backend() == tc.TC_BACKEND_CUDA
    wy, wr = oracle.rmsnorm_forward(X, gam)
    assert _ulps16(by.to_numpy((N, D), np.float16), wy) <= 1
    assert np.allclose(br.to_numpy((N,), np.float32), wr, rtol=3e-7, atol=0)
    tc.layernorm_forward(ctx, bx, bg, bb, by, bm, br, N, D, 1e-5)
    wy, wm, wr = oracle.layernorm_forward(X, gam, bet)
    assert _ulps16(by.to_numpy((N, D), np.float16), wy) <= 1
    assert np.allclose(bm.to_numpy((N,), np.float32), wm, rtol=1e-6, atol=1e-9)
    assert np.allclose(br.to_numpy((N,), np.float32), wr, rtol=3e-7, atol=0)
    for b in (bx, bg, bb, by, bm, br):
        b.close()


def test_step_ops_match_reference_golden_on_gpu(tc, ctx):
    g = np.load(os.path.join(GOLDEN, "step_ops.npz"))
    gate, up = g["swiglu_gate"].view(np.float16), g["swiglu_up"].view(np.float16)
    bg, bu, bo = dev(ctx, gate), dev(ctx, up), ctx.buffer(gate.size * 2)
    tc.swiglu_forward(ctx, bg, bu, bo, gate.size)
    assert _ulps16(bo.to_numpy((gate.size,), np.float16), g["swiglu_out"].view(np.float16)) <= 1   # expf differs in the last fp32 place
    X = g["rope_X"].view(np.float16)
    B, H, S, D = X.shape
    bx, bc, bs = dev(ctx, X), dev(ctx, g["rope_cos"]), dev(ctx, g["rope_sin"])
    tc.rope_forward(ctx, bx, bc, bs, B, H, S, D)
    assert np.array_equal(bx.to_numpy(X.shape, np.uint16), g["rope_out"])          # no freedom at all: bit for bit
    for key in sorted({k.rsplit("_", 1)[0] for k in g.files if k.startswith("norm_") and k.endswith("_X")}):
        Xn, gam = g[key + "_X"].view(np.float16), g[key + "_gamma"].view(np.float16)
        N, Dn = Xn.shape
        b1, b2, b3, b4 = dev(ctx, Xn), dev(ctx, gam), ctx.buffer(N * Dn * 2), ctx.buffer(N * 4)
        tc.rmsnorm_forward(ctx, b1, b2, b3, b4, N, Dn, 1e-5)
        assert _ulps16(b3.to_numpy((N, Dn), np.float16), g[key + "_Yrms"].view(np.float16)) <= 1, key
        for b in (b1, b2, b3, b4):
            b.close()
    for b in (bg, bu, bo, bx, bc, bs):
        b.close()


def test_swiglu_and_rope_bulk(tc, ctx, oracle):
    rng = np.random.default_rng(808)
    n = 11008 * 3
    gate, up = (rng.standard_normal(n) * 3).astype(np.float16), rng.standard_normal(n).astype(np.float16)
    bg, bu, bo = dev(ctx, gate), dev(ctx, up), ctx.buffer(n * 2)
    tc.swiglu_forward(ctx, bg, bu, bo, n)
    assert _ulps16(bo.to_numpy((n,), np.float16), oracle.swiglu_forward(gate, up)) <= 1
    B, H, S, D = 1, 32, 3, 128
    X = rng.standard_normal((B, H, S, D)).astype(np.float16)
    ang = np.outer(np.arange(S) + 17, 10000.0 ** (-np.arange(D // 2) / (D // 2))).astype(np.float32)
    bx, bc, bs = dev(ctx, X), dev(ctx, np.cos(ang)), dev(ctx, np.sin(ang))
    tc.rope_forward(ctx, bx, bc, bs, B, H, S, D)
    assert np.array_equal(bx.to_numpy(X.shape, np.uint16), oracle.rope_forward(X, np.cos(ang), np.sin(ang)).view(np.uint16))
    for b in (bg, bu, bo, bx, bc, bs):
        b.close()


# ---- attention forward (decode rows and a few short prefill shapes) ---------------------------
def _run_attention(tc, ctx, Q, K, V, causal, window, slopes, want_lse):
    B, Hq, Sq, D = Q.shape
    _, Hkv, Sk, _ = K.shape
    bq, bk, bv = ctx.buffer_from_array(Q), ctx.buffer_from_array(K), ctx.buffer_from_array(V)
    bo = ctx.buffer(Q.nbytes)
    bl = ctx.buffer(B * Hq * Sq * 4) if want_lse else None
    tc.attention_forward(ctx, bq, bk, bv, bo, B, Hq, Sq, Sk, D, LSE=bl, causal=causal, kv_heads=Hkv,
                         window_size=window, alibi_slopes=slopes)
    assert tc.last_backend() == tc.TC_BACKEND_CUDA
    O = bo.to_numpy(Q.shape, np.float16)
    L = bl.to_numpy((B, Hq, Sq), np.float32) if want_lse else None
    for b in (bq, bk, bv, bo) + ((bl,) if bl else ()):
        b.close()
    return O, L


def test_attention_forward_golden_vectors(tc, ctx):
    """Against what the reference's CPU backend produced (tests/golden/attention.npz).  Bar: the
    reference's own for this operation, max abs error below 1e-3 on outputs of order one
    (tests/test_attention_correctness.c:254-262); log-sum-exp within 1e-4."""
    g = np.load(os.path.join(GOLDEN, "attention.npz"))
    for name in sorted(k[:-2] for k in g.files if k.endswith("_Q")):
        Q, K, V = (g[name + s].view(np.float16) for s in ("_Q", "_K", "_V"))
        causal, window = (int(v) for v in g[name + "_cfg"])
        sl = g[name + "_slopes"] if g[name + "_slopes"].size else None
        O, L = _run_attention(tc, ctx, Q, K, V, bool(causal), window, sl, True)
        err = np.abs(O.astype(np.float32) - g[name + "_O"].view(np.float16).astype(np.float32)).max()
        assert err < 1e-3, (name, err)
        assert np.abs(L - g[name + "_LSE"]).max() < 1e-4, name


@pytest.mark.parametrize("B,Hq,Hkv,Sk,D", [(1, 32, 32, 2048, 128), (1, 32, 8, 4096, 128), (4, 8, 8, 1000, 64),
                                            (1, 2, 1, 33, 80)])
def test_attention_decode_row_matches_oracle(tc, ctx, oracle, B, Hq, Hkv, Sk, D):
    """One query row per head over a long K/V cache - the call of a decode step; the key range is
    cut into chunks that are merged by a second kernel."""
    rng = np.random.default_rng(Sk + D)
    Q = rng.standard_normal((B, Hq, 1, D)).astype(np.float16)
    K = rng.standard_normal((B, Hkv, Sk, D)).astype(np.float16)
    V = rng.standard_normal((B, Hkv, Sk, D)).astype(np.float16)
    O, L = _run_attention(tc, ctx, Q, K, V, False, 0, None, True)
    Oo, Lo = oracle.attention_forward(Q, K, V, 0.0, False, 0, None, True)
    assert np.abs(O.astype(np.float32) - Oo.astype(np.float32)).max() < 1e-3
    assert np.abs(L - Lo).max() < 1e-4


def test_attention_argument_checks(tc, ctx):
    b = ctx.buffer(4096)
    with pytest.raises(tc.TensorcoreError) as e:
        tc.attention_forward(ctx, b, b, b, b, 1, 1, 1, 8, 256)           # head_dim above 128
    assert e.value.status == tc.TC_ERR_INVALID_SHAPE
    with pytest.raises(tc.TensorcoreError) as e:
        tc.attention_forward(ctx, b, b, b, b, 1, 3, 1, 8, 64, kv_heads=2)  # kv_heads does not divide heads
    assert e.value.status == tc.TC_ERR_INVALID_ARG
    with pytest.raises(tc.TensorcoreError) as e:
        tc.attention_forward(ctx, b, b, b, b, 1, 1, 1, 8, 64, dtype="bf16")
    assert e.value.status == tc.TC_ERR_UNSUPPORTED_DTYPE
    b.close()


def test_raw_attention_entry_matches_oracle(tc, ctx, oracle):
    """tcx_raw_attention_forward (device pointers, asynchronous on a stream), as the timing harness
    drives it: the output of the last launch against the oracle."""
    from tensorcore_b200 import decode as D
    rng = np.random.default_rng(77)
    B, H, Hkv, Sk, Dh = 1, 16, 4, 1500, 128
    Q = rng.standard_normal((B, H, 1, Dh)).astype(np.float16)
    Ks = [rng.standard_normal((B, Hkv, Sk, Dh)).astype(np.float16) for _ in range(2)]
    Vs = [rng.standard_normal((B, Hkv, Sk, Dh)).astype(np.float16) for _ in range(2)]
    bq, bo = ctx.buffer_from_array(Q), ctx.buffer(Q.nbytes)
    bks, bvs = [ctx.buffer_from_array(k) for k in Ks], [ctx.buffer_from_array(v) for v in Vs]
    D.attention_bench(ctx, bq, bks, bvs, bo, B, H, Hkv, Sk, Dh, 4)       # launches use copies 0, 1, 0, 1
    O = bo.to_numpy(Q.shape, np.float16)
    Oo = oracle.attention_forward(Q, Ks[1], Vs[1], 0.0, False, 0, None, False)
    assert np.abs(O.astype(np.float32) - Oo.astype(np.float32)).max() < 1e-3
    for b in [bq, bo] + bks + bvs:
        b.close()
