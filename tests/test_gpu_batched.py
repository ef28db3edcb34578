"""GPU: the tcgen05 batched-decode GEMV (Q4_0, fp16 activations, 5 <= M) against the oracle.

The kernel dequantises weights to fp16 for the tensor cores, so its bar is the 2e-3 scaled-RMS
bound that applies to fp16 activations (observed 1.8e-4 against an fp64 dequantise-and-dot, 2.8e-4
with fp16 outputs).  Covered: both batch widths (16 and 32 MMA columns), M above 32 (several
launches), row counts that are not a multiple of the 256-row tile, every K-split (cluster) size,
repeated launches on cache-resident weights (the timing that once exposed a stale-stage race),
and that calls outside the kernel's domain go elsewhere.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 2e-3


def case(oracle, N, K, M, seed=0):
    rng = np.random.default_rng(N * 7 + K * 3 + M + seed)
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32).astype(np.float16)
    X = rng.standard_normal((M, K)).astype(np.float16)
    Wq = oracle.quantize_weights(W, 0)
    return X, Wq, oracle.dequant_dot_f64(X.astype(np.float64), Wq, 0, N)


def run(tc, ctx, X, Wq, N, y_f32, reps=1):
    M, K = X.shape
    ydt = np.float32 if y_f32 else np.float16
    outs = []
    with ctx.buffer_from_array(X) as bx, ctx.buffer_from_array(Wq) as bw, \
            ctx.buffer(M * N * np.dtype(ydt).itemsize) as by:
        for _ in range(reps):
            if y_f32:
                tc.gemv_quantized_ex(ctx, bx, bw, by, 0, M, N, K, "f16", "f32", None)
            else:
                ctx.gemv_quantized(bx, bw, by, 0, M, N, K)
            outs.append(by.to_numpy((M, N), ydt).astype(np.float64))
    return outs


@pytest.fixture
def split_env():
    old = os.environ.pop("TC_TC_SPLIT", None)
    yield
    if old is None:
        os.environ.pop("TC_TC_SPLIT", None)
    else:
        os.environ["TC_TC_SPLIT"] = old


@pytest.mark.parametrize("shape", [(256, 256, 16), (256, 512, 8), (512, 1024, 32), (300, 768, 9),
                                   (512, 1024, 5), (4096, 4096, 7),
                                   (130, 256, 32), (1000, 2048, 12), (4096, 4096, 16),
                                   (4096, 4096, 40), (11008, 4096, 24), (2048, 11008, 32)])
@pytest.mark.parametrize("y_f32", [True, False])
def test_batched_matches_fp64_dequant_dot(tc, ctx, oracle, split_env, shape, y_f32):
    N, K, M = shape
    X, Wq, want = case(oracle, N, K, M)
    got = run(tc, ctx, X, Wq, N, y_f32)[0]
    assert "tcgen05" in tc.cuda_last_kernel_name()
    assert oracle.scaled_rms(got, want) <= TOL
    assert tc.take_device_error(ctx) == 0


@pytest.mark.parametrize("split", [1, 2, 3, 4, 5, 6, 7, 8])
def test_every_k_split_size(tc, ctx, oracle, split_env, split):
    N, K, M = 1024, 4096, 32
    X, Wq, want = case(oracle, N, K, M)
    os.environ["TC_TC_SPLIT"] = str(split)
    got = run(tc, ctx, X, Wq, N, True)[0]
    assert oracle.scaled_rms(got, want) <= TOL
    # the split-K reduction is a fixed-order sum: results do not depend on timing
    again = run(tc, ctx, X, Wq, N, True)[0]
    assert np.array_equal(got, again)


@pytest.mark.parametrize("shape", [(2048, 4096, 32, 1), (1024, 8192, 32, 2), (11008, 4096, 24, 1)])
def test_repeated_launches_on_resident_weights(tc, ctx, oracle, split_env, shape):
    N, K, M, split = shape
    X, Wq, want = case(oracle, N, K, M, seed=5)
    os.environ["TC_TC_SPLIT"] = str(split)
    outs = run(tc, ctx, X, Wq, N, True, reps=40)
    errs = [oracle.scaled_rms(o, want) for o in outs]
    assert max(errs) <= TOL, errs
    assert all(np.array_equal(outs[0], o) for o in outs[1:])
    assert tc.take_device_error(ctx) == 0


def test_batched_agrees_with_the_streaming_kernel(tc, ctx, oracle, split_env):
    N, K, M = 4096, 4096, 16
    X, Wq, want = case(oracle, N, K, M)
    try:
        tc.set_gemv_variant("simt")
        ref = run(tc, ctx, X, Wq, N, True)[0]
        assert any(k in tc.cuda_last_kernel_name() for k in ("box", "stream"))
        tc.set_gemv_variant("tc")
        got = run(tc, ctx, X, Wq, N, True)[0]
        assert "tcgen05" in tc.cuda_last_kernel_name()
    finally:
        tc.set_gemv_variant("auto")
    assert oracle.scaled_rms(got, ref) <= TOL
    assert oracle.scaled_rms(ref, want) <= 1e-4


def test_domain(tc, ctx, oracle, split_env):
    """fp32 activations, Q8_0 (up to 12 rows), small M and K % 256 != 0 stay off the tensor cores; the fused RMSNorm form takes it
    behind a normalisation pass."""
    rng = np.random.default_rng(3)
    N, K, M = 256, 512, 16
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    X16 = rng.standard_normal((M, K)).astype(np.float16)
    names = {}
    with ctx.buffer_from_array(oracle.quantize_weights(W, 0)) as w4, \
            ctx.buffer_from_array(oracle.quantize_weights(W, 1)) as w8, \
            ctx.buffer_from_array(X16) as x16, ctx.buffer_from_array(X16.astype(np.float32)) as x32, \
            ctx.buffer_from_array(np.ones(K, np.float16)) as g16, ctx.buffer(M * N * 4) as y:
        tc.gemv_quantized_ex(ctx, x32, w4, y, 0, M, N, K, "f32", "f32", None)
        names["f32"] = tc.cuda_last_kernel_name()
        ctx.fused_rmsnorm_gemv_quantized(x16, g16, w4, y, 0, M, N, K, 1e-5)
        names["fused"] = tc.cuda_last_kernel_name()
        ctx.gemv_quantized(x16, w8, y, 1, 12, N, K)
        names["q8"] = tc.cuda_last_kernel_name()
        ctx.gemv_quantized(x16, w8, y, 1, M, N, K)      # 13 rows or more: dequantised once, then the GEMM
        assert tc.cuda_last_kernel_name() == "q8_0_dequant_gemm_tcgen05_sm100"
        ctx.gemv_quantized(x16, w4, y, 0, 4, N, K)
        names["m4"] = tc.cuda_last_kernel_name()
        ctx.gemv_quantized(x16, w4, y, 0, M, N, K)
        names["m16"] = tc.cuda_last_kernel_name()
    assert "tcgen05" in names.pop("m16")
    assert "tcgen05" in names.pop("fused")
    assert all("tcgen05" not in n for n in names.values()), names


@pytest.mark.parametrize("M,N,K", [(8, 1024, 2048), (16, 4096, 4096), (32, 512, 8192), (40, 300, 1024)])
def test_fused_rmsnorm_batched_matches_oracle(tc, ctx, oracle, M, N, K):
    """Fused RMSNorm + Q4_0 GEMV with fp16 activations and M >= 5: rows normalised to fp16 in the
    stream's scratch, then the tensor-core kernel.  Bar: the 2e-3 of fp16 activations."""
    rng = np.random.default_rng(M * 7 + N)
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    X = (rng.standard_normal((M, K)) * 1.5).astype(np.float16)
    gam = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    Wq = oracle.quantize_weights(W, 0)
    want = oracle.fused_rmsnorm_gemv_quantized(X, gam, Wq, 0, N)
    with ctx.buffer_from_array(Wq) as w4, ctx.buffer_from_array(X) as bx, ctx.buffer_from_array(gam) as bg, \
            ctx.buffer(M * N * 2) as by:
        ctx.fused_rmsnorm_gemv_quantized(bx, bg, w4, by, 0, M, N, K, 1e-5)
        assert "tcgen05" in tc.cuda_last_kernel_name()
        got = by.to_numpy((M, N), np.float16)
        assert oracle.scaled_rms(got, want) <= TOL
        # the same recorded on a stream (twice: the second submission may replay a captured graph)
        s = ctx.stream()
        for _ in range(3):
            ctx.gemv_quantized_async(bx, w4, by, 0, M, N, K, s)
            tc.fused_rmsnorm_gemv_quantized_ex(ctx, bx, bg, w4, by, 0, M, N, K, 1e-5, "f16", "f16", s)
            s.sync()
            assert oracle.scaled_rms(by.to_numpy((M, N), np.float16), want) <= TOL
        s.close()


@pytest.mark.parametrize("fmt,shape", [(0, (1024, 512, 128)), (0, (520, 1056, 200)), (0, (4096, 4096, 512)),
                                       (1, (1024, 512, 128)), (1, (520, 1056, 200)), (1, (4096, 4096, 512)),
                                       (1, (1024, 2048, 13)), (1, (4096, 4096, 32))])
def test_prefill_sized_calls_dequantise_once_and_use_the_gemm(tc, ctx, oracle, fmt, shape):
    """96 activation rows or more (Q4_0; Q8_0, which has no batched kernel, from 13) with fp16 results: the weights are dequantised once to fp16 in the
    stream's scratch and multiplied on the tensor cores (Q4_0 and Q8_0, plain and fused RMSNorm);
    same bar as the batched kernel, against the fp64 dequantise-and-dot."""
    N, K, M = shape
    rng = np.random.default_rng(N + K * 3 + M * 7 + fmt)
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32).astype(np.float16)
    X = rng.standard_normal((M, K)).astype(np.float16)
    gam = (1 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    Wq = oracle.quantize_weights(W, fmt)
    want = oracle.dequant_dot_f64(X.astype(np.float64), Wq, fmt, N)
    with ctx.buffer_from_array(X) as bx, ctx.buffer_from_array(Wq) as bw, ctx.buffer_from_array(gam) as bg, \
            ctx.buffer(M * N * 2) as by:
        ctx.gemv_quantized(bx, bw, by, fmt, M, N, K)
        name = tc.cuda_last_kernel_name()
        got = by.to_numpy((M, N), np.float16).astype(np.float64)
        assert name == ("q4_0" if fmt == 0 else "q8_0") + "_dequant_gemm_tcgen05_sm100"
        assert oracle.scaled_rms(got, want) <= TOL
        # fused RMSNorm form, on a few rows against the oracle's fp32 chain
        ctx.fused_rmsnorm_gemv_quantized(bx, bg, bw, by, fmt, M, N, K, 1e-5)
        assert tc.cuda_last_kernel_name() == name
        gotf = by.to_numpy((M, N), np.float16)
        rows = [0, M // 2, M - 1]
        wantf = oracle.fused_rmsnorm_gemv_quantized_f32(X[rows].astype(np.float32), gam.astype(np.float32), Wq, fmt, N)
        assert oracle.scaled_rms(gotf[rows], wantf) <= TOL
        # fp32 results keep the kernels that stream the blocks
        with ctx.buffer(M * N * 4) as by32:
            tc.gemv_quantized_ex(ctx, bx, bw, by32, fmt, M, N, K, "f16", "f32", None)
            assert "dequant_gemm" not in tc.cuda_last_kernel_name()
    assert tc.take_device_error(ctx) == 0
