"""GPU: the persistent decode launch (one cooperative kernel for a whole recorded list of Q4_0,
M = 1 GEMVs).  Lists that qualify are routed there by tc_stream_sync; the results must be those
of the per-operation kernels / the oracle, across dependent and independent operations, mixed K,
fp16 and fp32 activations and fused norms, and across repeated submissions (the grid-barrier
generation persists between launches)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_mixed_list_matches_oracle(tc, ctx, oracle):
    rng = np.random.default_rng(314)
    d, f = 1024, 2816
    mk = lambda n, k: oracle.quantize_weights((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float16), 0)
    Wq, Wk, Wo, Wg, Wd = mk(d, d), mk(256, d), mk(d, d), mk(f, d), mk(d, f)
    x16 = rng.standard_normal((1, d)).astype(np.float16)
    gam16 = (1 + 0.1 * rng.standard_normal(d)).astype(np.float16)
    gam32 = gam16.astype(np.float32)
    # oracle: q = fused(x) ; k = fused(x) ; o = gemv(q) [fp32 out] ; g = fused_f32(o) ; y = gemv(g)
    q = oracle.fused_rmsnorm_gemv_quantized(x16, gam16, Wq, 0, d)
    k = oracle.fused_rmsnorm_gemv_quantized(x16, gam16, Wk, 0, 256)
    o = oracle.gemv_quantized_f32(q.astype(np.float32), Wo, 0, d)
    g = oracle.fused_rmsnorm_gemv_quantized_f32(o, gam32, Wg, 0, f).astype(np.float16)
    y = oracle.gemv_quantized(g, Wd, 0, d)

    B = ctx.buffer_from_array
    bx, bg16, bg32 = B(x16), B(gam16), B(gam32)
    bWq, bWk, bWo, bWg, bWd = B(Wq), B(Wk), B(Wo), B(Wg), B(Wd)
    bq, bk, bo, bgt, by = ctx.buffer(d * 2), ctx.buffer(256 * 2), ctx.buffer(d * 4), ctx.buffer(f * 2), ctx.buffer(d * 2)
    s = ctx.stream()
    for rep in range(4):
        tc.fused_rmsnorm_gemv_quantized_ex(ctx, bx, bg16, bWq, bq, 0, 1, d, d, 1e-5, "f16", "f16", s)
        tc.fused_rmsnorm_gemv_quantized_ex(ctx, bx, bg16, bWk, bk, 0, 1, 256, d, 1e-5, "f16", "f16", s)
        tc.gemv_quantized_ex(ctx, bq, bWo, bo, 0, 1, d, d, "f16", "f32", s)
        tc.fused_rmsnorm_gemv_quantized_ex(ctx, bo, bg32, bWg, bgt, 0, 1, f, d, 1e-5, "f32", "f16", s)
        ctx.gemv_quantized_async(bgt, bWd, by, 0, 1, d, f, s)
        s.sync()
        assert "persistent" in tc.cuda_last_kernel_name()
        assert oracle.scaled_rms(bq.to_numpy((1, d), np.float16), q) <= 3e-4
        assert oracle.scaled_rms(bk.to_numpy((1, 256), np.float16), k) <= 3e-4
        assert oracle.scaled_rms(bo.to_numpy((1, d), np.float32), o) <= 2e-3
        assert oracle.scaled_rms(by.to_numpy((1, d), np.float16), y) <= 2e-3
    assert tc.take_device_error(ctx) == 0
    s.close()


def test_lists_that_do_not_qualify_use_per_operation_kernels(tc, ctx, oracle):
    rng = np.random.default_rng(5)
    N, K = 200, 512
    W8 = oracle.quantize_weights((rng.standard_normal((N, K)) * 0.02).astype(np.float16), 1)
    W4 = oracle.quantize_weights((rng.standard_normal((N, K)) * 0.02).astype(np.float16), 0)
    X = rng.standard_normal((2, K)).astype(np.float16)
    bx, b8, b4 = ctx.buffer_from_array(X), ctx.buffer_from_array(W8), ctx.buffer_from_array(W4)
    y1, y2 = ctx.buffer(2 * N * 2), ctx.buffer(2 * N * 2)
    s = ctx.stream()
    for rep in range(3):
        ctx.gemv_quantized_async(bx, b8, y1, 1, 2, N, K, s)     # Q8_0, M = 2
        ctx.gemv_quantized_async(bx, b4, y2, 0, 2, N, K, s)     # M = 2
        s.sync()
        assert "persistent" not in tc.cuda_last_kernel_name()
        assert oracle.scaled_rms(y1.to_numpy((2, N), np.float16), oracle.gemv_quantized(X, W8, 1, N)) <= 3e-4
        assert oracle.scaled_rms(y2.to_numpy((2, N), np.float16), oracle.gemv_quantized(X, W4, 0, N)) <= 3e-4
    s.close()



def test_long_list_and_wide_rows(tc, ctx, oracle):
    """More than 512 operations (the table no longer fits the kernel's shared-memory copy and is
    read from global memory) and a K of 28672 (the 70B down-projection width: the largest staged
    activation row), with row counts that leave partly filled 32-row boxes."""
    rng = np.random.default_rng(77)
    K1, N1 = 256, 70
    W1 = oracle.quantize_weights((rng.standard_normal((N1, K1)) / np.sqrt(K1)).astype(np.float16), 0)
    x1 = rng.standard_normal((1, K1)).astype(np.float16)
    want1 = oracle.gemv_quantized(x1, W1, 0, N1)
    bW1, bx1 = ctx.buffer_from_array(W1), ctx.buffer_from_array(x1)
    outs = [ctx.buffer(N1 * 2) for _ in range(8)]
    K2, N2 = 28672, 333
    W2 = oracle.quantize_weights((rng.standard_normal((N2, K2)) / np.sqrt(K2)).astype(np.float16), 0)
    x2 = rng.standard_normal((1, K2)).astype(np.float32)
    g2 = (1 + 0.1 * rng.standard_normal(K2)).astype(np.float32)
    want2 = oracle.fused_rmsnorm_gemv_quantized_f32(x2, g2, W2, 0, N2, 1e-5)
    bW2, bx2, by2 = ctx.buffer_from_array(W2), ctx.buffer_from_array(x2), ctx.buffer(N2 * 4)
    bg2 = ctx.buffer_from_array(g2)
    s = ctx.stream()
    for rep in range(2):
        for i in range(600):
            ctx.gemv_quantized_async(bx1, bW1, outs[i % 8], 0, 1, N1, K1, s)
        tc.fused_rmsnorm_gemv_quantized_ex(ctx, bx2, bg2, bW2, by2, 0, 1, N2, K2, 1e-5, "f32", "f32", s)
        s.sync()
        assert "persistent" in tc.cuda_last_kernel_name()
        for o in outs:
            assert oracle.scaled_rms(o.to_numpy((1, N1), np.float16), want1) <= 3e-4
        assert oracle.scaled_rms(by2.to_numpy((1, N2), np.float32), want2) <= 1e-4
    assert tc.take_device_error(ctx) == 0
    s.close()


@pytest.mark.parametrize("K", [256, 512, 768, 1280, 1536, 2816])
def test_narrow_and_ragged_bands(tc, ctx, oracle, K):
    """K ranges as tensor parallelism cuts them: fewer than four groups (one narrow band), and a
    last band of one, two or three groups after full ones; a chain of two operations so that the
    second takes its input from the first one's accumulators."""
    rng = np.random.default_rng(K)
    N = 2 * K                                   # the second operation reads all of the first one's rows
    W1 = oracle.quantize_weights((rng.standard_normal((N, K)) * 0.05).astype(np.float16), 0)
    W2 = oracle.quantize_weights((rng.standard_normal((300, N)) * 0.05).astype(np.float16), 0) if N % 256 == 0 else None
    X = rng.standard_normal((1, K)).astype(np.float16)
    bx, bw1 = ctx.buffer_from_array(X), ctx.buffer_from_array(W1)
    y1 = ctx.buffer(N * 2)
    s = ctx.stream()
    bw2 = ctx.buffer_from_array(W2)
    y2 = ctx.buffer(300 * 2)
    for rep in range(2):
        ctx.gemv_quantized_async(bx, bw1, y1, 0, 1, N, K, s)
        ctx.gemv_quantized_async(y1, bw2, y2, 0, 1, 300, N, s)
        s.sync()
        assert "persistent" in tc.cuda_last_kernel_name()
        r1 = oracle.gemv_quantized(X, W1, 0, N)
        assert oracle.scaled_rms(y1.to_numpy((1, N), np.float16), r1) <= 3e-4
        r2 = oracle.gemv_quantized(r1, W2, 0, 300)
        assert oracle.scaled_rms(y2.to_numpy((1, 300), np.float16), r2) <= 2e-3
    assert tc.take_device_error(ctx) == 0
    s.close()
