"""GPU: tc_gemm (fp16 storage, fp32 accumulation) against the oracle's restatement of the
reference's CPU loop (lib/ops/gemm_cpu.cpp:544-568), through the C ABI.

The reference adds the K products in k order in fp32; the tensor-core kernel adds them in the
MMA's order, the few-row kernel with fused multiply-adds.  Both keep fp32 sums, so results differ
from the oracle by fp32 rounding of the sum and, after the fp16 store, by an occasional last-place
flip: the bar is a scaled RMS of 3e-4 (one flipped element in a thousand is 1.5e-5)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 3e-4


def _run(tc, ctx, A, B, tb, alpha=1.0, beta=0.0, C0=None, lda=0, ldb=0, ldc=0, M=None, N=None, K=None):
    M = M if M is not None else A.shape[0]
    K = K if K is not None else A.shape[1]
    N = N if N is not None else (B.shape[0] if tb else B.shape[1])
    a, b = ctx.buffer_from_array(A), ctx.buffer_from_array(B)
    c_host = np.zeros((M, ldc or N), dtype=np.float16) if C0 is None else C0.copy()
    c = ctx.buffer_from_array(c_host)
    tc.gemm(ctx, a, b, c, M, N, K, transpose_b=tb, alpha=alpha, beta=beta, lda=lda, ldb=ldb, ldc=ldc)
    out = c.to_numpy(c_host.shape, np.float16)
    return out, tc.cuda_last_kernel_name()


@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 384, 512), (100, 72, 136), (513, 1000, 1024),
                                   (32, 4096, 4096), (130, 264, 8)])
@pytest.mark.parametrize("tb", [False, True])
def test_tensor_core_gemm_matches_oracle(tc, ctx, oracle, shape, tb):
    M, N, K = shape
    rng = np.random.default_rng(M * 7 + N * 3 + K + int(tb))
    A = rng.standard_normal((M, K)).astype(np.float16)
    B = (rng.standard_normal((N, K) if tb else (K, N)) * 0.05).astype(np.float16)
    got, kernel = _run(tc, ctx, A, B, tb)
    assert kernel == "gemm_f16_tcgen05_sm100"
    want = oracle.gemm_f16(A, B, tb)
    assert np.isfinite(got.astype(np.float32)).all()
    assert oracle.scaled_rms(got, want) <= TOL
    assert tc.take_device_error(ctx) == 0


def test_alpha_beta_and_leading_dimensions(tc, ctx, oracle):
    rng = np.random.default_rng(5)
    M, N, K = 200, 136, 320
    A = rng.standard_normal((M, K)).astype(np.float16)
    B = (rng.standard_normal((K, N)) * 0.05).astype(np.float16)
    C0 = rng.standard_normal((M, N)).astype(np.float16)
    got, kernel = _run(tc, ctx, A, B, False, alpha=0.5, beta=1.5, C0=C0)
    assert kernel == "gemm_f16_tcgen05_sm100"
    assert oracle.scaled_rms(got, oracle.gemm_f16(A, B, False, 0.5, 1.5, C0)) <= TOL
    # sub-matrices of wider arrays: lda, ldb, ldc larger than the extents; the rest of C stays untouched
    Aw = rng.standard_normal((M, K + 24)).astype(np.float16)
    Bw = (rng.standard_normal((K, N + 40)) * 0.05).astype(np.float16)
    Cw = rng.standard_normal((M, N + 8)).astype(np.float16)
    got, _ = _run(tc, ctx, Aw, Bw, False, C0=Cw, lda=K + 24, ldb=N + 40, ldc=N + 8, M=M, N=N, K=K)
    want = oracle.gemm_f16(Aw[:, :K], Bw[:, :N], False)
    assert oracle.scaled_rms(got[:, :N], want) <= TOL
    assert np.array_equal(got[:, N:].view(np.uint16), Cw[:, N:].view(np.uint16))


def test_few_rows_and_shapes_outside_the_tiled_copies(tc, ctx, oracle):
    """Up to four rows (a decode step) take the row kernel; so does a shape whose K is not a multiple
    of 8, which the tiled copies cannot describe."""
    rng = np.random.default_rng(6)
    for (M, N, K) in ((1, 1000, 4096), (4, 512, 1024), (40, 96, 100)):
        A = rng.standard_normal((M, K)).astype(np.float16)
        B = (rng.standard_normal((K, N)) * 0.05).astype(np.float16)
        got, kernel = _run(tc, ctx, A, B, False)
        assert kernel == "gemm_f16_rows_sm100", (M, N, K)
        assert oracle.scaled_rms(got, oracle.gemm_f16(A, B, False)) <= TOL


def test_argument_checks(tc, ctx):
    a = ctx.buffer(64 * 64 * 2)
    with pytest.raises(tc.TensorcoreError) as e:
        tc.gemm(ctx, a, a, a, 64, 64, 64, dtype="f32", accum="f32")
    assert e.value.status == tc.TC_ERR_UNSUPPORTED_DTYPE
    with pytest.raises(tc.TensorcoreError) as e:
        tc.gemm(ctx, a, a, a, 64, 64, 64, transpose_a=True, lda=60)      # a leading dimension the tiled copies cannot take
    assert e.value.status in (tc.TC_ERR_UNSUPPORTED_FAMILY, tc.TC_ERR_INVALID_ARG)
    with pytest.raises(tc.TensorcoreError) as e:
        tc.gemm(ctx, a, a, a, 64, 64, 64, lda=32)
    assert e.value.status == tc.TC_ERR_INVALID_ARG
    with pytest.raises(tc.TensorcoreError) as e:
        tc.gemm(ctx, a, a, a, 128, 64, 64)          # A would need 128 x 64 halves
    assert e.value.status != tc.TC_OK


@pytest.mark.parametrize("shape", [(128, 256, 64), (200, 264, 520), (3, 512, 1024), (512, 1024, 2048)])
@pytest.mark.parametrize("tb", [False, True])
def test_bfloat16_gemm_matches_oracle(tc, ctx, oracle, shape, tb):
    """bfloat16 operands and result, fp32 accumulation: always the tensor-core kernel.  A bfloat16 result
    has 8 significant bits: one last-place flip is 3.9e-3 of that element, so the bar is 2e-3 scaled RMS."""
    M, N, K = shape
    rng = np.random.default_rng(M + N * 3 + K * 5 + int(tb))
    A = oracle.to_bf16_bits(rng.standard_normal((M, K)))
    B = oracle.to_bf16_bits(rng.standard_normal((N, K) if tb else (K, N)) * 0.05)
    C0 = oracle.to_bf16_bits(rng.standard_normal((M, N)))
    for alpha, beta in ((1.0, 0.0), (0.75, 0.5)):
        a, b, c = ctx.buffer_from_array(A), ctx.buffer_from_array(B), ctx.buffer_from_array(C0)
        tc.gemm(ctx, a, b, c, M, N, K, dtype="bf16", transpose_b=tb, alpha=alpha, beta=beta)
        assert tc.cuda_last_kernel_name() == "gemm_f16_tcgen05_sm100"
        got = oracle.from_bf16_bits(c.to_numpy((M, N), np.uint16))
        want = oracle.from_bf16_bits(oracle.gemm_bf16(A, B, tb, alpha, beta, C0))
        assert np.isfinite(got).all()
        assert oracle.scaled_rms(got, want) <= 2e-3, (alpha, beta)
        for x in (a, b, c):
            x.close()
    assert tc.take_device_error(ctx) == 0


@pytest.mark.parametrize("shape", [(128, 128, 64), (200, 264, 520), (8, 512, 1024)])
@pytest.mark.parametrize("tb", [False, True])
def test_transposed_a_matches_oracle(tc, ctx, oracle, shape, tb):
    """A given as [K][M] (transpose_a), with B either way, and through tc_gemm_async."""
    M, N, K = shape
    rng = np.random.default_rng(M * 11 + N + K + int(tb))
    At = rng.standard_normal((K, M)).astype(np.float16)
    B = (rng.standard_normal((N, K) if tb else (K, N)) * 0.05).astype(np.float16)
    a, b = ctx.buffer_from_array(At), ctx.buffer_from_array(B)
    c = ctx.buffer(M * N * 2)
    tc.gemm(ctx, a, b, c, M, N, K, transpose_a=True, transpose_b=tb)
    assert tc.cuda_last_kernel_name() == "gemm_f16_tcgen05_sm100"
    got = c.to_numpy((M, N), np.float16)
    want = oracle.gemm_f16(At, B, tb, transpose_a=True)
    assert oracle.scaled_rms(got, want) <= TOL
    # the recorded form runs at once and gives the same bytes
    import ctypes
    st = ctx.stream()
    d = tc.TCGemmDesc(M, N, K, 0, 0, 0, 2, True, bool(tb), 1.0, 0.0, 0, 0, 0)
    c2 = ctx.buffer(M * N * 2)
    L = tc.lib()
    L.tc_gemm_async.argtypes = [ctypes.c_void_p] * 6
    assert L.tc_gemm_async(ctx.handle, ctypes.byref(d), a.handle, b.handle, c2.handle, st.handle) == 0
    assert L.tc_gemm_async(ctx.handle, ctypes.byref(d), a.handle, b.handle, c2.handle, None) == tc.TC_ERR_INVALID_ARG
    st.sync()
    assert np.array_equal(c2.to_numpy((M, N), np.uint16), got.view(np.uint16))
    assert tc.take_device_error(ctx) == 0


def test_batched_gemm_matches_oracle_per_product(tc, ctx, oracle):
    """tc_gemm_batched: products of one shape at element strides, B transposed in half of the cases."""
    rng = np.random.default_rng(77)
    M, N, K, batch = 136, 264, 320, 3
    sa, sb, sc = M * K + 64, K * N + 128, M * N + 8
    A = rng.standard_normal(batch * sa).astype(np.float16)
    C0 = np.zeros(batch * sc, dtype=np.float16)
    for tb in (False, True):
        Bf = (rng.standard_normal(batch * sb) * 0.05).astype(np.float16)
        a, b, c = ctx.buffer_from_array(A), ctx.buffer_from_array(Bf), ctx.buffer_from_array(C0)
        tc.gemm_batched(ctx, a, b, c, M, N, K, batch, sa, sb, sc, transpose_b=tb)
        assert tc.cuda_last_kernel_name() == "gemm_f16_tcgen05_sm100"
        got = c.to_numpy((batch * sc,), np.float16)
        for i in range(batch):
            Ai = A[i * sa:i * sa + M * K].reshape(M, K)
            Bi = Bf[i * sb:i * sb + K * N].reshape((N, K) if tb else (K, N))
            want = oracle.gemm_f16(Ai, Bi, tb)
            assert oracle.scaled_rms(got[i * sc:i * sc + M * N].reshape(M, N), want) <= TOL, (tb, i)
            assert not got[i * sc + M * N:(i + 1) * sc].any()          # the gap between results stays untouched
        for x in (a, b, c):
            x.close()
    a = ctx.buffer(1 << 20)
    with pytest.raises(tc.TensorcoreError) as e:
        tc.gemm_batched(ctx, a, a, a, 64, 64, 64, 0, 4096, 4096, 4096)
    assert e.value.status == tc.TC_ERR_INVALID_ARG
    with pytest.raises(tc.TensorcoreError) as e:
        tc.gemm_batched(ctx, a, a, a, 64, 64, 64, 2, 100, 4096, 4096)       # stride shorter than a matrix
    assert e.value.status == tc.TC_ERR_INVALID_SHAPE


def test_gemm_against_reference_golden_vectors(tc, ctx, oracle):
    """The reference's own CPU results (tests/golden/gemm.npz): fp16 within the 3e-4 bar (its narrowing
    differs from IEEE on ties and on a carry out of the mantissa, a handful of elements), bf16 within 2e-3."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gemm.npz"))
    for name in sorted({k.rsplit("_A", 1)[0] for k in g.files if k.endswith("_A")}):
        A, B, C0, dt = g[name + "_A"], g[name + "_B"], g[name + "_C0"], int(g[name + "_dtype"][0])
        M, K = A.shape
        N = B.shape[1]
        widen = (lambda a: a.view(np.float16).astype(np.float32)) if dt == 0 else oracle.from_bf16_bits
        for ta in (0, 1):
            for tb in (0, 1):
                for tag, alpha, beta in (("plain", 1.0, 0.0), ("ab", 0.5, 1.5)):
                    Ax = np.ascontiguousarray(A.T) if ta else A
                    Bx = np.ascontiguousarray(B.T) if tb else B
                    a, b, c = ctx.buffer_from_array(Ax), ctx.buffer_from_array(Bx), ctx.buffer_from_array(C0)
                    try:
                        tc.gemm(ctx, a, b, c, M, N, K, dtype="f16" if dt == 0 else "bf16", transpose_a=bool(ta),
                                transpose_b=bool(tb), alpha=alpha, beta=beta)
                    except tc.TensorcoreError as e:
                        # operands the tiled copies cannot describe (a leading dimension that is not a multiple of 8)
                        assert e.status == tc.TC_ERR_UNSUPPORTED_FAMILY and (ta or tb or dt == 1), (name, ta, tb)
                        continue
                    got = widen(c.to_numpy((M, N), np.uint16))
                    want = widen(g[f"{name}_Y_{ta}{tb}_{tag}"])
                    bar = 3e-4 if dt == 0 else 2e-3
                    # the reference's fp16 narrowing can lose a carry (a factor of two on that element): compare robustly
                    close = np.abs(got - want) <= 0.02 * np.maximum(1.0, np.abs(want))
                    assert close.mean() >= 0.995, (name, ta, tb, tag)
                    assert oracle.scaled_rms(got[close], want[close]) <= bar, (name, ta, tb, tag)
                    for x in (a, b, c):
                        x.close()
