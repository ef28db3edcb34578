"""CPU: pins the oracle (oracle/tc_oracle.c) against the reference's own known answers, the
committed golden vectors produced by the reference's CPU backend, and - where it was compiled
from a reference checkout - that backend itself."""
import os

import numpy as np
import pytest

from conftest import GOLDEN

FMTS = {"q4_0": 0, "q8_0": 1}


def test_fp16_widening_matches_ieee(oracle):
    allh = np.arange(65536, dtype=np.uint16)
    got = oracle.f16_bits_to_f32(allh)
    want = allh.view(np.float16).astype(np.float32)
    ok = ~np.isnan(want)
    assert np.array_equal(got.view(np.uint32)[ok], want.view(np.uint32)[ok])
    assert np.all(np.isnan(got[~ok]))


def test_fp16_narrowing_is_round_to_nearest_even(oracle):
    rng = np.random.default_rng(3)
    parts = [rng.standard_normal(100000).astype(np.float32) * s
             for s in (1e-8, 1e-6, 1e-4, 1.0, 100.0, 70000.0)]
    edge = np.array([np.inf, -np.inf, 0.0, -0.0, 65504, 65519.99, 65520, 2.0**-25,
                     2.0**-25 * 1.0000001, 2.0**-24 * 1.5, 2.0**-24 * 2.5, 2.0**-14,
                     2.0**-14 * (1 - 2.0**-11)], dtype=np.float32)
    x = np.concatenate(parts + [edge])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(oracle.f32_to_f16_bits(x), want)
    # NaN keeps its sign and becomes the quiet pattern (lib/core/cpu_float.h:52-55)
    nan = np.array([np.nan, -np.nan], dtype=np.float32)
    assert list(oracle.f32_to_f16_bits(nan) & 0x7FFF) == [0x7E00, 0x7E00]


def test_quantized_size(oracle):
    # tests/test_quantized.c:152-156,244-248,359-363 and tests/test_portable_cpu.c:570-571
    assert oracle.quantized_size(0, 128, 256) == 128 * 8 * 18
    assert oracle.quantized_size(1, 129, 256) == 129 * 8 * 34
    assert oracle.quantized_size(0, 3, 32) == 3 * 18
    assert oracle.quantized_size(7, 4, 32) == 0
    assert oracle.quantized_size(0, 4, 33) == 0
    assert oracle.quantized_size(0, 0, 32) == 0
    assert oracle.quantized_size(0, 4096, 4096) == 9437184
    assert oracle.quantized_size(1, 11008, 4096) == 47906816


def test_gguf_known_answer_gemv(oracle):
    # tests/test_gguf.c:119-122,267-279: scale 0x3800 (0.5), sixteen 0xAB bytes, x = 32 x 1.0
    blk = np.array([0x00, 0x38] + [0xAB] * 16, dtype=np.uint8)
    x = np.full((1, 32), 0x3C00, dtype=np.uint16).view(np.float16)
    y = oracle.gemv_quantized(x, blk, 0, 1)
    assert y.view(np.uint16)[0, 0] == 0x5100


def test_portable_cpu_closed_form_case(oracle):
    # tests/test_portable_cpu.c:564-602: M=1 N=3 K=32 Q4_0, x_i = 0.01(i-15), w_i = 0.02((i%17)-8)
    K, N = 32, 3
    x = oracle.f32_to_f16_bits((0.01 * (np.arange(K, dtype=np.float32) - 15)).astype(np.float32))
    w = oracle.f32_to_f16_bits(
        (0.02 * ((np.arange(N * K) % 17).astype(np.float32) - 8)).astype(np.float32))
    wq = oracle.quantize_weights(w.reshape(N, K), 0)
    assert wq.size == N * 18
    y = oracle.gemv_quantized(x.reshape(1, K), wq, 0, N).astype(np.float32)[0]
    xf = oracle.f16_bits_to_f32(x)
    for n in range(N):
        blk = wq[n * 18:(n + 1) * 18]
        d = oracle.f16_bits_to_f32(blk[:2].view(np.uint16))[0]
        lo = (blk[2:] & 0x0F).astype(np.float32) - 8
        hi = (blk[2:] >> 4).astype(np.float32) - 8
        want = float(np.sum(xf[:16] * d * lo) + np.sum(xf[16:] * d * hi))
        assert abs(y[n] - np.float32(np.float16(want))) <= 1e-3


@pytest.mark.parametrize("tag", ["q4_0", "q8_0"])
def test_golden_quantized_path(oracle, tag):
    g = np.load(os.path.join(GOLDEN, "quantized_path.npz"))
    fmt = FMTS[tag]
    keys = sorted({k.rsplit("_", 1)[0] for k in g.files if k.startswith(tag)})
    assert len(keys) == 5
    for key in keys:
        N = int(key.split("_N")[1].split("_")[0])
        W = g[key + "_W"]
        X = g[key + "_X"].view(np.float16)
        gam = g[key + "_gamma"].view(np.float16)
        wq = oracle.quantize_weights(W, fmt)
        assert np.array_equal(wq, g[key + "_Wq"]), key
        assert np.array_equal(oracle.gemv_quantized(X, wq, fmt, N).view(np.uint16), g[key + "_Y"])
        yf = oracle.fused_rmsnorm_gemv_quantized(X, gam, wq, fmt, N, 1e-5)
        assert np.array_equal(yf.view(np.uint16), g[key + "_Yfused"]), key


def test_golden_zero_block_and_clamp(oracle):
    g = np.load(os.path.join(GOLDEN, "quantized_path.npz"))
    wq = g["q4_0_N130_K256_M1_Wq"].reshape(130, 8, 18)
    assert wq[0, 0, 0] == 0 and wq[0, 0, 1] == 0 and np.all(wq[0, 0, 2:] == 0x88)
    assert np.all(wq[1, 1, 2:] == 0x00)          # -amax -> code 0 in both nibbles
    w8 = g["q8_0_N130_K256_M1_Wq"].reshape(130, 8, 34)
    assert np.all(w8[0, 0] == 0)
    assert np.all(w8[1, 1, 2:].view(np.int8) == -127)


def test_golden_dense_fused(oracle):
    g = np.load(os.path.join(GOLDEN, "dense_fused.npz"))
    keys = sorted({k.rsplit("_", 1)[0] for k in g.files})
    assert len(keys) == 4
    for key in keys:
        X = g[key + "_X"].view(np.float16)
        gam = g[key + "_gamma"].view(np.float16)
        bet = g[key + "_beta"].view(np.float16)
        W = g[key + "_W"].view(np.float16)
        assert np.array_equal(oracle.fused_rmsnorm_gemv(X, gam, W, 1e-5).view(np.uint16),
                              g[key + "_Yrms"]), key
        assert np.array_equal(oracle.fused_layernorm_gemv(X, gam, bet, W, 1e-5).view(np.uint16),
                              g[key + "_Yln"]), key


def test_fp32_variant_is_the_same_loop(oracle):
    """With fp16-representable inputs the fp32 entry points must agree with the fp16 ABI ones
    after the final rounding."""
    rng = np.random.default_rng(5)
    N, K = 40, 512
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    X = rng.standard_normal((2, K)).astype(np.float16)
    for fmt in (0, 1):
        wq = oracle.quantize_weights(W, fmt)
        y16 = oracle.gemv_quantized(X, wq, fmt, N)
        y32 = oracle.gemv_quantized_f32(X.astype(np.float32), wq, fmt, N)
        assert np.array_equal(oracle.f32_to_f16_bits(y32), y16.view(np.uint16))
        y64 = oracle.dequant_dot_f64(X.astype(np.float64), wq, fmt, N)
        assert oracle.scaled_rms(y32, y64) < 2e-6


def test_against_reference_backend_when_built(oracle):
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    R = oracle.RefLib()
    rng = np.random.default_rng(11)
    for fmt in (0, 1):
        for (N, K, M) in ((17, 64, 1), (128, 256, 2), (9, 2048, 3)):
            W = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
            X = rng.standard_normal((M, K)).astype(np.float16)
            gam = (1 + 0.1 * rng.standard_normal(K)).astype(np.float16)
            wq = oracle.quantize_weights(W, fmt)
            assert np.array_equal(wq, R.quantize_weights(W, fmt))
            assert np.array_equal(oracle.gemv_quantized(X, wq, fmt, N).view(np.uint16),
                                  R.gemv_quantized(X, wq, fmt, N).view(np.uint16))
            assert np.array_equal(
                oracle.fused_rmsnorm_gemv_quantized(X, gam, wq, fmt, N).view(np.uint16),
                R.fused_rmsnorm_gemv_quantized(X, gam, wq, fmt, N).view(np.uint16))


def _step_inputs(rng, N, D):
    X = (rng.standard_normal((N, D)) * 1.5).astype(np.float16)
    g = (1 + 0.1 * rng.standard_normal(D)).astype(np.float16)
    b = (0.1 * rng.standard_normal(D)).astype(np.float16)
    return X, g, b


def test_step_ops_match_reference_golden(oracle):
    """RMSNorm / LayerNorm forward, SwiGLU and RoPE against outputs of the reference's CPU backend
    (tests/golden/step_ops.npz, written by make_golden.py): bit for bit."""
    g = np.load(os.path.join(GOLDEN, "step_ops.npz"))
    for key in sorted({k.rsplit("_", 1)[0] for k in g.files if k.startswith("norm_") and k.endswith("_X")}):
        X, gam, bet = (g[key + s].view(np.float16) for s in ("_X", "_gamma", "_beta"))
        y, r = oracle.rmsnorm_forward(X, gam)
        assert np.array_equal(y.view(np.uint16), g[key + "_Yrms"]) and np.array_equal(r, g[key + "_rstd_rms"]), key
        y, m, r = oracle.layernorm_forward(X, gam, bet)
        assert np.array_equal(y.view(np.uint16), g[key + "_Yln"]), key
        assert np.array_equal(m, g[key + "_mean_ln"]) and np.array_equal(r, g[key + "_rstd_ln"]), key
    out = oracle.swiglu_forward(g["swiglu_gate"].view(np.float16), g["swiglu_up"].view(np.float16))
    assert np.array_equal(out.view(np.uint16), g["swiglu_out"])
    out = oracle.rope_forward(g["rope_X"].view(np.float16), g["rope_cos"], g["rope_sin"])
    assert np.array_equal(out.view(np.uint16), g["rope_out"])


def test_step_ops_against_reference_backend_when_built(oracle):
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    R = oracle.RefLib()
    rng = np.random.default_rng(21)
    for (N, D) in ((1, 32), (4, 1000), (2, 8192)):
        X, gam, bet = _step_inputs(rng, N, D)
        a, b = oracle.rmsnorm_forward(X, gam), R.rmsnorm_forward(X, gam)
        assert np.array_equal(a[0].view(np.uint16), b[0].view(np.uint16)) and np.array_equal(a[1], b[1])
        a, b = oracle.layernorm_forward(X, gam, bet), R.layernorm_forward(X, gam, bet)
        assert all(np.array_equal(np.asarray(p).view(np.uint8), np.asarray(q).view(np.uint8)) for p, q in zip(a, b))
    gate, up = (rng.standard_normal(5000) * 6).astype(np.float16), rng.standard_normal(5000).astype(np.float16)
    assert np.array_equal(oracle.swiglu_forward(gate, up).view(np.uint16), R.swiglu_forward(gate, up).view(np.uint16))
    X = rng.standard_normal((1, 4, 7, 128)).astype(np.float16)
    ang = rng.uniform(0, 6.28, (7, 64)).astype(np.float32)
    assert np.array_equal(oracle.rope_forward(X, np.cos(ang), np.sin(ang)).view(np.uint16),
                          R.rope_forward(X, np.cos(ang), np.sin(ang)).view(np.uint16))


def test_gemm_against_reference_backend_when_built(oracle):
    """orc_gemm_f16 restates lib/ops/gemm_cpu.cpp:544-568; bit for bit against the reference's CPU
    tc_gemm, B as given and transposed, with alpha and beta - with the reference GEMM's own narrowing
    (ties up, a carry out of the mantissa lost when the exponent is odd).  With the IEEE narrowing,
    which parity targets use, only such elements differ."""
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    R = oracle.RefLib()
    rng = np.random.default_rng(33)
    differing = total = 0
    for (M, N, K) in ((1, 8, 8), (5, 24, 72), (33, 40, 256), (33, 40, 64)):
        A = rng.standard_normal((M, K)).astype(np.float16)
        B = rng.standard_normal((K, N)).astype(np.float16)
        C0 = rng.standard_normal((M, N)).astype(np.float16)
        for tb in (False, True):
            Bx = np.ascontiguousarray(B.T) if tb else B
            for alpha, beta in ((1.0, 0.0), (0.5, 0.0), (0.5, 1.5)):
                b = R.gemm_f16(A, Bx, tb, alpha, beta, C0)
                a = oracle.gemm_f16(A, Bx, tb, alpha, beta, C0, ref_narrowing=True)
                assert np.array_equal(a.view(np.uint16), b.view(np.uint16)), (M, N, K, tb, alpha, beta)
                ieee = oracle.gemm_f16(A, Bx, tb, alpha, beta, C0)
                differing += int(np.count_nonzero(ieee.view(np.uint16) != b.view(np.uint16)))
                total += ieee.size
    assert differing <= total // 200          # ties and lost carries are rare
    # A given transposed ([K][M])
    A = rng.standard_normal((40, 9)).astype(np.float16)
    B = rng.standard_normal((40, 16)).astype(np.float16)
    for tb in (False, True):
        Bx = np.ascontiguousarray(B.T) if tb else B
        a = oracle.gemm_f16(A, Bx, tb, 1.0, 0.0, None, True, transpose_a=True)
        b = R.gemm_f16(A, Bx, tb, 1.0, 0.0, None, 0, True)
        assert np.array_equal(a.view(np.uint16), b.view(np.uint16))


def test_gemm_matches_reference_golden_vectors(oracle):
    """tests/golden/gemm.npz holds outputs of the reference's CPU tc_gemm (fp16 with that file's own
    narrowing, bf16), either operand transposed, with alpha and beta: the oracle reproduces every byte."""
    g = np.load(os.path.join(GOLDEN, "gemm.npz"))
    names = sorted({k.rsplit("_A", 1)[0] for k in g.files if k.endswith("_A")})
    assert len(names) == 3
    for name in names:
        A, B, C0, dt = g[name + "_A"], g[name + "_B"], g[name + "_C0"], int(g[name + "_dtype"][0])
        for ta in (0, 1):
            for tb in (0, 1):
                for tag, alpha, beta in (("plain", 1.0, 0.0), ("ab", 0.5, 1.5)):
                    Ax = np.ascontiguousarray(A.T) if ta else A
                    Bx = np.ascontiguousarray(B.T) if tb else B
                    want = g[f"{name}_Y_{ta}{tb}_{tag}"]
                    if dt == 0:
                        got = oracle.gemm_f16(Ax.view(np.float16), Bx.view(np.float16), bool(tb), alpha, beta,
                                              C0.view(np.float16), True, bool(ta)).view(np.uint16)
                    else:
                        got = oracle.gemm_bf16(Ax, Bx, bool(tb), alpha, beta, C0, bool(ta))
                    assert np.array_equal(got, want), (name, ta, tb, tag)


def test_gemm_bf16_against_reference_backend_when_built(oracle):
    """The bfloat16 case of the same loop (conversions lib/ops/gemm_cpu.cpp:217-230): bit for bit."""
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    R = oracle.RefLib()
    rng = np.random.default_rng(34)
    for (M, N, K) in ((3, 8, 16), (17, 40, 136)):
        A = oracle.to_bf16_bits(rng.standard_normal((M, K)))
        B = oracle.to_bf16_bits(rng.standard_normal((K, N)))
        C0 = oracle.to_bf16_bits(rng.standard_normal((M, N)))
        for tb in (False, True):
            Bx = np.ascontiguousarray(B.T) if tb else B
            for alpha, beta in ((1.0, 0.0), (0.5, 1.5)):
                a = oracle.gemm_bf16(A, Bx, tb, alpha, beta, C0)
                b = R.gemm_f16(A, Bx, tb, alpha, beta, C0, dtype=1).view(np.uint16)
                assert np.array_equal(a, b), (M, N, K, tb, alpha, beta)
    # the bit helpers agree with a widening round trip
    x = rng.standard_normal(1000).astype(np.float32)
    assert np.array_equal(oracle.to_bf16_bits(oracle.from_bf16_bits(oracle.to_bf16_bits(x))), oracle.to_bf16_bits(x))


def _attention_cases(g):
    return sorted(k[:-2] for k in g.files if k.endswith("_Q"))


def test_attention_forward_matches_reference_golden_vectors(oracle):
    """lib/ops/attention_cpu.cpp:131-277 as run by the reference's CPU backend
    (tests/golden/attention.npz, written by make_golden.py on an AVX2 machine, hence dot_order 1):
    outputs and log-sum-exps bit for bit - decode rows, grouped-query heads, causal mask, sliding
    window, ALiBi, a head_dim that is not a multiple of 8."""
    g = np.load(os.path.join(GOLDEN, "attention.npz"))
    for name in _attention_cases(g):
        Q, K, V = (g[name + s].view(np.float16) for s in ("_Q", "_K", "_V"))
        causal, window = (int(v) for v in g[name + "_cfg"])
        sl = g[name + "_slopes"] if g[name + "_slopes"].size else None
        O, L = oracle.attention_forward(Q, K, V, 0.0, bool(causal), window, sl, True, dot_order=1)
        assert np.array_equal(O.view(np.uint16), g[name + "_O"]), name
        assert np.array_equal(L, g[name + "_LSE"]), name
        # the scalar dot-product order differs only in rounding
        O0 = oracle.attention_forward(Q, K, V, 0.0, bool(causal), window, sl, False, dot_order=0)
        assert np.abs(O0.astype(np.float32) - O.astype(np.float32)).max() < 2e-3, name


def test_attention_forward_against_fp64_softmax(oracle):
    """The tolerance the reference's own test uses against an fp64 reference
    (tests/test_attention_correctness.c:254-262): max abs error below 1e-3."""
    rng = np.random.default_rng(12)
    B, Hq, Hkv, Sq, Sk, D = 1, 4, 2, 3, 130, 64
    Q, K, V = (rng.standard_normal(s).astype(np.float16) for s in ((B, Hq, Sq, D), (B, Hkv, Sk, D), (B, Hkv, Sk, D)))
    O = oracle.attention_forward(Q, K, V, 0.0, True, 0, None, False).astype(np.float64)
    for h in range(Hq):
        for i in range(Sq):
            s = (K[0, h // 2].astype(np.float64) @ Q[0, h, i].astype(np.float64)) / np.sqrt(D)
            s[np.arange(Sk) > i] = -np.inf
            p = np.exp(s - s.max()); p /= p.sum()
            assert np.abs(p @ V[0, h // 2].astype(np.float64) - O[0, h, i]).max() < 1e-3
