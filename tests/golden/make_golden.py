"""Generates tests/golden/*.npz by running the reference's own portable-CPU backend
(oracle/_ref/libtensorcore_ref.so, compiled from the reference sources by oracle/Makefile).

Run where a reference checkout is present:  python tests/golden/make_golden.py
The fixtures are small (a few hundred KB in total) and are committed; the GPU box has no
reference checkout and reads only these files.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as O  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def weights(rng, N, K):
    """fp32 N(0, 0.02^2) rounded to fp16, with the edge blocks the quantiser must get right."""
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32).astype(np.float16)
    W[0, :32] = 0                       # all-zero block: scale 0, codes 8 / 0
    W[1, 32:64] = np.float16(-0.5)      # constant negative block: codes clamp at 0 / -127
    W[2, :32] = np.float16(6.1e-5)      # smallest normal fp16: subnormal scale
    W[3, 5] = np.float16(3.0)           # one large value: the rest of the block rounds to zero
    W[4, :32] = np.linspace(-1, 1, 32).astype(np.float16)   # exact .5 ties after scaling
    return W


def main() -> None:
    R = O.RefLib()
    rng = np.random.default_rng(0x7C0DE)
    cases = {}
    for fmt, tag in ((O.Q4_0, "q4_0"), (O.Q8_0, "q8_0")):
        for (N, K, M) in ((8, 32, 1), (130, 256, 1), (97, 512, 3), (64, 1024, 4), (33, 4096, 2)):
            W = weights(rng, N, K)
            X = rng.standard_normal((M, K)).astype(np.float32).astype(np.float16)
            g = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32).astype(np.float16)
            Wq = R.quantize_weights(W, fmt)
            key = f"{tag}_N{N}_K{K}_M{M}"
            cases[key + "_W"] = W.view(np.uint16)
            cases[key + "_X"] = X.view(np.uint16)
            cases[key + "_gamma"] = g.view(np.uint16)
            cases[key + "_Wq"] = Wq
            cases[key + "_Y"] = R.gemv_quantized(X, Wq, fmt, N).view(np.uint16)
            cases[key + "_Yfused"] = R.fused_rmsnorm_gemv_quantized(X, g, Wq, fmt, N, 1e-5).view(np.uint16)
    np.savez_compressed(os.path.join(OUT, "quantized_path.npz"), **cases)

    dense = {}
    for (M, N, K) in ((1, 128, 256), (2, 96, 512), (4, 40, 1024), (1, 33, 64)):
        X = rng.standard_normal((M, K)).astype(np.float32).astype(np.float16)
        g = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32).astype(np.float16)
        b = (0.1 * rng.standard_normal(K)).astype(np.float32).astype(np.float16)
        W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32).astype(np.float16)
        key = f"M{M}_N{N}_K{K}"
        dense[key + "_X"] = X.view(np.uint16)
        dense[key + "_gamma"] = g.view(np.uint16)
        dense[key + "_beta"] = b.view(np.uint16)
        dense[key + "_W"] = W.view(np.uint16)
        dense[key + "_Yrms"] = R.fused_rmsnorm_gemv(X, g, W, 1e-5).view(np.uint16)
        dense[key + "_Yln"] = R.fused_layernorm_gemv(X, g, b, W, 1e-5).view(np.uint16)
    np.savez_compressed(os.path.join(OUT, "dense_fused.npz"), **dense)
    step = {}
    for (N, D) in ((1, 64), (3, 256), (2, 4096)):
        X = (rng.standard_normal((N, D)) * 1.5).astype(np.float32).astype(np.float16)
        g = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32).astype(np.float16)
        b = (0.1 * rng.standard_normal(D)).astype(np.float32).astype(np.float16)
        key = f"norm_N{N}_D{D}"
        step[key + "_X"], step[key + "_gamma"], step[key + "_beta"] = X.view(np.uint16), g.view(np.uint16), b.view(np.uint16)
        y, r = R.rmsnorm_forward(X, g, 1e-5)
        step[key + "_Yrms"], step[key + "_rstd_rms"] = y.view(np.uint16), r
        y, m, r = R.layernorm_forward(X, g, b, 1e-5)
        step[key + "_Yln"], step[key + "_mean_ln"], step[key + "_rstd_ln"] = y.view(np.uint16), m, r
    gate = np.concatenate([rng.standard_normal(2000) * 4, [-60.0, 60.0, 0.0, -0.0, 49.9, -49.9]]).astype(np.float16)
    up = rng.standard_normal(gate.size).astype(np.float16)
    step["swiglu_gate"], step["swiglu_up"] = gate.view(np.uint16), up.view(np.uint16)
    step["swiglu_out"] = R.swiglu_forward(gate, up).view(np.uint16)
    B, H, S, D = 2, 3, 5, 64
    X = rng.standard_normal((B, H, S, D)).astype(np.float16)
    ang = np.outer(np.arange(S), 10000.0 ** (-np.arange(D // 2) / (D // 2))).astype(np.float32)
    step["rope_X"], step["rope_cos"], step["rope_sin"] = X.view(np.uint16), np.cos(ang), np.sin(ang)
    step["rope_out"] = R.rope_forward(X, np.cos(ang), np.sin(ang)).view(np.uint16)
    np.savez_compressed(os.path.join(OUT, "step_ops.npz"), **step)
    # attention forward: decode rows (seq_q = 1) and a few short prefill shapes
    att = {}
    cases = [("dec_mha", 1, 4, 4, 1, 300, 64, False, 0, False), ("dec_gqa_alibi", 1, 8, 2, 1, 400, 128, False, 0, True),
             ("causal_gqa", 1, 4, 2, 5, 77, 128, True, 0, False), ("window_alibi", 1, 2, 2, 40, 70, 64, True, 16, True),
             ("odd_dim", 1, 3, 3, 1, 65, 40, False, 0, False)]
    for name, B, Hq, Hkv, Sq, Sk, D, causal, window, alibi in cases:
        Q = rng.standard_normal((B, Hq, Sq, D)).astype(np.float16)
        K = rng.standard_normal((B, Hkv, Sk, D)).astype(np.float16)
        V = rng.standard_normal((B, Hkv, Sk, D)).astype(np.float16)
        sl = (0.05 * rng.random(Hq)).astype(np.float32) if alibi else np.zeros(0, np.float32)
        Oa, La = R.attention_forward(Q, K, V, 0.0, causal, window, sl if alibi else None, True)
        att[name + "_Q"], att[name + "_K"], att[name + "_V"] = Q.view(np.uint16), K.view(np.uint16), V.view(np.uint16)
        att[name + "_slopes"], att[name + "_cfg"] = sl, np.array([int(causal), window], np.int32)
        att[name + "_O"], att[name + "_LSE"] = Oa.view(np.uint16), La
    np.savez_compressed(os.path.join(OUT, "attention.npz"), **att)
    gemm_fixture(R)
    print("wrote", sorted(os.listdir(OUT)))


def gemm_fixture(R) -> None:
    """tc_gemm of the reference's CPU backend: fp16 and bf16 storage, either operand transposed, alpha and
    beta.  Its own generator so that the other fixtures keep their random streams."""
    rng = np.random.default_rng(0x6E44)
    out = {}
    for name, M, N, K, dt in (("f16_small", 5, 24, 72, 0), ("f16_mid", 33, 40, 256, 0), ("bf16_mid", 17, 40, 136, 1)):
        conv = (lambda a: a.astype(np.float16).view(np.uint16)) if dt == 0 else O.to_bf16_bits
        A, B, C0 = conv(rng.standard_normal((M, K))), conv(rng.standard_normal((K, N))), conv(rng.standard_normal((M, N)))
        out[name + "_A"], out[name + "_B"], out[name + "_C0"] = A, B, C0
        out[name + "_dtype"] = np.array([dt], np.int32)
        for ta in (0, 1):
            for tb in (0, 1):
                for tag, alpha, beta in (("plain", 1.0, 0.0), ("ab", 0.5, 1.5)):
                    Ax = np.ascontiguousarray(A.T) if ta else A
                    Bx = np.ascontiguousarray(B.T) if tb else B
                    view = (lambda a: a.view(np.float16)) if dt == 0 else (lambda a: a)
                    Y = R.gemm_f16(view(Ax), view(Bx), bool(tb), alpha, beta, view(C0), dtype=dt, transpose_a=bool(ta))
                    out[f"{name}_Y_{ta}{tb}_{tag}"] = np.ascontiguousarray(Y).view(np.uint16)
    np.savez_compressed(os.path.join(OUT, "gemm.npz"), **out)


if __name__ == "__main__":
    main()
