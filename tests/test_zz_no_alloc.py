"""GPU: the decode entry point that allocates nothing (tcx_raw_decode_q4_static).

Who it is for: callers that cannot afford an allocation on the decode path - a server that has
handed all of its HBM to weights and KV cache at start-up, or a loop in which cudaMalloc's
device-wide synchronisation must not happen.  The entry point keeps the persistent kernel's
scratch (operation table, tensor maps, grid-barrier counter, fp32 accumulators) in a fixed device
array of the library image.

The check: the same five-operation decode fragment is run through the existing per-operation
raw entry points and through the new one, through the C ABI, twice in a row (the array keeps the
previous call's contents, so the second call proves that it is re-initialised), and the
outputs must agree with the existing entry points' and with the oracle's values for the same
fragment, within the tolerances of the other GPU tests.  The file sorts last so that a
run that stops at the first failure has executed every other test before it."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _fragment(tc, ctx, oracle, seed):
    rng = np.random.default_rng(seed)
    d, f = 1024, 2816
    mk = lambda n, k: oracle.quantize_weights((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float16), 0)
    B = ctx.buffer_from_array
    w = {n: B(mk(*s)) for n, s in (("q", (d, d)), ("k", (256, d)), ("o", (d, d)), ("g", (f, d)), ("dn", (d, f)))}
    x = B(rng.standard_normal((1, d)).astype(np.float16))
    g16 = (1 + 0.1 * rng.standard_normal(d)).astype(np.float16)
    gam16, gam32 = B(g16), B(g16.astype(np.float32))
    return d, f, w, x, gam16, gam32


def _oracle_values(oracle, ctx, d, f, w, x, gam16):
    """The fragment on the CPU: q, k = fused(x); o = gemv(q) in fp32; g = fused_f32(o); y = gemv(g)."""
    host = {n: b.to_numpy((b.nbytes,), np.uint8) for n, b in w.items()}
    x16 = x.to_numpy((1, d), np.float16)
    g16 = gam16.to_numpy((d,), np.float16)
    q = oracle.fused_rmsnorm_gemv_quantized(x16, g16, host["q"], 0, d)
    k = oracle.fused_rmsnorm_gemv_quantized(x16, g16, host["k"], 0, 256)
    o = oracle.gemv_quantized_f32(q.astype(np.float32), host["o"], 0, d)
    g = oracle.fused_rmsnorm_gemv_quantized_f32(o, g16.astype(np.float32), host["g"], 0, f).astype(np.float16)
    y = oracle.gemv_quantized(g, host["dn"], 0, d)
    return {"q": q.ravel(), "k": k.ravel(), "o": o.ravel(), "g": g.ravel(), "y": y.ravel()}


def _outputs(ctx, d, f):
    return {"q": ctx.buffer(d * 2), "k": ctx.buffer(256 * 2), "o": ctx.buffer(d * 4),
            "g": ctx.buffer(f * 2), "y": ctx.buffer(d * 2)}


def _read(out, d, f):
    return {"q": out["q"].to_numpy((d,), np.float16), "k": out["k"].to_numpy((256,), np.float16),
            "o": out["o"].to_numpy((d,), np.float32), "g": out["g"].to_numpy((f,), np.float16),
            "y": out["y"].to_numpy((d,), np.float16)}


def test_static_scratch_decode_matches_existing_entry_points(tc, ctx, oracle):
    import torch
    d, f, w, x, gam16, gam32 = _fragment(tc, ctx, oracle, 2718)
    ref, new = _outputs(ctx, d, f), _outputs(ctx, d, f)
    P = lambda b: b.device_ptr()
    stream = torch.cuda.Stream()
    st = stream.cuda_stream

    def run_existing(o):
        tc.raw_fused_rmsnorm_gemv_quantized(ctx, P(x), P(gam16), P(w["q"]), P(o["q"]), 0, 1, d, d, 1e-5, "f16", "f16", st)
        tc.raw_fused_rmsnorm_gemv_quantized(ctx, P(x), P(gam16), P(w["k"]), P(o["k"]), 0, 1, 256, d, 1e-5, "f16", "f16", st)
        tc.raw_gemv_quantized(ctx, P(o["q"]), P(w["o"]), P(o["o"]), 0, 1, d, d, "f16", "f32", st)
        tc.raw_fused_rmsnorm_gemv_quantized(ctx, P(o["o"]), P(gam32), P(w["g"]), P(o["g"]), 0, 1, f, d, 1e-5, "f32", "f16", st)
        tc.raw_gemv_quantized(ctx, P(o["g"]), P(w["dn"]), P(o["y"]), 0, 1, d, f, "f16", "f16", st)
        stream.synchronize()

    def run_static(o):
        ops = [
            dict(W=P(w["q"]), X=P(x), Y=P(o["q"]), gamma=P(gam16), N=d, K=d),
            dict(W=P(w["k"]), X=P(x), Y=P(o["k"]), gamma=P(gam16), N=256, K=d),
            dict(W=P(w["o"]), X=P(o["q"]), Y=P(o["o"]), N=d, K=d, y_dtype="f32"),
            dict(W=P(w["g"]), X=P(o["o"]), Y=P(o["g"]), gamma=P(gam32), N=f, K=d, x_dtype="f32"),
            dict(W=P(w["dn"]), X=P(o["g"]), Y=P(o["y"]), N=d, K=f),
        ]
        tc.raw_decode_q4_static(ctx, ops, st)
        stream.synchronize()
        assert "static" in tc.cuda_last_kernel_name()

    run_existing(ref)
    want = _read(ref, d, f)
    cpu = _oracle_values(oracle, ctx, d, f, w, x, gam16)
    for call in range(2):                      # two calls in a row share the static array
        for b in new.values():                 # poison the outputs so that stale data cannot pass
            b.upload(np.full(b.nbytes, 0x7F, np.uint8))
        run_static(new)
        got = _read(new, d, f)
        assert oracle.scaled_rms(got["q"], want["q"]) <= 3e-4, call
        assert oracle.scaled_rms(got["k"], want["k"]) <= 3e-4, call
        # downstream of an fp16 hand-off: rounding flips of q feed o (fp16-activation bar)
        assert oracle.scaled_rms(got["o"], want["o"]) <= 2e-3, call
        assert oracle.scaled_rms(got["g"], want["g"]) <= 2e-3, call
        assert oracle.scaled_rms(got["y"], want["y"]) <= 2e-3, call
        # and against the CPU restatement of the reference, bars as in test_gpu_persistent.py
        assert oracle.scaled_rms(got["q"], cpu["q"]) <= 3e-4, call
        assert oracle.scaled_rms(got["k"], cpu["k"]) <= 3e-4, call
        for n in ("o", "g", "y"):
            assert oracle.scaled_rms(got[n], cpu[n]) <= 2e-3, (call, n)
    assert tc.take_device_error(ctx) == 0


def test_static_scratch_decode_rejects_lists_beyond_its_capacity(tc, ctx):
    buf = ctx.buffer(1 << 20)
    p = buf.device_ptr()
    op = dict(W=p, X=p, Y=p + (1 << 19), N=16, K=256)
    with pytest.raises(tc.TensorcoreError) as e:
        tc.raw_decode_q4_static(ctx, [op] * (tc.DECODE_STATIC_MAX_OPS + 1))
    assert e.value.status == tc.TC_ERR_INVALID_SHAPE
    with pytest.raises(tc.TensorcoreError) as e:
        tc.raw_decode_q4_static(ctx, [dict(op, K=96)])          # outside the kernel's domain
    assert e.value.status == tc.TC_ERR_INVALID_SHAPE
    buf.close()
