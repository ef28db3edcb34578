"""GPU: behaviour of the drop-in boundary on a device - status codes in the reference's order,
host-mapped buffers, host-pointer wrappers, recorded streams and their graph replay, and the
GGUF device loader."""
import ctypes
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _small_case(oracle, fmt=0, N=130, K=256, M=1, seed=1):
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    X = rng.standard_normal((M, K)).astype(np.float16)
    return W, X, oracle.quantize_weights(W, fmt)


def test_context_is_a_refcounted_singleton(tc, ctx):
    h = ctypes.c_void_p()
    assert tc.lib().tc_init(ctypes.byref(h)) == tc.TC_ERR_ALREADY_INITIALIZED
    assert h.value == ctx.handle.value
    assert tc.lib().tc_shutdown(h) == tc.TC_OK          # drops the extra reference only
    info = ctx.device_info()
    assert info.name == b"cuda" and info.thread_execution_width == 32
    assert tc.cuda_device_count() >= 1


def test_status_codes_follow_the_reference_order(tc, ctx, oracle):
    W, X, Wq = _small_case(oracle)
    N, K = W.shape
    L = tc.lib()
    bx, bw, by = ctx.buffer_from_array(X), ctx.buffer_from_array(Wq), ctx.buffer(N * 2)
    small = ctx.buffer(16)
    c = ctx.handle
    args = (bx.handle, bw.handle, by.handle)
    assert L.tc_gemv_quantized(c, *args, 0, 1, N, K) == tc.TC_OK
    assert L.tc_gemv_quantized(c, None, bw.handle, by.handle, 0, 1, N, K) == tc.TC_ERR_INVALID_ARG
    assert L.tc_gemv_quantized(c, *args, 0, 0, N, K) == tc.TC_ERR_INVALID_ARG
    assert L.tc_gemv_quantized(c, *args, 0, 1, N, K + 16) == tc.TC_ERR_INVALID_ARG
    assert L.tc_gemv_quantized(c, *args, 9, 1, N, K) == tc.TC_ERR_INVALID_ARG      # unknown fmt
    assert L.tc_gemv_quantized(c, bx.handle, bw.handle, small.handle, 0, 1, N, K) == tc.TC_ERR_INVALID_SHAPE
    assert L.tc_gemv_quantized(c, small.handle, bw.handle, by.handle, 0, 1, N, K) == tc.TC_ERR_INVALID_SHAPE
    assert L.tc_gemv_quantized(c, bx.handle, small.handle, by.handle, 0, 1, N, K) == tc.TC_ERR_INVALID_SHAPE
    assert L.tc_quantize_weights(c, small.handle, bw.handle, 0, N, K) == tc.TC_ERR_INVALID_SHAPE
    assert L.tc_fused_rmsnorm_gemv_quantized(c, bx.handle, small.handle, bw.handle, by.handle, 0,
                                             1, N, K, 1e-5) == tc.TC_ERR_INVALID_SHAPE
    assert L.tc_fused_layernorm_gemv(c, bx.handle, bx.handle, None, bw.handle, by.handle, 1, 8, K,
                                     1e-5) == tc.TC_ERR_INVALID_ARG
    assert L.tc_fused_rmsnorm_gemv(c, bx.handle, bx.handle, small.handle, by.handle, 1, 8, K,
                                   1e-5) == tc.TC_ERR_INVALID_SHAPE
    s = ctx.stream()
    assert L.tc_gemv_quantized_async(c, *args, 0, 1, N, K, None) == tc.TC_ERR_INVALID_ARG
    assert L.tc_gemv_quantized_async(c, *args, 0, 1, N, K + 1, s.handle) == tc.TC_ERR_INVALID_ARG
    assert L.tc_buffer_alloc(c, 0, ctypes.byref(ctypes.c_void_p())) == tc.TC_ERR_INVALID_ARG
    for b in (bx, bw, by, small):
        b.close()
    s.close()


def test_mapped_buffers_reference_call_pattern(tc, ctx, oracle):
    """alloc -> map -> write -> op -> read through the mapped pointer, pointers held across
    operations and rewritten between them (tests/test_quantized.c:96-187)."""
    for fmt in (0, 1):
        W, X, _ = _small_case(oracle, fmt, N=128, K=256, seed=fmt + 2)
        N, K = W.shape
        bwf, bq = ctx.buffer(W.nbytes), ctx.buffer(tc.quantized_size(fmt, N, K))
        bx, by = ctx.buffer(X.nbytes), ctx.buffer(N * 2)
        bwf.write(W)
        ctx.quantize_weights(bwf, bq, fmt, N, K)
        q = np.empty(tc.quantized_size(fmt, N, K), np.uint8)
        bq.read(q)
        assert np.array_equal(q, oracle.quantize_weights(W, fmt))
        px, py = bx.map(), by.map()
        assert px == bx.map() and py == by.map()          # stable for the buffer's life
        for rep in range(3):
            Xr = (X.astype(np.float32) * (rep + 1)).astype(np.float16)
            ctypes.memmove(px, Xr.ctypes.data, Xr.nbytes)  # write through the held pointer
            ctx.gemv_quantized(bx, bq, by, fmt, 1, N, K)
            y = np.frombuffer(ctypes.string_at(py, N * 2), dtype=np.float16)
            want = oracle.gemv_quantized(Xr, q, fmt, N)[0]
            assert oracle.scaled_rms(y, want) <= 3e-4
        for b in (bwf, bq, bx, by):
            b.close()


def test_map_keeps_device_written_contents(tc, ctx, oracle):
    W, X, Wq = _small_case(oracle, 0, N=64, K=512, seed=9)
    bx, bw, by = ctx.buffer_from_array(X), ctx.buffer_from_array(Wq), ctx.buffer(64 * 2)
    ctx.gemv_quantized(bx, bw, by, 0, 1, 64, 512)
    before = by.to_numpy((64,), np.float16)
    y = np.empty(64, np.float16)
    by.read(y)                                            # first map: storage moves, data kept
    assert np.array_equal(y.view(np.uint16), before.view(np.uint16))
    for b in (bx, bw, by):
        b.close()


def test_host_pointer_wrappers_are_staged(tc, ctx, oracle):
    W, X, Wq = _small_case(oracle, 1, N=96, K=256, seed=4)
    Xh, Wh, Yh = X.copy(), Wq.copy(), np.zeros(96, np.float16)
    bx = ctx.buffer_from_ptr(Xh.ctypes.data, Xh.nbytes)
    bw = ctx.buffer_from_ptr(Wh.ctypes.data, Wh.nbytes)
    by = ctx.buffer_from_ptr(Yh.ctypes.data, Yh.nbytes)
    ctx.gemv_quantized(bx, bw, by, 1, 1, 96, 256)
    assert oracle.scaled_rms(Yh, oracle.gemv_quantized(X, Wq, 1, 96)[0]) <= 3e-4
    Xh *= np.float16(0.5)                                 # caller memory changes between calls
    ctx.gemv_quantized(bx, bw, by, 1, 1, 96, 256)
    assert oracle.scaled_rms(Yh, oracle.gemv_quantized(Xh.reshape(1, -1), Wq, 1, 96)[0]) <= 3e-4
    assert bx.map() == Xh.ctypes.data
    for b in (bx, bw, by):
        b.close()


def test_async_stream_records_and_replays(tc, ctx, oracle):
    """Seven GEMVs recorded per sync, repeated: the first submission launches directly, the
    second builds a graph, later ones replay it; results never change."""
    rng = np.random.default_rng(21)
    K, Ns = 512, [64, 130, 96, 257, 64, 64, 300]
    X = rng.standard_normal((1, K)).astype(np.float16)
    Wqs = [oracle.quantize_weights((rng.standard_normal((n, K)) * 0.02).astype(np.float16), 0)
           for n in Ns]
    want = [oracle.gemv_quantized(X, wq, 0, n)[0] for wq, n in zip(Wqs, Ns)]
    bx = ctx.buffer_from_array(X)
    bws = [ctx.buffer_from_array(w) for w in Wqs]
    bys = [ctx.buffer(n * 2) for n in Ns]
    s = ctx.stream()
    first = None
    launches0 = tc.launch_count()
    for rep in range(5):
        for bw, by, n in zip(bws, bys, Ns):
            ctx.gemv_quantized_async(bx, bw, by, 0, 1, n, K, s)
        s.sync()
        outs = [by.to_numpy((n,), np.float16) for by, n in zip(bys, Ns)]
        for o, w in zip(outs, want):
            assert oracle.scaled_rms(o, w) <= 3e-4
        if first is None:
            first = outs
    # one kernel per GEMV, or one persistent launch per synchronisation for a qualifying list
    assert tc.launch_count() - launches0 in (5 * len(Ns), 5)
    assert tc.take_device_error(ctx) == 0
    # a dependent chain on one stream: y of one GEMV is x of the next
    Wa = oracle.quantize_weights((rng.standard_normal((K, K)) * 0.05).astype(np.float16), 0)
    ba, bm, bo = ctx.buffer_from_array(Wa), ctx.buffer(K * 2), ctx.buffer(K * 2)
    for rep in range(3):
        ctx.gemv_quantized_async(bx, ba, bm, 0, 1, K, K, s)
        ctx.gemv_quantized_async(bm, ba, bo, 0, 1, K, K, s)
        s.sync()
        mid = oracle.gemv_quantized(X, Wa, 0, K)
        assert oracle.scaled_rms(bo.to_numpy((K,), np.float16),
                                 oracle.gemv_quantized(mid, Wa, 0, K)[0]) <= 2e-4
    for b in [bx, ba, bm, bo] + bws + bys:
        b.close()
    s.close()


def test_gguf_load_to_device_and_known_answer(tc, ctx, tmp_path, oracle):
    from tensorcore_b200 import gguf_writer as gw
    rng = np.random.default_rng(8)
    N, K = 200, 512
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float16)
    wq4, wq8 = oracle.quantize_weights(W, 0), oracle.quantize_weights(W, 1)
    norm = np.ones(K, np.float32)
    kat = struct.pack("<H", 0x3800) + bytes([0xAB] * 16)
    path = str(tmp_path / "m.gguf")
    gw.write_gguf(path, gw.llama_metadata(K, 4 * K, 1, 8, 8, 10), [
        gw.TensorSpec("weight.test", [32, 1], gw.GGML_Q4_0, 18, data=kat),
        gw.TensorSpec("blk.0.attn_q.weight", [K, N], gw.GGML_Q4_0, wq4.size, data=wq4),
        gw.TensorSpec("blk.0.attn_k.weight", [K, N], gw.GGML_Q8_0, wq8.size, data=wq8),
        gw.TensorSpec("blk.0.attn_norm.weight", [K], gw.GGML_F32, K * 4, data=norm),
        gw.TensorSpec("odd", [32], 999, 0, data=b""),
    ])
    with tc.GgufFile(path) as g, g.load_supported_tensors(ctx) as model:
        assert model.tensor_count() == 4 and model.skipped_tensor_count() == 1
        t = model.get_tensor("blk.0.attn_norm.weight")
        assert t["dims"] == [K] and t["n_bytes"] == K * 4
        kq = model.quantized_matrix("weight.test")
        assert (kq.N, kq.K, kq.n_bytes) == (1, 32, 18)
        x1 = ctx.buffer_from_array(np.full(32, 0x3C00, np.uint16))
        y1 = kq.output()
        kq.gemv(x1, y1)
        assert y1.to_numpy((1,), np.uint16)[0] == 0x5100          # tests/test_gguf.c:274-279
        X = rng.standard_normal((1, K)).astype(np.float16)
        bx = ctx.buffer_from_array(X)
        for name, fmt, wq in (("blk.0.attn_q.weight", 0, wq4), ("blk.0.attn_k.weight", 1, wq8)):
            qm = model.quantized_matrix(name)
            assert (qm.N, qm.K, qm.quant_type) == (N, K, fmt)
            assert np.array_equal(qm.buffer.to_numpy((wq.size,), np.uint8), wq)
            by = qm.output()
            qm.gemv(bx, by)
            assert oracle.scaled_rms(by.to_numpy((N,), np.float16),
                                     oracle.gemv_quantized(X, wq, fmt, N)[0]) <= 3e-4
            by.close()
        with pytest.raises(tc.TensorcoreError) as e:
            model.quantized_matrix("blk.0.attn_norm.weight")
        assert e.value.status == tc.TC_ERR_UNSUPPORTED_DTYPE
        single = g.tensor_to_buffer(ctx, "blk.0.attn_q.weight")
        assert np.array_equal(single.to_numpy((wq4.size,), np.uint8), wq4)
        with pytest.raises(tc.TensorcoreError):
            g.tensor_to_buffer(ctx, "odd")
        for b in (x1, y1, bx, single):
            b.close()


def test_first_map_between_record_and_sync(tc, ctx, oracle):
    """Legal under the reference contract (include/tensorcore/device.h:59-62: the mapped pointer is
    stable and coherent at sync points): record an operation, map its never-mapped result and
    input buffers for the first time - which moves them to host-visible storage - then sync and
    read the result through the mapped pointer."""
    import ctypes
    rng = np.random.default_rng(31)
    N, K = 96, 512
    for fmt in (0, 1):
        Wq = oracle.quantize_weights((rng.standard_normal((N, K)) * 0.02).astype(np.float16), fmt)
        X = rng.standard_normal((1, K)).astype(np.float16)
        want = oracle.gemv_quantized(X, Wq, fmt, N)
        bw, bx, by = ctx.buffer_from_array(Wq), ctx.buffer(K * 2), ctx.buffer(N * 2)
        bx.upload(X)
        s = ctx.stream()
        ctx.gemv_quantized_async(bx, bw, by, fmt, 1, N, K, s)
        ctx.gemv_quantized_async(bx, bw, by, fmt, 1, N, K, s)
        py = by.map()                    # first map of Y: after recording, before the sync
        px = bx.map()                    # and of X
        s.sync()
        got = np.ctypeslib.as_array(ctypes.cast(py, ctypes.POINTER(ctypes.c_uint16)), (1, N)).view(np.float16)
        assert oracle.scaled_rms(got.copy(), want) <= 3e-4, fmt
        assert by.map() == py and bx.map() == px          # stable pointers
        s.close()
        for b in (bw, bx, by):
            b.close()
    assert tc.take_device_error(ctx) == 0
