"""GPU: the recorded decode step (compiled harness over the C ABI) on a small Llama-shaped
model loaded from a synthetic GGUF file, checked projection by projection against the oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def oracle_token(oracle, shape, fmt, W, norms, x, fused):
    """Mirror of csrc/harness/decode_harness.cpp:record_token on the CPU."""
    def proj(xin, gamma, name, which):
        N, _ = shape.proj_shape(which)
        if fused and gamma is not None:
            return oracle.fused_rmsnorm_gemv_quantized(xin, gamma, W[name], fmt, N, 1e-5)
        return oracle.gemv_quantized(xin, W[name], fmt, N)
    cur = x
    for l in range(shape.n_layers):
        an, fn = norms[f"blk.{l}.attn_norm.weight"], norms[f"blk.{l}.ffn_norm.weight"]
        q = proj(cur, an, f"blk.{l}.attn_q.weight", "attn_q")
        o = proj(q, None, f"blk.{l}.attn_output.weight", "attn_output")
        gate = proj(o, fn, f"blk.{l}.ffn_gate.weight", "ffn_gate")
        cur = proj(gate, None, f"blk.{l}.ffn_down.weight", "ffn_down")
    return proj(cur, norms["output_norm.weight"], "output.weight", "output")


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("M", [1, 3])
def test_decode_session_matches_oracle_chain(tc, ctx, oracle, tmp_path, fmt, M):
    from tensorcore_b200 import decode as D
    shape = D.tiny_shape()
    path = str(tmp_path / "tiny.gguf")
    nbytes = D.build_synthetic_gguf(path, shape, ctx, fmt)
    assert nbytes == shape.weight_bytes(fmt)
    model = D.model_from_gguf(ctx, path, shape, fmt)
    assert model.owner.tensor_count() == shape.n_layers * 9 + 2
    # host copies of what was loaded, for the oracle
    W, norms = {}, {}
    for i in range(model.owner.tensor_count()):
        t = model.owner.tensor_at(i)
        buf = tc.Buffer(ctx, handle=__import__("ctypes").c_void_p(t["buffer"]), owned=False)
        if t["type"] in (tc.TC_GGUF_TYPE_Q4_0, tc.TC_GGUF_TYPE_Q8_0):
            W[t["name"]] = buf.to_numpy((t["n_bytes"],), np.uint8)
        else:
            norms[t["name"]] = buf.to_numpy((t["dims"][0],), np.float16)
    # the device quantiser produced exactly what the oracle would from the same fp16 weights
    w16 = D.device_weights_fp16(*shape.proj_shape("attn_q"), D.tensor_seed(0, 0)).cpu().numpy()
    assert np.array_equal(W["blk.0.attn_q.weight"], oracle.quantize_weights(w16, fmt))

    rng = np.random.default_rng(D.X_SEED)
    x = rng.standard_normal((M, shape.d_model)).astype(np.float16)
    sess = D.DecodeSession(ctx, model, M)
    for fused in (False, True):
        want = oracle_token(oracle, shape, fmt, W, norms, x, fused)
        for rep in range(3):          # direct launch, graph build, graph replay
            sess.x.upload(x)
            sess.run(1, fused_norms=fused)
            got = sess.logits.to_numpy((M, shape.vocab), np.float16)
            # Nine dependent GEMVs with fp16 hand-offs: an fp16 rounding flip in one output
            # (a different but equally valid fp32 summation order) perturbs the next one's
            # input.  The same chain on the CPU (fp64 accumulation vs the reference order)
            # grows from 1e-5 to 6e-4 over nine stages; the bar is the fp16-activation
            # tolerance.
            assert oracle.scaled_rms(got, want) <= 2e-3, (fused, rep)
    gpu_ms, wall_ms = sess.run(4, fused_norms=True)
    assert gpu_ms > 0 and wall_ms > 0
    assert tc.take_device_error(ctx) == 0
    sess.close()
    model.owner.close()


def test_tp_decoder_fused_backend_world1_matches_oracle_chain(tc, ctx, oracle):
    """The tensor-parallel decoder's data flow (fp32 hidden states, K-split projections with fp32
    results, logits 'gathered' into the full vector) on ONE GPU through the fused back end - one
    persistent launch per token via tcx_stream_decode_tp - against the same chain on the CPU."""
    import torch
    from tensorcore_b200 import decode as D
    from tensorcore_b200 import tp as TP
    shape = D.tiny_shape()
    device = torch.device("cuda", torch.cuda.current_device())

    class Recording(TP.FusedBackend):
        def weight(self, which, seed, rows, cols):
            N, K = self.shape.proj_shape(which)
            w = D.device_weights_fp16(N, K, seed, self.device)
            if rows is not None:
                w = w[rows[0]:rows[1]]
            if cols is not None:
                w = w[:, cols[0]:cols[1]]
            self.host = getattr(self, "host", {})
            ptr = super().weight(which, seed, rows, cols)
            self.host[ptr] = oracle.quantize_weights(w.contiguous().cpu().numpy(), 0)
            return ptr

    be = Recording(ctx, shape, 0, device, TP.TPLink(ctx, None, 1, 0))
    dec = TP.TPDecoder(TP.TPPlan(shape, 1, 0), be, 0)
    dec.token()
    be.commit()
    rng = np.random.default_rng(D.X_SEED)
    x = rng.standard_normal(shape.d_model).astype(np.float32)
    # the same chain on the CPU
    g = lambda t: t.cpu().numpy()
    cur = x[None, :]
    for l, lw in enumerate(dec.w):
        q = oracle.fused_rmsnorm_gemv_quantized_f32(cur, g(lw["attn_norm"]), be.host[lw["attn_q"]], 0, shape.d_model).astype(np.float16)
        o = oracle.gemv_quantized_f32(q.astype(np.float32), be.host[lw["attn_output"]], 0, shape.d_model)
        gate = oracle.fused_rmsnorm_gemv_quantized_f32(o, g(lw["ffn_norm"]), be.host[lw["ffn_gate"]], 0, shape.d_ff).astype(np.float16)
        cur = oracle.gemv_quantized_f32(gate.astype(np.float32), be.host[lw["ffn_down"]], 0, shape.d_model)
    want = oracle.fused_rmsnorm_gemv_quantized_f32(cur, g(dec.out_norm), be.host[dec.lm_head], 0, shape.vocab).astype(np.float16)
    for rep in range(3):
        dec.x_in.copy_(torch.from_numpy(x))
        torch.cuda.synchronize()
        be.run()
        be.sync()
        assert "persistent" in tc.cuda_last_kernel_name()
        got = dec.logits.cpu().numpy()[None, :]
        assert oracle.scaled_rms(got, want) <= 2e-3, rep      # nine dependent GEMVs with fp16 hand-offs
        assert oracle.scaled_rms(dec.h[(shape.n_layers - 1) & 1].cpu().numpy()[None, :], cur) <= 2e-3
    assert tc.take_device_error(ctx) == 0
    be.stream.close()


@pytest.mark.parametrize("use_graph", [False, True])
def test_batched_step_world1_matches_oracle_chain(tc, ctx, oracle, use_graph):
    """The batched decode step of the tensor-parallel bench (eight rows, one kernel per projection,
    fp32 partial sums rounded to fp16 between projections) on ONE GPU against the same chain on the
    CPU; launched eagerly and replayed from a captured CUDA graph."""
    import torch
    from tensorcore_b200 import decode as D
    from tensorcore_b200 import tp as TP
    shape = D.tiny_shape()
    device = torch.device("cuda", torch.cuda.current_device())

    class Recording(TP.FusedBackend):
        def weight(self, which, seed, rows, cols):
            N, K = self.shape.proj_shape(which)
            w = D.device_weights_fp16(N, K, seed, self.device)
            self.host = getattr(self, "host", {})
            ptr = super().weight(which, seed, rows, cols)
            self.host[ptr] = oracle.quantize_weights(w.contiguous().cpu().numpy(), 0)
            return ptr

    be = Recording(ctx, shape, 0, device, TP.TPLink(ctx, None, 1, 0))
    dec = TP.TPDecoder(TP.TPPlan(shape, 1, 0), be, 0)
    M = 8
    xb = TP.batch_input(shape, M)
    g = lambda t: t.cpu().numpy()
    f32 = lambda a: a.astype(np.float32)
    cur = xb
    for lw in dec.w:
        q = oracle.fused_rmsnorm_gemv_quantized_f32(f32(cur), g(lw["attn_norm"]), be.host[lw["attn_q"]], 0, shape.d_model).astype(np.float16)
        cur = oracle.gemv_quantized_f32(f32(q), be.host[lw["attn_output"]], 0, shape.d_model).astype(np.float16)
        gate = oracle.fused_rmsnorm_gemv_quantized_f32(f32(cur), g(lw["ffn_norm"]), be.host[lw["ffn_gate"]], 0, shape.d_ff).astype(np.float16)
        cur = oracle.gemv_quantized_f32(f32(gate), be.host[lw["ffn_down"]], 0, shape.d_model).astype(np.float16)
    want = oracle.fused_rmsnorm_gemv_quantized_f32(f32(cur), g(dec.out_norm), be.host[dec.lm_head], 0, shape.vocab).astype(np.float16)

    step = TP.BatchedStep(dec, ctx, None, device, M, collectives=False)
    step.x_in.copy_(torch.from_numpy(xb))
    torch.cuda.synchronize()
    step.prepare(use_graph)
    assert (step.graph is not None) == use_graph
    for rep in range(3):
        step.run()
        step.stream.synchronize()
        got = step.logits().cpu().numpy()
        assert got.shape == want.shape
        assert oracle.scaled_rms(got, want) <= 2e-3, rep
    assert step.launches == 7 * shape.n_layers + 1
    assert tc.take_device_error(ctx) == 0
    be.stream.close()
