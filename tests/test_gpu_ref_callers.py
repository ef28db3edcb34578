"""GPU: the reference's own callers driven against this library.

`build()` compiles, from a reference checkout, the reference's C tests for the path
(tests/test_quantized.c with its backend assertion widened by one `sed` to accept "cuda",
tests/test_gguf.c, tests/test_fused_norm_gemv.c) and its decode benchmark
(bench/bench_inference_7b.c) against tensorcore_b200/lib/libtensorcore.so, and stages the
reference's unchanged Python binding; all of it lives under baseline/_ref/ (git-ignored, carried
to the GPU box as built files).  These tests run them and look for the markers the reference's
own evidence script requires (scripts/run_quantized_gguf_runtime_evidence.py:26-62).
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

BIN = os.path.join(ROOT, "baseline", "_ref", "bin")
REF_PY = os.path.join(ROOT, "baseline", "_ref", "python")


def run_binary(name, *args, timeout=300):
    path = os.path.join(BIN, name)
    if not os.path.exists(path):
        pytest.skip(f"{path} was not built (no reference checkout when build() ran)")
    out = subprocess.run([path, *args], capture_output=True, text=True, timeout=timeout)
    return out.returncode, out.stdout + out.stderr


def test_reference_test_quantized(tc):
    rc, text = run_binary("test_quantized")
    assert rc == 0, text
    for marker in ("q4_0_gemv M=1 N=128 K=256", "q4_0_async M=1 N=128 K=256", "q8_0_gemv M=1 N=129 K=256",
                   "fused_rmsnorm_q4_0_gemv", "fused_rmsnorm_q8_0_gemv", "invalid quant size: 0 OK"):
        assert marker in text, (marker, text)


def test_reference_test_gguf(tc):
    rc, text = run_binary("test_gguf")
    assert rc == 0, text
    for marker in ("tensor       : name=weight.test", "gpu copy     : OK", "bulk load    : OK",
                   "gguf gemv    : OK", "test_gguf: OK"):
        assert marker in text, (marker, text)


def test_reference_test_fused_norm_gemv(tc):
    rc, text = run_binary("test_fused_norm_gemv")
    assert rc == 0, text


def test_reference_bench_inference_7b_runs(tc):
    """The reference's decode benchmark (tc_buffer_map'ed weights, 224 recorded GEMVs and one
    tc_stream_sync per token) completes and prints its result block."""
    rc, text = run_binary("bench_inference_7b", timeout=600)
    assert rc == 0, text
    assert "tok/s" in text or "tokens/s" in text or "Results" in text, text
    os.makedirs(os.path.join(ROOT, "gpurun_out"), exist_ok=True)
    with open(os.path.join(ROOT, "gpurun_out", "ref_bench_inference_7b.txt"), "w") as f:
        f.write(text)


BINDING_SCRIPT = r"""
import ctypes, os, struct, sys, tempfile
import numpy as np
import tensorcore as tc          # the reference's binding, unchanged; TENSORCORE_LIB selects this library

def dq4(raw, N, K):
    out = np.zeros((N, K), np.float32); nb = K // 32
    for n in range(N):
        for b in range(nb):
            blk = raw[(n * nb + b) * 18:(n * nb + b + 1) * 18]
            d = np.frombuffer(blk[:2], np.float16)[0].astype(np.float32)
            q = np.frombuffer(blk[2:], np.uint8)
            out[n, b * 32:b * 32 + 16] = ((q & 15).astype(np.float32) - 8) * d
            out[n, b * 32 + 16:b * 32 + 32] = ((q >> 4).astype(np.float32) - 8) * d
    return out

ctx = tc.init()
rng = np.random.default_rng(5)
M, N, K = 1, 96, 512
X = rng.standard_normal((M, K)).astype(np.float16)
W = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
gam = (1 + 0.1 * rng.standard_normal(K)).astype(np.float16)
nbytes = tc.quantized_size("q4_0", N, K)
assert nbytes == N * (K // 32) * 18 and tc.quantized_size("q8_0", N, K) == N * (K // 32) * 34
bx, bw, bq, by, bg = (tc.buffer_alloc(ctx, n) for n in (X.nbytes, W.nbytes, nbytes, M * N * 2, gam.nbytes))
tc.buffer_write(bx, X); tc.buffer_write(bw, W); tc.buffer_write(bg, gam)
tc.quantize_weights(ctx, bw, bq, "q4_0", N, K)
assert tc.last_backend_name() == "cuda", tc.last_backend_name()
Y = np.zeros((M, N), np.float16)
tc.gemv_quantized(ctx, bx, bq, by, "q4_0", M, N, K); tc.buffer_read(by, Y)
raw = ctypes.string_at(tc.buffer_map(bq), nbytes)
Wd = dq4(raw, N, K)
ref = X.astype(np.float32) @ Wd.T
assert np.abs(Y.astype(np.float32) - ref).max() < 2e-2, np.abs(Y.astype(np.float32) - ref).max()
st = tc.stream_create(ctx)
Y2 = np.zeros_like(Y)
tc.gemv_quantized_async(ctx, bx, bq, by, "q4_0", M, N, K, st); tc.stream_sync(st); tc.stream_destroy(ctx, st)
tc.buffer_read(by, Y2)
assert np.abs(Y2.astype(np.float32) - ref).max() < 2e-2
xf = X.astype(np.float32)
xn = xf / np.sqrt((xf ** 2).mean() + 1e-5) * gam.astype(np.float32)
tc.fused_rmsnorm_gemv_quantized(ctx, bx, bg, bq, by, "q4_0", M, N, K, 1e-5); tc.buffer_read(by, Y)
assert np.abs(Y.astype(np.float32) - xn @ Wd.T).max() < 3e-2
# dense fused norm + GEMV
Wk = (rng.standard_normal((K, N)) * 0.05).astype(np.float16)
bwk = tc.buffer_alloc(ctx, Wk.nbytes); tc.buffer_write(bwk, Wk)
tc.fused_rmsnorm_gemv(ctx, bx, bg, bwk, by, M, N, K, 1e-5); tc.buffer_read(by, Y)
assert np.abs(Y.astype(np.float32) - xn.astype(np.float16).astype(np.float32) @ Wk.astype(np.float32)).max() < 3e-2
# GGUF: a one-tensor Q4_0 file written here, loaded through the binding, used by a GEMV
def s(x): b = x.encode(); return struct.pack("<Q", len(b)) + b
path = os.path.join(tempfile.mkdtemp(), "t.gguf")
hdr = struct.pack("<IIQQ", 0x46554747, 3, 1, 2)
hdr += s("general.architecture") + struct.pack("<I", 8) + s("llama")
hdr += s("general.alignment") + struct.pack("<II", 4, 32)
hdr += s("w.weight") + struct.pack("<I", 2) + struct.pack("<QQ", K, N) + struct.pack("<IQ", 2, 0)
pad = (-len(hdr)) % 32
open(path, "wb").write(hdr + b"\0" * pad + raw)
g = tc.gguf_open(path)
assert tc.gguf_tensor_count(g) == 1
model = tc.gguf_load_supported_tensors(ctx, g)
assert tc.gguf_loaded_tensor_count(model) == 1
t = tc.gguf_loaded_get_tensor(model, "w.weight")
info = tc.gguf_loaded_tensor_quantized_matrix_info(t)
tc.gemv_quantized(ctx, bx, t["buffer"], by, "q4_0", M, N, K); tc.buffer_read(by, Y)
assert np.abs(Y.astype(np.float32) - ref).max() < 2e-2
tc.gguf_loaded_model_free(ctx, model); tc.gguf_close(g)
# dense GEMM (fp16 and bf16 storage), its recorded and batched forms
Mg, Ng, Kg = 136, 264, 320
Ag = rng.standard_normal((Mg, Kg)).astype(np.float16)
Bg = (rng.standard_normal((Kg, Ng)) * 0.05).astype(np.float16)
ba, bb, bc = (tc.buffer_alloc(ctx, n) for n in (Ag.nbytes, Bg.nbytes, Mg * Ng * 2))
tc.buffer_write(ba, Ag); tc.buffer_write(bb, Bg)
Cg = np.zeros((Mg, Ng), np.float16)
tc.gemm(ctx, ba, bb, bc, Mg, Ng, Kg); tc.buffer_read(bc, Cg)
refg = Ag.astype(np.float32) @ Bg.astype(np.float32)
assert np.abs(Cg.astype(np.float32) - refg).max() < 2e-2, np.abs(Cg.astype(np.float32) - refg).max()
assert tc.last_backend_name() == "cuda"
st = tc.stream_create(ctx)
tc.gemm_async(ctx, ba, bb, bc, Mg, Ng, Kg, st, alpha=0.5); tc.stream_sync(st); tc.stream_destroy(ctx, st)
tc.buffer_read(bc, Cg)
assert np.abs(Cg.astype(np.float32) - 0.5 * refg).max() < 2e-2
A2 = np.stack([Ag, -Ag]); B2 = np.stack([Bg, Bg])
ba2, bb2, bc2 = (tc.buffer_alloc(ctx, n) for n in (A2.nbytes, B2.nbytes, 2 * Mg * Ng * 2))
tc.buffer_write(ba2, A2); tc.buffer_write(bb2, B2)
C2 = np.zeros((2, Mg, Ng), np.float16)
tc.gemm_batched(ctx, ba2, bb2, bc2, 2, Mg, Ng, Kg); tc.buffer_read(bc2, C2)
assert np.abs(C2[0].astype(np.float32) - refg).max() < 2e-2 and np.abs(C2[1].astype(np.float32) + refg).max() < 2e-2
print("binding ok", info)
"""


def test_unchanged_reference_binding_drives_the_path(tc, tmp_path):
    """Quantise, GEMV (sync and recorded), fused RMSNorm GEMV, dense fused GEMV, the GGUF loader
    and the dense GEMM (plain, recorded, batched), called through the reference's own ctypes binding (python/tensorcore/__init__.py, not
    modified) with TENSORCORE_LIB pointing at this library - the operations that
    python/tests/test_basic.py:981-1026, 690-717 and 1040-1190 cover."""
    if not os.path.isdir(REF_PY):
        pytest.skip("the reference binding was not staged (no reference checkout when build() ran)")
    script = tmp_path / "drive.py"
    script.write_text(BINDING_SCRIPT)
    env = dict(os.environ, TENSORCORE_LIB=tc.LIB_PATH, PYTHONPATH=REF_PY)
    out = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "binding ok" in out.stdout
