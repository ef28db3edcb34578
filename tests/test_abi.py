"""CPU: the C-ABI library loads, exports every declared symbol, refuses to run without a
device, and its host-only parts (size arithmetic, string tables, the GGUF reader) behave as
the reference's do.  No compute call is made here."""
import ctypes
import os
import re
import struct

import numpy as np
import pytest

from conftest import GOLDEN, ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tensorcore_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(tcx?_[a-z0-9_]+)\s*\(", text))
    names.add("tensorcore_abi_version")
    return sorted(names)


def test_exports_every_declared_symbol(tc):
    L = tc.lib()
    declared = _declared_symbols()
    assert len(declared) > 60
    for name in declared:
        assert hasattr(L, name), name


def test_exports_the_reference_symbol_list(tc):
    L = tc.lib()
    names = open(os.path.join(GOLDEN, "reference_exports.txt")).read().split()
    assert len(names) == 126
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing
    assert ctypes.c_int.in_dll(L, "tensorcore_abi_version").value == 1


def test_reference_binding_imports_against_this_library(tc):
    """The unchanged reference ctypes binding resolves all its symbols at import."""
    ref_py = os.path.join(ROOT, "baseline", "_ref", "python")      # staged by build() from the checkout
    if not os.path.isdir(ref_py):
        ref_py = os.path.join(os.environ.get("TENSORCORE_REF") or os.path.join(ROOT, "..", "reference"), "python")
    if not os.path.isdir(ref_py):
        pytest.skip("no reference checkout on this machine and no staged copy of its binding")
    import subprocess
    import sys
    code = "import tensorcore as t; print(t.version()); print(t.quantized_size('q4_0', 4096, 4096))"
    env = dict(os.environ, TENSORCORE_LIB=tc.LIB_PATH, PYTHONPATH=ref_py)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["tensorcore", "0.1.22", "9437184"]


def test_string_tables(tc):
    # lib/core/status.c:3-20, lib/core/dtype.c:3-17, lib/core/device_cpu.cpp:61-76
    assert tc.version() == "tensorcore 0.1.22"
    assert tc.status_string(0) == "ok"
    assert tc.status_string(-3) == "no Metal device available"
    assert tc.status_string(-7) == "invalid argument"
    assert tc.status_string(12345) == "unknown status"
    assert tc.dtype_name(0) == "f16" and tc.dtype_name(2) == "f32" and tc.dtype_name(99) == "?"
    assert tc.backend_name(9) == "cuda" and tc.backend_name(7) == "portable_cpu"
    assert tc.backend_name(99) == "?"


def test_quantized_size_and_null_checks(tc):
    assert tc.quantized_size("q4_0", 4096, 4096) == 9437184
    assert tc.quantized_size("q8_0", 11008, 4096) == 47906816
    assert tc.quantized_size(5, 8, 32) == 0
    assert tc.quantized_size("q4_0", 8, 48) == 0
    assert tc.quantized_size("q4_0", -1, 32) == 0
    L = tc.lib()
    # ctx == NULL -> TC_ERR_NOT_INITIALIZED before anything else (quantized_cpu.cpp:108,171,243)
    assert L.tc_quantize_weights(None, None, None, 0, 1, 32) == -1
    assert L.tc_gemv_quantized(None, None, None, None, 0, 1, 1, 32) == -1
    assert L.tc_fused_rmsnorm_gemv_quantized(None, None, None, None, None, 0, 1, 1, 32, 1e-5) == -1
    assert L.tc_fused_rmsnorm_gemv(None, None, None, None, None, 1, 1, 32, 1e-5) == -1
    assert L.tc_fused_layernorm_gemv(None, None, None, None, None, None, 1, 1, 32, 1e-5) == -1
    # NULL stream is rejected first by the async form (quantized_cpu.cpp:331)
    assert L.tc_gemv_quantized_async(None, None, None, None, 0, 1, 1, 32, None) == -7
    assert L.tc_stream_sync(None) == -7
    assert L.tc_buffer_size(None) == 0
    assert L.tc_init(None) == -7


def test_no_device_means_failure_not_fallback(tc):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = ctypes.c_void_p()
    assert tc.lib().tc_init(ctypes.byref(h)) == tc.TC_ERR_NO_DEVICE
    assert not h.value
    assert tc.last_backend() == tc.TC_BACKEND_NONE


def test_stubs_report_unsupported(tc):
    L = tc.lib()
    for name in ("tc_attention_backward", "tc_rmsnorm_backward", "tc_adamw_step", "tc_conv2d_forward"):
        fn = getattr(L, name)
        fn.restype = ctypes.c_int
        assert fn() == tc.TC_ERR_UNSUPPORTED_FAMILY
    # entry points of the path answer a NULL context the way the reference does
    assert L.tc_rmsnorm_forward(None, None, None, None, None, 1, 32, 1e-5) == tc.TC_ERR_NOT_INITIALIZED
    assert L.tc_layernorm_forward(None, None, None, None, None, None, None, 1, 32, 1e-5) == tc.TC_ERR_NOT_INITIALIZED
    assert L.tc_swiglu_forward(None, None, None, None, 8) == tc.TC_ERR_NOT_INITIALIZED
    assert L.tc_rope_forward(None, None, None, None, 1, 1, 1, 2) == tc.TC_ERR_NOT_INITIALIZED
    assert L.tc_attention_forward(None, None, None, None, None, None, None) == tc.TC_ERR_NOT_INITIALIZED
    assert L.tc_gemm(None, None, None, None, None) == tc.TC_ERR_NOT_INITIALIZED
    assert L.tc_gemm_batched(None, None, None, None, None) == tc.TC_ERR_NOT_INITIALIZED
    assert L.tc_gemm_async(None, None, None, None, None, None) == tc.TC_ERR_INVALID_ARG      # NULL stream first
    assert L.tc_dist_init(None, 0, 1, 0, None, None) == tc.TC_ERR_NOT_INITIALIZED
    assert L.tc_allreduce(None, None, 0, 2, 0) == tc.TC_ERR_INVALID_ARG and L.tc_barrier(None) == tc.TC_ERR_INVALID_ARG
    assert L.tc_dist_world_size(None) == 0


# ---- GGUF reader (host only) ------------------------------------------------------------
def _write_reference_style_file(path):
    """The structure tests/test_gguf.c:72-124 writes: scalar and array metadata, one Q4_0
    [K=32,N=1] tensor (scale 0x3800, sixteen 0xAB bytes) and one tensor of unknown type."""
    from tensorcore_b200 import gguf_writer as gw
    meta = [
        ("general.architecture", gw.STRING, "llama"),
        ("general.name", gw.STRING, "unit"),
        ("llama.context_length", gw.U32, 2048),
        ("llama.embedding_length", gw.U32, 64),
        ("llama.feed_forward_length", gw.U32, 128),
        ("llama.block_count", gw.U32, 2),
        ("llama.attention.head_count", gw.U32, 4),
        ("llama.rope.dimension_count", gw.U32, 16),
        ("llama.attention.layer_norm_rms_epsilon", gw.F32, 1e-6),
        ("llama.rope.freq_base", gw.F32, 500000.0),
        ("tokenizer.ggml.tokens", gw.ARRAY, ["<s>", "</s>", "hello"], gw.STRING),
        ("tokenizer.ggml.scores", gw.ARRAY, [0.5, -1.0, 2.25], gw.F32),
        ("tokenizer.ggml.token_type", gw.ARRAY, [1, 2, 3], gw.I32),
        ("flag", gw.BOOL, 1),
    ]
    blk = struct.pack("<H", 0x3800) + bytes([0xAB] * 16)
    tensors = [gw.TensorSpec("weight.test", [32, 1], gw.GGML_Q4_0, 18, data=blk),
               gw.TensorSpec("unsupported.test", [32], 999, 0, data=b"")]
    gw.write_gguf(path, meta, tensors)


def test_gguf_reader_metadata_and_tensor_table(tc, tmp_path):
    path = str(tmp_path / "unit.gguf")
    _write_reference_style_file(path)
    with tc.GgufFile(path) as g:
        assert g.tensor_count() == 2 and g.metadata_count() == 14
        assert g.meta_get_str("general.architecture") == "llama"
        assert g.meta_get_str("llama.block_count") is None
        assert g.meta_get_i64("llama.block_count") == 2
        assert g.meta_get_i64("missing", 7) == 7
        assert g.meta_get_i64("flag", 9) == 9            # bool is not an integer scalar
        assert abs(g.meta_get_f64("llama.rope.freq_base") - 500000.0) < 1e-3
        assert g.meta_get_f64("llama.block_count") == 2.0
        assert g.meta_array_count("tokenizer.ggml.tokens") == 3
        assert g.meta_array_get_str("tokenizer.ggml.tokens", 2) == "hello"
        assert tc.gguf_meta_array_get_f64(g, "tokenizer.ggml.scores", 2) == 2.25
        assert tc.gguf_meta_array_get_i64(g, "tokenizer.ggml.token_type", 1) == 2
        assert tc.gguf_meta_array_get_i64(g, "tokenizer.ggml.scores", 1, -5) == -5
        with pytest.raises(tc.TensorcoreError):
            g.meta_array_get_str("tokenizer.ggml.tokens", 3)
        cfg = g.llama_config()
        assert cfg["embedding_length"] == 64 and cfg["block_count"] == 2
        assert cfg["attention_head_count_kv"] == 4      # defaults to head_count
        assert cfg["vocab_size"] == 3 and cfg["rope_freq_scale"] == 1.0
        t = g.get_tensor("weight.test")
        assert t["dims"] == [32, 1] and t["type"] == tc.TC_GGUF_TYPE_Q4_0 and t["n_bytes"] == 18
        assert ctypes.string_at(t["data"], 18) == struct.pack("<H", 0x3800) + bytes([0xAB] * 16)
        u = g.tensor_at(1)
        assert u["type"] == tc.TC_GGUF_TYPE_UNSUPPORTED and u["n_bytes"] == 0
        mi = tc.gguf_tensor_quantized_matrix_info(g, "weight.test")
        assert (mi["N"], mi["K"], mi["quant_type"], mi["n_bytes"]) == (1, 32, 0, 18)
        with pytest.raises(tc.TensorcoreError):
            g.get_tensor("nope")


def test_gguf_reader_rejects_malformed_files(tc, tmp_path):
    good = str(tmp_path / "good.gguf")
    _write_reference_style_file(good)
    raw = open(good, "rb").read()
    cases = {
        "magic": b"XXXX" + raw[4:],
        "version": raw[:4] + struct.pack("<I", 2) + raw[8:],
        "truncated": raw[:len(raw) - 10],
        "huge_count": raw[:8] + struct.pack("<Q", 1 << 60) + raw[16:],
        "empty": b"",
    }
    for name, data in cases.items():
        p = str(tmp_path / f"{name}.gguf")
        open(p, "wb").write(data)
        with pytest.raises(tc.TensorcoreError) as e:
            tc.gguf_open(p)
        assert e.value.status == tc.TC_ERR_INTERNAL, name
    with pytest.raises(tc.TensorcoreError):
        tc.gguf_open(str(tmp_path / "does-not-exist.gguf"))


def test_gguf_alignment_key_moves_the_data_start(tc, tmp_path):
    from tensorcore_b200 import gguf_writer as gw
    p = str(tmp_path / "al.gguf")
    a = np.arange(64, dtype=np.float32)
    b = np.arange(8, dtype=np.float16)
    gw.write_gguf(p, [("general.architecture", gw.STRING, "x")],
                  [gw.TensorSpec("a", [64], gw.GGML_F32, 256, data=a),
                   gw.TensorSpec("b", [8], gw.GGML_F16, 16, data=b)], alignment=128)
    with tc.GgufFile(p) as g:
        ta, tb = g.get_tensor("a"), g.get_tensor("b")
        assert ta["offset"] == 0 and tb["offset"] == 256
        got = np.frombuffer(ctypes.string_at(tb["data"], 16), dtype=np.float16)
        assert np.array_equal(got, b)
        assert ta["data"] % 128 == (ta["data"] - 0) % 128  # pointer arithmetic only
