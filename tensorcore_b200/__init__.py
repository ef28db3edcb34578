"""Python binding of the B200 tensorcore library for the quantized-decode path.

Mirrors the names and argument order of the reference's ctypes binding
(python/tensorcore/__init__.py) for the operations this library implements - ``init``,
``buffer_*``, ``stream_*``, ``quantized_size``, ``quantize_weights``, ``gemv_quantized``,
``gemv_quantized_async``, ``fused_rmsnorm_gemv_quantized``, ``fused_rmsnorm_gemv``,
``fused_layernorm_gemv``, ``gguf_*`` and the ``Context`` / ``Buffer`` / ``Stream`` /
``GgufFile`` / ``LoadedModel`` / ``QuantizedMatrix`` wrappers - so code and tests written for the
reference binding read the same here.  Everything is a thin call into ``libtensorcore.so``
(built from ``tensorcore_b200/csrc``); nothing is computed in Python and there is no fallback:
if the library is missing or no sm_100 device is present the calls raise.

Additive ``*_ex`` / ``raw_*`` functions expose the library's fp32-activation forms and raw
device-pointer launches.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, byref, c_bool, c_char, c_char_p, c_double, c_float, c_int,
                    c_int32, c_int64, c_size_t, c_uint32, c_uint64, c_void_p)

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TENSORCORE_LIB") or os.path.join(_HERE, "lib", "libtensorcore.so")

# status codes (include/tensorcore/status.h:8-22)
TC_OK = 0
TC_ERR_NOT_INITIALIZED = -1
TC_ERR_ALREADY_INITIALIZED = -2
TC_ERR_NO_DEVICE = -3
TC_ERR_UNSUPPORTED_FAMILY = -4
TC_ERR_UNSUPPORTED_DTYPE = -5
TC_ERR_INVALID_SHAPE = -6
TC_ERR_INVALID_ARG = -7
TC_ERR_ALLOC = -8
TC_ERR_DISPATCH = -11
TC_ERR_INTERNAL = -99

TC_DTYPE_F16, TC_DTYPE_BF16, TC_DTYPE_F32 = 0, 1, 2
TC_QUANT_Q4_0, TC_QUANT_Q8_0 = 0, 1
TC_BACKEND_NONE, TC_BACKEND_PORTABLE_CPU, TC_BACKEND_CUDA = 0, 7, 9
TC_GGUF_TYPE_F32, TC_GGUF_TYPE_F16, TC_GGUF_TYPE_Q4_0, TC_GGUF_TYPE_Q4_1 = 0, 1, 2, 3
TC_GGUF_TYPE_Q8_0, TC_GGUF_TYPE_BF16, TC_GGUF_TYPE_UNSUPPORTED = 8, 30, -1


class TCDeviceInfo(Structure):
    _fields_ = [("family", c_int), ("name", c_char * 128), ("max_buffer_bytes", c_uint64),
                ("recommended_working_set_bytes", c_uint64), ("max_threadgroup_memory", c_uint32),
                ("max_threads_per_threadgroup", c_uint32), ("thread_execution_width", c_uint32),
                ("unified_memory", c_bool), ("supports_bf16_simdgroup", c_bool),
                ("supports_i8_simdgroup", c_bool), ("supports_tensorops_m5", c_bool),
                ("supports_fp64_native", c_bool)]


class TCCudaDeviceInfo(Structure):
    _fields_ = [("device_name", c_char * 128), ("compute_capability", c_char * 16),
                ("major", c_int), ("minor", c_int), ("global_memory_bytes", c_uint64),
                ("shared_memory_per_block", c_uint64), ("multiprocessor_count", c_uint32),
                ("max_threads_per_block", c_uint32), ("warp_size", c_uint32),
                ("supports_fp16", c_bool), ("supports_bf16", c_bool),
                ("supports_int8_tensor_core", c_bool), ("supports_tf32", c_bool),
                ("unified_memory", c_bool)]


class TCGGufTensorInfo(Structure):
    _fields_ = [("name", c_char_p), ("n_dims", c_int32), ("dims", c_uint64 * 4), ("type", c_int),
                ("offset", c_uint64), ("n_bytes", c_size_t), ("data", c_void_p)]


class TCGGufLoadedTensorInfo(Structure):
    _fields_ = [("name", c_char_p), ("n_dims", c_int32), ("dims", c_uint64 * 4), ("type", c_int),
                ("offset", c_uint64), ("n_bytes", c_size_t), ("buffer", c_void_p)]


class TCGGufLlamaConfig(Structure):
    _fields_ = [(n, c_int64) for n in ("context_length", "embedding_length", "feed_forward_length",
                                       "block_count", "attention_head_count",
                                       "attention_head_count_kv", "rope_dimension_count",
                                       "vocab_size")] + \
               [(n, c_double) for n in ("rms_norm_epsilon", "rope_freq_base", "rope_freq_scale")]


class TCGGufQuantizedMatrixInfo(Structure):
    _fields_ = [("N", c_int), ("K", c_int), ("gguf_type", c_int), ("quant_type", c_int),
                ("n_bytes", c_size_t), ("buffer", c_void_p)]


class TCXDecodeOp(Structure):
    _fields_ = [("W", c_void_p), ("X", c_void_p), ("Y", c_void_p), ("gamma", c_void_p),
                ("N", c_int), ("K", c_int), ("x_dtype", c_int), ("y_dtype", c_int),
                ("eps", c_float)]


class TCXDecodeTpOp(Structure):
    _fields_ = [("op", TCXDecodeOp), ("peers", c_int), ("y_row0", c_int), ("y_rows", c_int),
                ("layout_rows", c_int), ("expect", c_int)]


DECODE_STATIC_MAX_OPS = 256


class TensorcoreError(RuntimeError):
    def __init__(self, status: int):
        self.status = int(status)
        super().__init__(f"tensorcore error {self.status}: {status_string(self.status)}")


_lib = None


def lib() -> ctypes.CDLL:
    """Loads libtensorcore.so on first use.  A missing library is an error, never a fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m tensorcore_b200.build` "
                "(nvcc, sm_100a); there is no CPU fallback")
        _lib = ctypes.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(L) -> None:
    vp, i, sz, f = c_void_p, c_int, c_size_t, c_float

    def sig(name, res, *args):
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = list(args)

    sig("tc_init", i, POINTER(vp))
    sig("tc_shutdown", i, vp)
    sig("tc_device_info_get", i, vp, POINTER(TCDeviceInfo))
    sig("tc_version", c_char_p)
    sig("tc_status_string", c_char_p, i)
    sig("tc_dtype_name", c_char_p, i)
    sig("tc_backend_name", c_char_p, i)
    sig("tc_last_backend", i)
    sig("tc_cuda_last_kernel_name", c_char_p)
    sig("tc_cuda_device_count", i)
    sig("tc_cuda_device_at", i, i, POINTER(TCCudaDeviceInfo))
    sig("tc_cuda_select_device", i, vp, i)
    sig("tc_cuda_init", i, vp)
    sig("tc_buffer_alloc", i, vp, sz, POINTER(vp))
    sig("tc_buffer_from_ptr", i, vp, vp, sz, POINTER(vp))
    sig("tc_buffer_free", i, vp, vp)
    sig("tc_buffer_map", i, vp, POINTER(vp))
    sig("tc_buffer_size", sz, vp)
    sig("tc_stream_create", i, vp, POINTER(vp))
    sig("tc_stream_destroy", i, vp, vp)
    sig("tc_stream_sync", i, vp)
    sig("tc_quantized_size", sz, i, i, i)
    sig("tc_quantize_weights", i, vp, vp, vp, i, i, i)
    sig("tc_gemv_quantized", i, vp, vp, vp, vp, i, i, i, i)
    sig("tc_gemv_quantized_async", i, vp, vp, vp, vp, i, i, i, i, vp)
    sig("tc_fused_rmsnorm_gemv_quantized", i, vp, vp, vp, vp, vp, i, i, i, i, f)
    sig("tc_fused_rmsnorm_gemv", i, vp, vp, vp, vp, vp, i, i, i, f)
    sig("tc_fused_layernorm_gemv", i, vp, vp, vp, vp, vp, vp, i, i, i, f)
    sig("tc_dist_init", i, vp, i, i, i, c_char_p, POINTER(vp))
    sig("tc_dist_finalize", i, vp)
    sig("tc_dist_world_size", i, vp)
    sig("tc_dist_rank", i, vp)
    sig("tc_allreduce", i, vp, vp, sz, i, i)
    sig("tc_broadcast", i, vp, vp, sz, i, i)
    sig("tc_allgather", i, vp, vp, vp, sz, i)
    sig("tc_barrier", i, vp)
    sig("tc_rmsnorm_forward", i, vp, vp, vp, vp, vp, i, i, f)
    sig("tc_layernorm_forward", i, vp, vp, vp, vp, vp, vp, vp, i, i, f)
    sig("tc_swiglu_forward", i, vp, vp, vp, vp, i)
    sig("tc_rope_forward", i, vp, vp, vp, vp, i, i, i, i)
    sig("tc_attention_forward", i, vp, vp, vp, vp, vp, vp, vp)
    sig("tc_attention_forward_async", i, vp, vp, vp, vp, vp, vp, vp, vp)
    # GGUF
    sig("tc_gguf_open", i, c_char_p, POINTER(vp))
    sig("tc_gguf_close", None, vp)
    sig("tc_gguf_tensor_count", c_uint64, vp)
    sig("tc_gguf_metadata_count", c_uint64, vp)
    sig("tc_gguf_get_tensor", i, vp, c_char_p, POINTER(TCGGufTensorInfo))
    sig("tc_gguf_tensor_at", i, vp, c_uint64, POINTER(TCGGufTensorInfo))
    sig("tc_gguf_meta_get_str", c_char_p, vp, c_char_p)
    sig("tc_gguf_meta_get_i64", c_int64, vp, c_char_p, c_int64)
    sig("tc_gguf_meta_get_f64", c_double, vp, c_char_p, c_double)
    sig("tc_gguf_meta_array_count", c_uint64, vp, c_char_p)
    sig("tc_gguf_meta_array_get_str", i, vp, c_char_p, c_uint64, POINTER(vp), POINTER(sz))
    sig("tc_gguf_meta_array_get_i64", c_int64, vp, c_char_p, c_uint64, c_int64)
    sig("tc_gguf_meta_array_get_f64", c_double, vp, c_char_p, c_uint64, c_double)
    sig("tc_gguf_get_llama_config", i, vp, POINTER(TCGGufLlamaConfig))
    sig("tc_gguf_tensor_to_buffer", i, vp, vp, c_char_p, POINTER(vp))
    sig("tc_gguf_tensor_quantized_matrix_info", i, POINTER(TCGGufTensorInfo),
        POINTER(TCGGufQuantizedMatrixInfo))
    sig("tc_gguf_loaded_tensor_quantized_matrix_info", i, POINTER(TCGGufLoadedTensorInfo),
        POINTER(TCGGufQuantizedMatrixInfo))
    sig("tc_gguf_load_supported_tensors", i, vp, vp, POINTER(vp))
    sig("tc_gguf_loaded_model_free", None, vp, vp)
    sig("tc_gguf_loaded_tensor_count", c_uint64, vp)
    sig("tc_gguf_loaded_skipped_tensor_count", c_uint64, vp)
    sig("tc_gguf_loaded_tensor_at", i, vp, c_uint64, POINTER(TCGGufLoadedTensorInfo))
    sig("tc_gguf_loaded_get_tensor", i, vp, c_char_p, POINTER(TCGGufLoadedTensorInfo))
    # additive entry points
    sig("tcx_gemv_quantized_ex", i, vp, vp, vp, vp, i, i, i, i, i, i, vp)
    sig("tcx_fused_rmsnorm_gemv_quantized_ex", i, vp, vp, vp, vp, vp, i, i, i, i, f, i, i, vp)
    sig("tcx_buffer_upload", i, vp, sz, vp, sz)
    sig("tcx_buffer_download", i, vp, sz, vp, sz)
    sig("tcx_buffer_device_ptr", i, vp, POINTER(vp))
    sig("tcx_stream_cuda_handle", i, vp, POINTER(vp))
    sig("tcx_stream_flush", i, vp)
    sig("tcx_stream_set_persistent", i, vp, i)
    sig("tcx_stream_tp_export", i, vp, sz, vp)
    sig("tcx_stream_tp_connect", i, vp, i, i, vp)
    sig("tcx_stream_decode_tp", i, vp, POINTER(TCXDecodeTpOp), i)
    sig("tcx_raw_quantize_weights", i, vp, vp, vp, i, i, i, vp)
    sig("tcx_raw_gemv_quantized", i, vp, vp, vp, vp, i, i, i, i, i, i, vp)
    sig("tcx_raw_fused_rmsnorm_gemv_quantized", i, vp, vp, vp, vp, vp, i, i, i, i, f, i, i, vp)
    sig("tcx_raw_fused_norm_gemv_f16", i, vp, vp, vp, vp, vp, vp, i, i, i, f, vp)
    sig("tcx_raw_decode_q4_static", i, vp, POINTER(TCXDecodeOp), i, vp)
    sig("tcx_set_gemv_variant", i, c_char_p)
    sig("tcx_take_device_error", c_uint32, vp)
    sig("tcx_launch_count", c_uint64)


def _check(status: int) -> None:
    if status != TC_OK:
        raise TensorcoreError(status)


def _h(x):
    """Handle of a wrapper object or a raw handle."""
    return getattr(x, "handle", x)


def _quant(fmt) -> int:
    if isinstance(fmt, str):
        table = {"q4_0": TC_QUANT_Q4_0, "q8_0": TC_QUANT_Q8_0}
        if fmt.lower() not in table:
            raise ValueError(f"unknown quant format {fmt!r}")
        return table[fmt.lower()]
    return int(fmt)


def _dtype(d) -> int:
    if isinstance(d, str):
        return {"f16": TC_DTYPE_F16, "bf16": TC_DTYPE_BF16, "f32": TC_DTYPE_F32}[d.lower()]
    return int(d)


# ----------------------------------------------------------------------------------------
# Functional API (names as in the reference binding)
# ----------------------------------------------------------------------------------------
def version() -> str:
    return lib().tc_version().decode()


def status_string(status: int) -> str:
    return lib().tc_status_string(int(status)).decode()


def dtype_name(d: int) -> str:
    return lib().tc_dtype_name(int(d)).decode()


def backend_name(b: int) -> str:
    return lib().tc_backend_name(int(b)).decode()


def last_backend() -> int:
    return int(lib().tc_last_backend())


def last_backend_name() -> str:
    return backend_name(last_backend())


def cuda_last_kernel_name() -> str:
    return lib().tc_cuda_last_kernel_name().decode()


def cuda_device_count() -> int:
    return int(lib().tc_cuda_device_count())


def cuda_select_device(ctx, index: int) -> None:
    _check(lib().tc_cuda_select_device(_h(ctx), int(index)))


def init():
    ctx = c_void_p()
    st = lib().tc_init(byref(ctx))
    if st not in (TC_OK, TC_ERR_ALREADY_INITIALIZED):
        raise TensorcoreError(st)
    return ctx


def shutdown(ctx) -> None:
    _check(lib().tc_shutdown(_h(ctx)))


def device_info(ctx) -> TCDeviceInfo:
    info = TCDeviceInfo()
    _check(lib().tc_device_info_get(_h(ctx), byref(info)))
    return info


def buffer_alloc(ctx, nbytes: int):
    out = c_void_p()
    _check(lib().tc_buffer_alloc(_h(ctx), int(nbytes), byref(out)))
    return out


def buffer_from_ptr(ctx, ptr: int, nbytes: int):
    out = c_void_p()
    _check(lib().tc_buffer_from_ptr(_h(ctx), c_void_p(int(ptr)), int(nbytes), byref(out)))
    return out


def buffer_free(ctx, buf) -> None:
    _check(lib().tc_buffer_free(_h(ctx), _h(buf)))


def buffer_map(buf) -> int:
    p = c_void_p()
    _check(lib().tc_buffer_map(_h(buf), byref(p)))
    return p.value


def buffer_size(buf) -> int:
    return int(lib().tc_buffer_size(_h(buf)))


def buffer_write(buf, arr: np.ndarray) -> None:
    """Copies `arr` into the buffer through tc_buffer_map (python/tensorcore/__init__.py:1153)."""
    a = np.ascontiguousarray(arr)
    if a.nbytes > buffer_size(buf):
        raise ValueError("array larger than buffer")
    ctypes.memmove(buffer_map(buf), a.ctypes.data, a.nbytes)


def buffer_read(buf, arr: np.ndarray) -> np.ndarray:
    """Copies the buffer's leading bytes into `arr` through tc_buffer_map (ibid. :1165)."""
    if not arr.flags["C_CONTIGUOUS"]:
        raise ValueError("destination must be contiguous")
    if arr.nbytes > buffer_size(buf):
        raise ValueError("array larger than buffer")
    ctypes.memmove(arr.ctypes.data, buffer_map(buf), arr.nbytes)
    return arr


def buffer_upload(buf, arr: np.ndarray, offset: int = 0) -> None:
    a = np.ascontiguousarray(arr)
    _check(lib().tcx_buffer_upload(_h(buf), int(offset), c_void_p(a.ctypes.data), a.nbytes))


def buffer_download(buf, arr: np.ndarray, offset: int = 0) -> np.ndarray:
    assert arr.flags["C_CONTIGUOUS"]
    _check(lib().tcx_buffer_download(_h(buf), int(offset), c_void_p(arr.ctypes.data), arr.nbytes))
    return arr


def buffer_device_ptr(buf) -> int:
    p = c_void_p()
    _check(lib().tcx_buffer_device_ptr(_h(buf), byref(p)))
    return p.value or 0


def stream_create(ctx):
    out = c_void_p()
    _check(lib().tc_stream_create(_h(ctx), byref(out)))
    return out


def stream_sync(stream) -> None:
    _check(lib().tc_stream_sync(_h(stream)))


def stream_flush(stream) -> None:
    _check(lib().tcx_stream_flush(_h(stream)))


def stream_destroy(ctx, stream) -> None:
    _check(lib().tc_stream_destroy(_h(ctx), _h(stream)))


def stream_cuda_handle(stream) -> int:
    p = c_void_p()
    _check(lib().tcx_stream_cuda_handle(_h(stream), byref(p)))
    return p.value or 0


def quantized_size(fmt, N: int, K: int) -> int:
    return int(lib().tc_quantized_size(_quant(fmt), int(N), int(K)))


def quantize_weights(ctx, W_fp16, W_quant, fmt, N, K) -> None:
    _check(lib().tc_quantize_weights(_h(ctx), _h(W_fp16), _h(W_quant), _quant(fmt), int(N), int(K)))


def gemv_quantized(ctx, X, W_quant, Y, fmt, M, N, K) -> None:
    _check(lib().tc_gemv_quantized(_h(ctx), _h(X), _h(W_quant), _h(Y), _quant(fmt), int(M), int(N),
                                   int(K)))


def gemv_quantized_async(ctx, X, W_quant, Y, fmt, M, N, K, stream) -> None:
    _check(lib().tc_gemv_quantized_async(_h(ctx), _h(X), _h(W_quant), _h(Y), _quant(fmt), int(M),
                                         int(N), int(K), _h(stream)))


def fused_rmsnorm_gemv_quantized(ctx, X, gamma, W_quant, Y, fmt, M, N, K, eps=1e-5) -> None:
    _check(lib().tc_fused_rmsnorm_gemv_quantized(_h(ctx), _h(X), _h(gamma), _h(W_quant), _h(Y),
                                                 _quant(fmt), int(M), int(N), int(K), float(eps)))


def fused_rmsnorm_gemv(ctx, X, gamma, W, Y, M, N, K, eps=1e-5) -> None:
    _check(lib().tc_fused_rmsnorm_gemv(_h(ctx), _h(X), _h(gamma), _h(W), _h(Y), int(M), int(N),
                                       int(K), float(eps)))


def fused_layernorm_gemv(ctx, X, gamma, beta, W, Y, M, N, K, eps=1e-5) -> None:
    _check(lib().tc_fused_layernorm_gemv(_h(ctx), _h(X), _h(gamma), _h(beta), _h(W), _h(Y), int(M),
                                         int(N), int(K), float(eps)))


TC_DIST_SINGLE, TC_DIST_RING, TC_DIST_GLOO = 0, 1, 2
_REDUCE = {"sum": 0, "avg": 1, "max": 2, "min": 3}


class DistContext:
    """Mirror of the reference binding's DistContext: collectives among one process per GPU."""

    def __init__(self, ctx, backend=TC_DIST_SINGLE, world_size=1, rank=0, rendezvous_url=None):
        h = c_void_p()
        _check(lib().tc_dist_init(_h(ctx), int(backend), int(world_size), int(rank),
                                  rendezvous_url.encode() if rendezvous_url else None, byref(h)))
        self.handle = h

    def world_size(self) -> int:
        return int(lib().tc_dist_world_size(self.handle))

    def rank(self) -> int:
        return int(lib().tc_dist_rank(self.handle))

    def allreduce(self, buf, num_elements, dtype="f32", op="sum") -> None:
        _check(lib().tc_allreduce(self.handle, _h(buf), int(num_elements), _dtype(dtype), _REDUCE[op]))

    def broadcast(self, buf, num_elements, dtype="f32", root=0) -> None:
        _check(lib().tc_broadcast(self.handle, _h(buf), int(num_elements), _dtype(dtype), int(root)))

    def allgather(self, src, dst, num_elements_per_rank, dtype="f32") -> None:
        _check(lib().tc_allgather(self.handle, _h(src), _h(dst), int(num_elements_per_rank), _dtype(dtype)))

    def barrier(self) -> None:
        _check(lib().tc_barrier(self.handle))

    def close(self) -> None:
        if self.handle is not None:
            lib().tc_dist_finalize(self.handle)
            self.handle = None


def rmsnorm_forward(ctx, X, gamma, Y, rstd_out, N, D, eps=1e-5) -> None:
    _check(lib().tc_rmsnorm_forward(_h(ctx), _h(X), _h(gamma), _h(Y), _h(rstd_out), int(N), int(D), float(eps)))


def layernorm_forward(ctx, X, gamma, beta, Y, mean_out, rstd_out, N, D, eps=1e-5) -> None:
    _check(lib().tc_layernorm_forward(_h(ctx), _h(X), _h(gamma), _h(beta), _h(Y), _h(mean_out), _h(rstd_out),
                                      int(N), int(D), float(eps)))


def swiglu_forward(ctx, gate, up, out, n) -> None:
    _check(lib().tc_swiglu_forward(_h(ctx), _h(gate), _h(up), _h(out), int(n)))


def rope_forward(ctx, X, cos_t, sin_t, batch, heads, seq, head_dim) -> None:
    _check(lib().tc_rope_forward(_h(ctx), _h(X), _h(cos_t), _h(sin_t), int(batch), int(heads), int(seq),
                                 int(head_dim)))


class TCGemmDesc(Structure):          # tc_gemm_desc
    _fields_ = [("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32), ("a_dtype", c_int),
                ("b_dtype", c_int), ("c_dtype", c_int), ("accum_dtype", c_int), ("transpose_a", ctypes.c_bool),
                ("transpose_b", ctypes.c_bool), ("alpha", c_float), ("beta", c_float), ("lda", ctypes.c_int32),
                ("ldb", ctypes.c_int32), ("ldc", ctypes.c_int32)]


def gemm(ctx, A, B, C, M, N, K, dtype="f16", accum="f32", transpose_a=False, transpose_b=False, alpha=1.0,
         beta=0.0, lda=0, ldb=0, ldc=0) -> None:
    """C = alpha * op(A) . op(B) + beta * C, row-major (tc_gemm; same arguments as the reference binding)."""
    d = TCGemmDesc(int(M), int(N), int(K), _dtype(dtype), _dtype(dtype), _dtype(dtype), _dtype(accum),
                   bool(transpose_a), bool(transpose_b), float(alpha), float(beta), int(lda), int(ldb), int(ldc))
    _check(lib().tc_gemm(_h(ctx), byref(d), _h(A), _h(B), _h(C)))


class TCGemmBatchedDesc(Structure):   # tc_gemm_batched_desc
    _fields_ = [("base", TCGemmDesc), ("batch", ctypes.c_int32), ("stride_a", ctypes.c_int64),
                ("stride_b", ctypes.c_int64), ("stride_c", ctypes.c_int64)]


def gemm_batched(ctx, A, B, C, M, N, K, batch, stride_a, stride_b, stride_c, dtype="f16", accum="f32",
                 transpose_a=False, transpose_b=False, alpha=1.0, beta=0.0, lda=0, ldb=0, ldc=0) -> None:
    """`batch` products of one shape, consecutive matrices stride_* elements apart (tc_gemm_batched)."""
    d = TCGemmBatchedDesc(TCGemmDesc(int(M), int(N), int(K), _dtype(dtype), _dtype(dtype), _dtype(dtype), _dtype(accum),
                                     bool(transpose_a), bool(transpose_b), float(alpha), float(beta), int(lda), int(ldb),
                                     int(ldc)), int(batch), int(stride_a), int(stride_b), int(stride_c))
    _check(lib().tc_gemm_batched(_h(ctx), byref(d), _h(A), _h(B), _h(C)))


class TCAttentionDesc(Structure):     # tc_attention_desc
    _fields_ = [("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("seq_q", ctypes.c_int32),
                ("seq_kv", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("io_dtype", c_int),
                ("accum_dtype", c_int), ("softmax_scale", c_float), ("causal", ctypes.c_bool),
                ("return_lse", ctypes.c_bool), ("kv_heads", ctypes.c_int32), ("window_size", ctypes.c_int32),
                ("alibi_slopes", c_void_p)]


def _attention_desc(batch, heads, seq_q, seq_kv, head_dim, dtype, accum, softmax_scale, causal, return_lse,
                    kv_heads, window_size, alibi_slopes):
    slopes = None
    if alibi_slopes is not None:
        slopes = (c_float * int(heads))(*[float(v) for v in alibi_slopes])
    d = TCAttentionDesc(int(batch), int(heads), int(seq_q), int(seq_kv), int(head_dim), _dtype(dtype), _dtype(accum),
                        float(softmax_scale or 0.0), bool(causal), bool(return_lse), int(kv_heads), int(window_size),
                        ctypes.cast(slopes, c_void_p) if slopes is not None else None)
    return d, slopes


def attention_forward(ctx, Q, K, V, O, batch, heads, seq_q, seq_kv, head_dim, LSE=None, dtype="f16", accum="f32",
                      softmax_scale=None, causal=True, return_lse=False, kv_heads=0, window_size=0,
                      alibi_slopes=None) -> None:
    """Scaled-dot-product attention forward (same arguments as the reference binding)."""
    return_lse = bool(return_lse or LSE is not None)
    desc, slopes = _attention_desc(batch, heads, seq_q, seq_kv, head_dim, dtype, accum, softmax_scale, causal,
                                   return_lse, kv_heads, window_size, alibi_slopes)
    _check(lib().tc_attention_forward(_h(ctx), byref(desc), _h(Q), _h(K), _h(V), _h(O),
                                      _h(LSE) if LSE is not None else None))
    _ = slopes


def attention_forward_async(ctx, Q, K, V, O, batch, heads, seq_q, seq_kv, head_dim, stream, LSE=None, dtype="f16",
                            accum="f32", softmax_scale=None, causal=True, return_lse=False, kv_heads=0,
                            window_size=0, alibi_slopes=None) -> None:
    return_lse = bool(return_lse or LSE is not None)
    desc, slopes = _attention_desc(batch, heads, seq_q, seq_kv, head_dim, dtype, accum, softmax_scale, causal,
                                   return_lse, kv_heads, window_size, alibi_slopes)
    _check(lib().tc_attention_forward_async(_h(ctx), byref(desc), _h(Q), _h(K), _h(V), _h(O),
                                            _h(LSE) if LSE is not None else None, _h(stream)))
    _ = slopes


def gemv_quantized_ex(ctx, X, W_quant, Y, fmt, M, N, K, x_dtype="f16", y_dtype="f16",
                      stream=None) -> None:
    _check(lib().tcx_gemv_quantized_ex(_h(ctx), _h(X), _h(W_quant), _h(Y), _quant(fmt), int(M),
                                       int(N), int(K), _dtype(x_dtype), _dtype(y_dtype),
                                       _h(stream) if stream is not None else None))


def fused_rmsnorm_gemv_quantized_ex(ctx, X, gamma, W_quant, Y, fmt, M, N, K, eps=1e-5,
                                    x_dtype="f16", y_dtype="f16", stream=None) -> None:
    _check(lib().tcx_fused_rmsnorm_gemv_quantized_ex(
        _h(ctx), _h(X), _h(gamma), _h(W_quant), _h(Y), _quant(fmt), int(M), int(N), int(K),
        float(eps), _dtype(x_dtype), _dtype(y_dtype), _h(stream) if stream is not None else None))


def raw_quantize_weights(ctx, W_fp16_ptr, W_quant_ptr, fmt, N, K, cuda_stream=0) -> None:
    _check(lib().tcx_raw_quantize_weights(_h(ctx), c_void_p(W_fp16_ptr), c_void_p(W_quant_ptr),
                                          _quant(fmt), int(N), int(K), c_void_p(cuda_stream)))


def raw_gemv_quantized(ctx, X_ptr, W_ptr, Y_ptr, fmt, M, N, K, x_dtype="f16", y_dtype="f16",
                       cuda_stream=0) -> None:
    _check(lib().tcx_raw_gemv_quantized(_h(ctx), c_void_p(X_ptr), c_void_p(W_ptr), c_void_p(Y_ptr),
                                        _quant(fmt), int(M), int(N), int(K), _dtype(x_dtype),
                                        _dtype(y_dtype), c_void_p(cuda_stream)))


def raw_fused_rmsnorm_gemv_quantized(ctx, X_ptr, gamma_ptr, W_ptr, Y_ptr, fmt, M, N, K, eps=1e-5,
                                     x_dtype="f16", y_dtype="f16", cuda_stream=0) -> None:
    _check(lib().tcx_raw_fused_rmsnorm_gemv_quantized(
        _h(ctx), c_void_p(X_ptr), c_void_p(gamma_ptr), c_void_p(W_ptr), c_void_p(Y_ptr),
        _quant(fmt), int(M), int(N), int(K), float(eps), _dtype(x_dtype), _dtype(y_dtype),
        c_void_p(cuda_stream)))


def raw_fused_norm_gemv_f16(ctx, X_ptr, gamma_ptr, beta_ptr, W_ptr, Y_ptr, M, N, K, eps=1e-5,
                            cuda_stream=0) -> None:
    _check(lib().tcx_raw_fused_norm_gemv_f16(
        _h(ctx), c_void_p(X_ptr), c_void_p(gamma_ptr), c_void_p(beta_ptr) if beta_ptr else None,
        c_void_p(W_ptr), c_void_p(Y_ptr), int(M), int(N), int(K), float(eps),
        c_void_p(cuda_stream)))


def raw_decode_q4_static(ctx, ops, cuda_stream=0) -> None:
    """ops: list of dicts with device addresses W, X, Y, optional gamma, and N, K, x_dtype,
    y_dtype, eps - one decode step as one persistent launch whose scratch is a static device
    array (no allocation; at most DECODE_STATIC_MAX_OPS operations)."""
    arr = (TCXDecodeOp * len(ops))()
    for i, o in enumerate(ops):
        arr[i].W, arr[i].X, arr[i].Y = o["W"], o["X"], o["Y"]
        arr[i].gamma = o.get("gamma") or None
        arr[i].N, arr[i].K = int(o["N"]), int(o["K"])
        arr[i].x_dtype, arr[i].y_dtype = _dtype(o.get("x_dtype", "f16")), _dtype(o.get("y_dtype", "f16"))
        arr[i].eps = float(o.get("eps", 1e-5))
    _check(lib().tcx_raw_decode_q4_static(_h(ctx), arr, len(ops), c_void_p(cuda_stream)))


def stream_tp_export(stream, pool_floats: int) -> bytes:
    """Allocates the stream's decode scratch and returns its 128-byte IPC record."""
    buf = ctypes.create_string_buffer(128)
    _check(lib().tcx_stream_tp_export(_h(stream), int(pool_floats), buf))
    return buf.raw


def stream_tp_connect(stream, n_ranks: int, rank: int, records: bytes) -> None:
    """records: the ranks' 128-byte records concatenated in rank order."""
    assert len(records) == 128 * n_ranks
    _check(lib().tcx_stream_tp_connect(_h(stream), int(n_ranks), int(rank), ctypes.c_char_p(records)))


def make_decode_tp_ops(ops):
    """ctypes array for stream_decode_tp from a list of dicts (device addresses W, X, Y, optional
    gamma; N, K, x_dtype, y_dtype, eps; optional peers, y_row0, y_rows, layout_rows, expect)."""
    arr = (TCXDecodeTpOp * len(ops))()
    for i, o in enumerate(ops):
        a = arr[i].op
        a.W, a.X, a.Y = o["W"], o["X"], o["Y"]
        a.gamma = o.get("gamma") or None
        a.N, a.K = int(o["N"]), int(o["K"])
        a.x_dtype, a.y_dtype = _dtype(o.get("x_dtype", "f16")), _dtype(o.get("y_dtype", "f16"))
        a.eps = float(o.get("eps", 1e-5))
        arr[i].peers, arr[i].y_row0 = int(o.get("peers", 0)), int(o.get("y_row0", 0))
        arr[i].y_rows, arr[i].layout_rows = int(o.get("y_rows", 0)), int(o.get("layout_rows", 0))
        arr[i].expect = int(o.get("expect", 0))
    return arr


def stream_decode_tp(stream, arr) -> None:
    _check(lib().tcx_stream_decode_tp(_h(stream), arr, len(arr)))


def set_gemv_variant(name: str) -> None:
    _check(lib().tcx_set_gemv_variant(name.encode()))


def take_device_error(ctx) -> int:
    return int(lib().tcx_take_device_error(_h(ctx)))


def launch_count() -> int:
    return int(lib().tcx_launch_count())


# --- GGUF ---------------------------------------------------------------------------------
def gguf_open(path: str):
    out = c_void_p()
    _check(lib().tc_gguf_open(os.fsencode(path), byref(out)))
    return out


def gguf_close(g) -> None:
    lib().tc_gguf_close(_h(g))


def gguf_tensor_count(g) -> int:
    return int(lib().tc_gguf_tensor_count(_h(g)))


def gguf_metadata_count(g) -> int:
    return int(lib().tc_gguf_metadata_count(_h(g)))


def gguf_meta_get_str(g, key: str):
    v = lib().tc_gguf_meta_get_str(_h(g), key.encode())
    return None if v is None else v.decode()


def gguf_meta_get_i64(g, key: str, default: int = 0) -> int:
    return int(lib().tc_gguf_meta_get_i64(_h(g), key.encode(), int(default)))


def gguf_meta_get_f64(g, key: str, default: float = 0.0) -> float:
    return float(lib().tc_gguf_meta_get_f64(_h(g), key.encode(), float(default)))


def gguf_meta_array_count(g, key: str) -> int:
    return int(lib().tc_gguf_meta_array_count(_h(g), key.encode()))


def gguf_meta_array_get_str(g, key: str, index: int) -> str:
    p, n = c_void_p(), c_size_t()
    _check(lib().tc_gguf_meta_array_get_str(_h(g), key.encode(), int(index), byref(p), byref(n)))
    return ctypes.string_at(p, n.value).decode()


def gguf_meta_array_get_i64(g, key: str, index: int, default: int = 0) -> int:
    return int(lib().tc_gguf_meta_array_get_i64(_h(g), key.encode(), int(index), int(default)))


def gguf_meta_array_get_f64(g, key: str, index: int, default: float = 0.0) -> float:
    return float(lib().tc_gguf_meta_array_get_f64(_h(g), key.encode(), int(index), float(default)))


def _tensor_dict(info) -> dict:
    d = {"name": info.name.decode() if info.name else "", "n_dims": int(info.n_dims),
         "dims": [int(info.dims[k]) for k in range(info.n_dims)], "type": int(info.type),
         "offset": int(info.offset), "n_bytes": int(info.n_bytes)}
    if hasattr(info, "data"):
        d["data"] = info.data
    else:
        d["buffer"] = info.buffer
    return d


def gguf_get_llama_config(g) -> dict:
    cfg = TCGGufLlamaConfig()
    _check(lib().tc_gguf_get_llama_config(_h(g), byref(cfg)))
    return {n: getattr(cfg, n) for n, _ in TCGGufLlamaConfig._fields_}


def gguf_get_tensor(g, name: str) -> dict:
    info = TCGGufTensorInfo()
    _check(lib().tc_gguf_get_tensor(_h(g), name.encode(), byref(info)))
    return _tensor_dict(info)


def gguf_tensor_at(g, index: int) -> dict:
    info = TCGGufTensorInfo()
    _check(lib().tc_gguf_tensor_at(_h(g), int(index), byref(info)))
    return _tensor_dict(info)


def gguf_tensor_to_buffer(ctx, g, name: str):
    out = c_void_p()
    _check(lib().tc_gguf_tensor_to_buffer(_h(ctx), _h(g), name.encode(), byref(out)))
    return out


def gguf_load_supported_tensors(ctx, g):
    out = c_void_p()
    _check(lib().tc_gguf_load_supported_tensors(_h(ctx), _h(g), byref(out)))
    return out


def gguf_loaded_model_free(ctx, model) -> None:
    lib().tc_gguf_loaded_model_free(_h(ctx), _h(model))


def gguf_loaded_tensor_count(model) -> int:
    return int(lib().tc_gguf_loaded_tensor_count(_h(model)))


def gguf_loaded_skipped_tensor_count(model) -> int:
    return int(lib().tc_gguf_loaded_skipped_tensor_count(_h(model)))


def gguf_loaded_tensor_at(model, index: int) -> dict:
    info = TCGGufLoadedTensorInfo()
    _check(lib().tc_gguf_loaded_tensor_at(_h(model), int(index), byref(info)))
    return _tensor_dict(info)


def gguf_loaded_get_tensor(model, name: str) -> dict:
    info = TCGGufLoadedTensorInfo()
    _check(lib().tc_gguf_loaded_get_tensor(_h(model), name.encode(), byref(info)))
    return _tensor_dict(info)


def _matrix_dict(mi) -> dict:
    return {"N": int(mi.N), "K": int(mi.K), "gguf_type": int(mi.gguf_type),
            "quant_type": int(mi.quant_type), "n_bytes": int(mi.n_bytes), "buffer": mi.buffer}


def gguf_tensor_quantized_matrix_info(g, name: str) -> dict:
    info = TCGGufTensorInfo()
    _check(lib().tc_gguf_get_tensor(_h(g), name.encode(), byref(info)))
    mi = TCGGufQuantizedMatrixInfo()
    _check(lib().tc_gguf_tensor_quantized_matrix_info(byref(info), byref(mi)))
    return _matrix_dict(mi)


def gguf_loaded_tensor_quantized_matrix_info(model, name: str) -> dict:
    info = TCGGufLoadedTensorInfo()
    _check(lib().tc_gguf_loaded_get_tensor(_h(model), name.encode(), byref(info)))
    mi = TCGGufQuantizedMatrixInfo()
    _check(lib().tc_gguf_loaded_tensor_quantized_matrix_info(byref(info), byref(mi)))
    return _matrix_dict(mi)


# ----------------------------------------------------------------------------------------
# Object wrappers
# ----------------------------------------------------------------------------------------
class Context:
    """Owns one reference on the process-wide context."""

    def __init__(self):
        self.handle = init()

    def close(self) -> None:
        if self.handle is not None:
            shutdown(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def device_info(self):
        return device_info(self.handle)

    def buffer(self, nbytes: int) -> "Buffer":
        return Buffer(self, nbytes)

    def buffer_from_array(self, arr: np.ndarray, mapped: bool = False) -> "Buffer":
        a = np.ascontiguousarray(arr)
        b = Buffer(self, a.nbytes)
        (b.write if mapped else b.upload)(a)
        return b

    def buffer_from_ptr(self, ptr: int, nbytes: int) -> "Buffer":
        return Buffer(self, handle=buffer_from_ptr(self.handle, ptr, nbytes), nbytes=nbytes)

    def stream(self) -> "Stream":
        return Stream(self)

    def open_gguf(self, path: str) -> "GgufFile":
        return GgufFile(path)

    def load_supported_tensors(self, gguf) -> "LoadedModel":
        return LoadedModel(self, gguf)

    def quantize_weights(self, W_fp16, W_quant, fmt, N, K):
        quantize_weights(self.handle, W_fp16, W_quant, fmt, N, K)

    def gemv_quantized(self, X, W_quant, Y, fmt, M, N, K):
        gemv_quantized(self.handle, X, W_quant, Y, fmt, M, N, K)

    def gemv_quantized_async(self, X, W_quant, Y, fmt, M, N, K, stream):
        gemv_quantized_async(self.handle, X, W_quant, Y, fmt, M, N, K, stream)

    def fused_rmsnorm_gemv_quantized(self, X, gamma, W_quant, Y, fmt, M, N, K, eps=1e-5):
        fused_rmsnorm_gemv_quantized(self.handle, X, gamma, W_quant, Y, fmt, M, N, K, eps)

    def fused_rmsnorm_gemv(self, X, gamma, W, Y, M, N, K, eps=1e-5):
        fused_rmsnorm_gemv(self.handle, X, gamma, W, Y, M, N, K, eps)

    def fused_layernorm_gemv(self, X, gamma, beta, W, Y, M, N, K, eps=1e-5):
        fused_layernorm_gemv(self.handle, X, gamma, beta, W, Y, M, N, K, eps)


class Buffer:
    def __init__(self, ctx: Context, nbytes: int | None = None, handle=None, owned: bool = True):
        self.ctx = ctx
        self.handle = handle if handle is not None else buffer_alloc(ctx.handle, nbytes)
        self.owned = owned
        self.nbytes = buffer_size(self.handle)

    def close(self) -> None:
        if self.handle is not None and self.owned and self.ctx.handle is not None:
            buffer_free(self.ctx.handle, self.handle)
        self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def map(self) -> int:
        return buffer_map(self.handle)

    def write(self, arr):
        buffer_write(self.handle, arr)

    def read(self, arr):
        return buffer_read(self.handle, arr)

    def upload(self, arr, offset: int = 0):
        buffer_upload(self.handle, arr, offset)

    def download(self, arr, offset: int = 0):
        return buffer_download(self.handle, arr, offset)

    def device_ptr(self) -> int:
        return buffer_device_ptr(self.handle)

    def to_numpy(self, shape, dtype, offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        return self.download(out, offset)


class Stream:
    def __init__(self, ctx: Context):
        self.ctx = ctx
        self.handle = stream_create(ctx.handle)

    def sync(self) -> None:
        stream_sync(self.handle)

    def flush(self) -> None:
        stream_flush(self.handle)

    def cuda_handle(self) -> int:
        return stream_cuda_handle(self.handle)

    def close(self) -> None:
        if self.handle is not None and self.ctx.handle is not None:
            stream_destroy(self.ctx.handle, self.handle)
        self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


class GgufFile:
    def __init__(self, path: str):
        self.handle = gguf_open(path)

    def close(self) -> None:
        if self.handle is not None:
            gguf_close(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def tensor_count(self):
        return gguf_tensor_count(self.handle)

    def metadata_count(self):
        return gguf_metadata_count(self.handle)

    def get_tensor(self, name):
        return gguf_get_tensor(self.handle, name)

    def tensor_at(self, index):
        return gguf_tensor_at(self.handle, index)

    def meta_get_str(self, key):
        return gguf_meta_get_str(self.handle, key)

    def meta_get_i64(self, key, default=0):
        return gguf_meta_get_i64(self.handle, key, default)

    def meta_get_f64(self, key, default=0.0):
        return gguf_meta_get_f64(self.handle, key, default)

    def meta_array_count(self, key):
        return gguf_meta_array_count(self.handle, key)

    def meta_array_get_str(self, key, index):
        return gguf_meta_array_get_str(self.handle, key, index)

    def llama_config(self):
        return gguf_get_llama_config(self.handle)

    def tensor_to_buffer(self, ctx: Context, name: str) -> Buffer:
        return Buffer(ctx, handle=gguf_tensor_to_buffer(ctx.handle, self.handle, name))

    def load_supported_tensors(self, ctx: Context) -> "LoadedModel":
        return LoadedModel(ctx, self)


class LoadedModel:
    def __init__(self, ctx: Context, gguf: GgufFile):
        self.ctx = ctx
        self.handle = gguf_load_supported_tensors(ctx.handle, gguf.handle)

    def close(self) -> None:
        if self.handle is not None and self.ctx.handle is not None:
            gguf_loaded_model_free(self.ctx.handle, self.handle)
        self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def tensor_count(self):
        return gguf_loaded_tensor_count(self.handle)

    def skipped_tensor_count(self):
        return gguf_loaded_skipped_tensor_count(self.handle)

    def tensor_at(self, index):
        return gguf_loaded_tensor_at(self.handle, index)

    def get_tensor(self, name):
        return gguf_loaded_get_tensor(self.handle, name)

    def quantized_matrix(self, name) -> "QuantizedMatrix":
        return QuantizedMatrix(self, name)


class QuantizedMatrix:
    """A loaded 2-D Q4_0/Q8_0 tensor viewed as the [N,K] operand of gemv_quantized
    (python/tensorcore/__init__.py:2460-2496)."""

    def __init__(self, model: LoadedModel, name: str):
        self.model = model
        self.name = name
        info = gguf_loaded_tensor_quantized_matrix_info(model.handle, name)
        self.N, self.K = info["N"], info["K"]
        self.quant_type = info["quant_type"]
        self.n_bytes = info["n_bytes"]
        self.buffer = Buffer(model.ctx, handle=c_void_p(info["buffer"]), owned=False)

    def output(self, M: int = 1) -> Buffer:
        return Buffer(self.model.ctx, M * self.N * 2)

    def gemv(self, X, Y, M: int = 1) -> None:
        gemv_quantized(self.model.ctx.handle, X, self.buffer, Y, self.quant_type, M, self.N, self.K)

    def gemv_async(self, X, Y, stream, M: int = 1) -> None:
        gemv_quantized_async(self.model.ctx.handle, X, self.buffer, Y, self.quant_type, M, self.N,
                             self.K, stream)
