"""Writer for GGUF v3 files (little-endian), enough to package synthetic models for
tc_gguf_open / tc_gguf_load_supported_tensors.

Layout (what lib/io/gguf.c:341-455 of the reference reads): u32 magic 'GGUF', u32 version 3,
u64 tensor count, u64 key/value count; key/values (string key, u32 type, value); tensor infos
(string name, u32 n_dims, u64 dims[n], u32 ggml type, u64 offset from the data start); zero
padding to `general.alignment`; tensor data, each tensor starting on an aligned offset.
"""
from __future__ import annotations

import struct
from typing import BinaryIO, Callable, Iterable, Sequence

import numpy as np

GGUF_MAGIC = 0x46554747
# metadata value types
U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
# ggml tensor types
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q8_0, GGML_BF16 = 0, 1, 2, 3, 8, 30

_SCALAR_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f",
               BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def _string(s: str | bytes) -> bytes:
    b = s.encode() if isinstance(s, str) else bytes(s)
    return struct.pack("<Q", len(b)) + b


def _value(vtype: int, value, elem_type: int | None = None) -> bytes:
    if vtype in _SCALAR_FMT:
        return struct.pack(_SCALAR_FMT[vtype], value)
    if vtype == STRING:
        return _string(value)
    if vtype == ARRAY:
        assert elem_type is not None
        out = [struct.pack("<IQ", elem_type, len(value))]
        out.extend(_value(elem_type, v) for v in value)
        return b"".join(out)
    raise ValueError(f"bad metadata type {vtype}")


class TensorSpec:
    """A tensor to write: `dims` in GGUF order (dims[0] is the contiguous one), raw bytes given
    either directly or by a callable that writes them to the file (for large tensors)."""

    def __init__(self, name: str, dims: Sequence[int], ggml_type: int, n_bytes: int,
                 data: bytes | np.ndarray | None = None,
                 writer: Callable[[BinaryIO], None] | None = None):
        self.name, self.dims, self.ggml_type, self.n_bytes = name, list(dims), ggml_type, n_bytes
        self.data, self.writer = data, writer


def write_gguf(path: str, metadata: Iterable[tuple], tensors: Sequence[TensorSpec],
               alignment: int = 32) -> None:
    """metadata: (key, type, value) or (key, ARRAY, values, elem_type) tuples.  A
    `general.alignment` key is added when `alignment` differs from the default 32."""
    metadata = list(metadata)
    if alignment != 32 and not any(m[0] == "general.alignment" for m in metadata):
        metadata.append(("general.alignment", U32, alignment))
    offsets, off = [], 0
    for t in tensors:
        offsets.append(off)
        off += (t.n_bytes + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(metadata)))
        for m in metadata:
            key, vtype, value = m[0], m[1], m[2]
            f.write(_string(key))
            f.write(struct.pack("<I", vtype))
            f.write(_value(vtype, value, m[3] if len(m) > 3 else None))
        for t, o in zip(tensors, offsets):
            f.write(_string(t.name))
            f.write(struct.pack("<I", len(t.dims)))
            for d in t.dims:
                f.write(struct.pack("<Q", d))
            f.write(struct.pack("<IQ", t.ggml_type, o))
        pos = f.tell()
        f.write(b"\0" * ((alignment - pos % alignment) % alignment))
        data_start = f.tell()
        for t, o in zip(tensors, offsets):
            assert f.tell() == data_start + o
            if t.writer is not None:
                t.writer(f)
            elif t.data is not None:
                f.write(t.data.tobytes() if isinstance(t.data, np.ndarray) else t.data)
            written = f.tell() - (data_start + o)
            if t.ggml_type in (GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q8_0, GGML_BF16):
                assert written == t.n_bytes, (t.name, written, t.n_bytes)
            pad = (alignment - f.tell() % alignment) % alignment
            if pad and t is not tensors[-1]:
                f.write(b"\0" * pad)


def llama_metadata(d_model: int, d_ff: int, n_layers: int, n_heads: int, n_kv_heads: int,
                   vocab: int, context: int = 4096, eps: float = 1e-5) -> list[tuple]:
    """The keys tc_gguf_get_llama_config reads (lib/io/gguf.c:662-693).  The vocabulary is a list
    of `vocab` placeholder token strings: only its length is used."""
    return [
        ("general.architecture", STRING, "llama"),
        ("general.name", STRING, "synthetic-llama"),
        ("llama.context_length", U32, context),
        ("llama.embedding_length", U32, d_model),
        ("llama.feed_forward_length", U32, d_ff),
        ("llama.block_count", U32, n_layers),
        ("llama.attention.head_count", U32, n_heads),
        ("llama.attention.head_count_kv", U32, n_kv_heads),
        ("llama.rope.dimension_count", U32, d_model // n_heads),
        ("llama.attention.layer_norm_rms_epsilon", F32, eps),
        ("llama.rope.freq_base", F32, 10000.0),
        ("tokenizer.ggml.tokens", ARRAY, ["t"] * vocab, STRING),
    ]
