"""A small GGUF v3 writer (test images, the load benchmark's file): key/value pairs, tensor descriptions and
aligned tensor data, laid out as the reference's loader expects them
(src/emel/gguf/loader/detail.hpp:419-543)."""
from __future__ import annotations

import struct

import numpy as np

(T_UINT8, T_INT8, T_UINT16, T_INT16, T_UINT32, T_INT32, T_FLOAT32, T_BOOL, T_STRING, T_ARRAY, T_UINT64, T_INT64,
 T_FLOAT64) = range(13)
_FMT = {T_UINT8: "<B", T_INT8: "<b", T_UINT16: "<H", T_INT16: "<h", T_UINT32: "<I", T_INT32: "<i", T_FLOAT32: "<f",
        T_BOOL: "<?", T_UINT64: "<Q", T_INT64: "<q", T_FLOAT64: "<d"}


def gstr(s) -> bytes:
    b = s.encode() if isinstance(s, str) else bytes(s)
    return struct.pack("<Q", len(b)) + b


def value_payload(vtype: int, value, elem_type: int | None = None) -> bytes:
    if vtype == T_STRING:
        return gstr(value)
    if vtype == T_ARRAY:
        head = struct.pack("<IQ", elem_type, len(value))
        if elem_type == T_STRING:
            return head + b"".join(gstr(v) for v in value)
        return head + b"".join(struct.pack(_FMT[elem_type], v) for v in value)
    return struct.pack(_FMT[vtype], value)


def kv(key, vtype: int, value, elem_type: int | None = None) -> bytes:
    return gstr(key) + struct.pack("<I", vtype) + value_payload(vtype, value, elem_type)


def tensor_info(name, dims, ttype: int, offset: int) -> bytes:
    return gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + \
        struct.pack("<IQ", ttype, offset)


def pad(n: int, alignment: int) -> int:
    return (n + alignment - 1) // alignment * alignment


def build(kvs, tensors, alignment: int = 32, version: int = 3) -> bytes:
    """kvs: serialized pairs (kv(...)); tensors: (name, dims, ggml type, data bytes).  Offsets are the
    running padded offsets; `alignment` must agree with a general.alignment pair among kvs, if any."""
    out = bytearray(b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kvs)))
    for e in kvs:
        out += e
    offset = 0
    for name, dims, ttype, data in tensors:
        out += tensor_info(name, dims, ttype, offset)
        offset += pad(len(data), alignment)
    out += b"\0" * (pad(len(out), alignment) - len(out))
    for _name, _dims, _ttype, data in tensors:
        out += bytes(data) + b"\0" * (pad(len(data), alignment) - len(data))
    return bytes(out)


def reference_valid_file() -> bytes:
    """The image the reference's loader tests build (tests/gguf/loader/lifecycle_tests.cpp:94-110):
    one 2 x 3 f32 tensor, general.alignment = 32 and a two-string array."""
    return build([kv("general.alignment", T_UINT32, 32), kv("tokenizer.tokens", T_ARRAY, ["hi", "world"], T_STRING)],
                 [("weights.f32", (2, 3), 0, b"\0" * 24)], 32)


def rich_file(seed: int = 0) -> bytes:
    """Every metadata value type, an alignment of 64, and tensors of several block formats
    (one of them row-group packed, one scalar without dimensions)."""
    rng = np.random.default_rng(seed)
    kvs = [kv("general.architecture", T_STRING, "llama"), kv("general.alignment", T_UINT32, 64),
           kv("a.u8", T_UINT8, 200), kv("a.i8", T_INT8, -3), kv("a.u16", T_UINT16, 65000), kv("a.i16", T_INT16, -300),
           kv("a.i32", T_INT32, -70000), kv("a.f32", T_FLOAT32, 1.5), kv("a.bool", T_BOOL, True),
           kv("a.u64", T_UINT64, 1 << 40), kv("a.i64", T_INT64, -(1 << 40)), kv("a.f64", T_FLOAT64, 2.25),
           kv("a.floats", T_ARRAY, [0.5, 1.5, 2.5], T_FLOAT32), kv("a.bytes", T_ARRAY, list(range(7)), T_UINT8),
           kv("a.strings", T_ARRAY, ["", "x", "a longer token"], T_STRING), kv("a.empty", T_ARRAY, [], T_INT64)]
    shapes = [("t.f32", (5, 3), 0, 4 * 15), ("t.f16", (8,), 1, 16), ("t.q4_k", (512, 3), 12, 2 * 144 * 3),
              ("t.q6_k", (256, 2, 2), 14, 210 * 4), ("t.q8_0", (64, 5), 8, 2 * 34 * 5), ("t.q4_0", (32, 1, 1, 2), 2, 36),
              ("t.scalar", (), 0, 4), ("t.packed", (256, 9), 41, 2 * 1152), ("t.i32", (3,), 26, 12)]
    tensors = [(n, d, t, rng.integers(0, 256, size=b, dtype=np.uint8).tobytes()) for n, d, t, b in shapes]
    return build(kvs, tensors, 64)


# Llama tensor names (src/emel/model/llama/detail.cpp:9-10, src/emel/model/generation/any.cpp:15, 303-327)
def llama_file(cfg: dict, matrices: dict, norms: dict, alignment: int = 32, rope_freq_base: float = 500000.0,
               rms_eps: float = 1e-5) -> bytes:
    """matrices: name -> (K, M, ggml type, block bytes); norms: name -> f32 array of n_embd."""
    kvs = [kv("general.architecture", T_STRING, "llama"), kv("general.alignment", T_UINT32, alignment),
           kv("llama.context_length", T_UINT32, cfg["n_ctx"]), kv("llama.embedding_length", T_UINT32, cfg["n_embd"]),
           kv("llama.feed_forward_length", T_UINT32, cfg["n_ff"]),
           kv("llama.attention.head_count", T_UINT32, cfg["n_head"]),
           kv("llama.attention.head_count_kv", T_UINT32, cfg["n_head_kv"]),
           kv("llama.rope.dimension_count", T_UINT32, cfg["head_dim"]),
           kv("llama.block_count", T_UINT32, cfg["n_layer"]), kv("llama.vocab_size", T_UINT32, cfg["n_vocab"]),
           kv("llama.attention.layer_norm_rms_epsilon", T_FLOAT32, rms_eps),
           kv("llama.rope.freq_base", T_FLOAT32, rope_freq_base),
           kv("tokenizer.ggml.tokens", T_ARRAY, [f"<{i}>" for i in range(8)], T_STRING)]
    tensors = [(name, (k, m), t, np.ascontiguousarray(blocks).tobytes()) for name, (k, m, t, blocks) in matrices.items()]
    tensors += [(name, (len(w),), 0, np.ascontiguousarray(w, np.float32).tobytes()) for name, w in norms.items()]
    return build(kvs, tensors, alignment)
