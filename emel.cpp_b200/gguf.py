"""GGUF bindings (include/emelb_gguf.h): a file image parsed by the library into
the reference's tensor records and key/value entries
(src/emel/gguf/loader/detail.hpp:419-733, src/emel/model/data.hpp:123-134), and a
Llama decoder session built from such a file the way the reference's model loader
binds one (src/emel/model/llama/detail.cpp:14-41, 60-75;
src/emel/model/generation/any.cpp:294-341)."""
from __future__ import annotations

import ctypes as C
import os
import struct

import emel_cpp_b200 as eb
from emel_cpp_b200 import llama as el

_P = C.c_void_p

# loader error bitmask (src/emel/gguf/loader/errors.hpp:7-15)
OK, INVALID_REQUEST, MODEL_INVALID, CAPACITY, PARSE_FAILED, INTERNAL_ERROR, UNTRACKED = 0, 1, 2, 4, 8, 16, 32
ERROR_NAMES = {0: "none", 1: "invalid_request", 2: "model_invalid", 4: "capacity", 8: "parse_failed",
               16: "internal_error", 32: "untracked"}

# metadata value types (src/emel/gguf/loader/detail.hpp:26-39)
(T_UINT8, T_INT8, T_UINT16, T_INT16, T_UINT32, T_INT32, T_FLOAT32, T_BOOL, T_STRING, T_ARRAY, T_UINT64, T_INT64,
 T_FLOAT64) = range(13)
_SCALAR = {T_UINT8: "<B", T_INT8: "<b", T_UINT16: "<H", T_INT16: "<h", T_UINT32: "<I", T_INT32: "<i",
           T_FLOAT32: "<f", T_BOOL: "<?", T_UINT64: "<Q", T_INT64: "<q", T_FLOAT64: "<d"}


class Requirements(C.Structure):
    _fields_ = [("tensor_count", C.c_uint32), ("kv_count", C.c_uint32), ("max_key_bytes", C.c_uint32),
                ("max_value_bytes", C.c_uint32), ("tensor_data_bytes", C.c_uint64)]

    def as_tuple(self):
        return (self.tensor_count, self.kv_count, self.max_key_bytes, self.max_value_bytes, self.tensor_data_bytes)


class TensorRecord(C.Structure):
    _fields_ = [("name", _P), ("name_length", C.c_uint32), ("type", C.c_int32), ("n_dims", C.c_int32),
                ("dims", C.c_int64 * 4), ("data_offset", C.c_uint64), ("file_offset", C.c_uint64),
                ("data_size", C.c_uint64), ("data", _P)]


class KvRecord(C.Structure):
    _fields_ = [("key", _P), ("key_length", C.c_uint32), ("value_type", C.c_uint32), ("value", _P),
                ("value_length", C.c_uint32)]


SIGNATURES = {
    "emelb_gguf_probe": (C.c_uint32, [_P, C.c_uint64, C.POINTER(Requirements)]),
    "emelb_gguf_open_image": (C.c_uint32, [_P, C.c_uint64, C.POINTER(_P)]),
    "emelb_gguf_open_file": (C.c_uint32, [C.c_char_p, C.POINTER(_P)]),
    "emelb_gguf_close": (C.c_uint32, [_P]),
    "emelb_gguf_get_requirements": (C.c_uint32, [_P, C.POINTER(Requirements)]),
    "emelb_gguf_layout": (C.c_uint32, [_P, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]),
    "emelb_gguf_tensor_at": (C.c_uint32, [_P, C.c_uint32, C.POINTER(TensorRecord)]),
    "emelb_gguf_kv_at": (C.c_uint32, [_P, C.c_uint32, C.POINTER(KvRecord)]),
    "emelb_gguf_find_tensor": (C.c_int32, [_P, C.c_char_p]),
    "emelb_gguf_find_kv": (C.c_int32, [_P, C.c_char_p]),
    "emelb_gguf_upload": (C.c_uint32, [_P, _P, C.c_uint32, C.c_int32, C.POINTER(_P)]),
    "emelb_gguf_upload_all": (C.c_uint32, [_P, _P, C.c_int32]),
    "emelb_gguf_upload_rows": (C.c_uint32, [_P, _P, C.c_uint32, C.c_int32, C.c_uint64, C.c_uint64, C.POINTER(_P),
                                            C.POINTER(_P)]),
}


def register(lib):
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


class GgufError(RuntimeError):
    def __init__(self, what: str, err: int):
        super().__init__(f"{what} failed: {ERROR_NAMES.get(err, hex(err))}")
        self.err = err


def _address(image):
    """(address, byte count, keep-alive) of a bytes-like or numpy image."""
    if hasattr(image, "ctypes"):
        return image.ctypes.data, int(image.nbytes), image
    buf = (C.c_uint8 * len(image)).from_buffer_copy(bytes(image)) if len(image) else None
    return (C.addressof(buf) if buf is not None else 0), len(image), buf


def probe(image):
    """-> (error mask, Requirements): event::probe of the reference loader."""
    addr, n, _keep = _address(image)
    req = Requirements()
    err = eb.lib().emelb_gguf_probe(addr, n, C.byref(req))
    return err, req


def decode_value(value_type: int, payload: bytes):
    """A key/value payload as Python data: scalars, str, or a list for arrays."""
    if value_type == T_STRING:
        (n,) = struct.unpack_from("<Q", payload, 0)
        return payload[8:8 + n].decode("utf-8", "replace")
    if value_type == T_ARRAY:
        elem, count = struct.unpack_from("<IQ", payload, 0)
        at, out = 12, []
        if elem == T_STRING:
            for _ in range(count):
                (n,) = struct.unpack_from("<Q", payload, at)
                out.append(payload[at + 8:at + 8 + n].decode("utf-8", "replace"))
                at += 8 + n
            return out
        fmt = _SCALAR[elem]
        return [v[0] for v in struct.iter_unpack(fmt, payload[at:at + count * struct.calcsize(fmt)])]
    return struct.unpack_from(_SCALAR[value_type], payload, 0)[0]


class File:
    """An opened GGUF image.  `source` is a path (mapped read-only by the library) or a
    bytes-like / numpy image that this object keeps alive."""

    def __init__(self, source):
        self._h = _P()
        self._keep = None
        lib = eb.lib()
        if isinstance(source, (str, os.PathLike)):
            err = lib.emelb_gguf_open_file(os.fsencode(source), C.byref(self._h))
        else:
            addr, n, self._keep = _address(source)
            err = lib.emelb_gguf_open_image(addr, n, C.byref(self._h))
        if err != OK:
            raise GgufError("gguf open", err)
        req = Requirements()
        lib.emelb_gguf_get_requirements(self._h, C.byref(req))
        self.requirements = req
        a, off = C.c_uint32(0), C.c_uint64(0)
        lib.emelb_gguf_layout(self._h, C.byref(a), C.byref(off))
        self.alignment, self.data_section_offset = a.value, off.value

    def close(self):
        if self._h:
            eb.lib().emelb_gguf_close(self._h)
            self._h = _P()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def handle(self):
        return self._h

    def tensor(self, index: int) -> dict:
        t = TensorRecord()
        err = eb.lib().emelb_gguf_tensor_at(self._h, index, C.byref(t))
        if err != OK:
            raise GgufError("gguf tensor_at", err)
        raw = C.string_at(t.name, t.name_length)
        return {"name": raw.decode("utf-8", "replace"), "name_bytes": raw, "type": t.type,
                "n_dims": t.n_dims, "dims": tuple(t.dims), "data_offset": t.data_offset,
                "file_offset": t.file_offset, "data_size": t.data_size, "data": t.data or 0, "index": index}

    def tensors(self):
        return [self.tensor(i) for i in range(self.requirements.tensor_count)]

    def kv(self, index: int, raw_key: bool = False):
        """-> (key, value type, raw payload bytes); the key as bytes with raw_key"""
        e = KvRecord()
        err = eb.lib().emelb_gguf_kv_at(self._h, index, C.byref(e))
        if err != OK:
            raise GgufError("gguf kv_at", err)
        key = C.string_at(e.key, e.key_length)
        return key if raw_key else key.decode("utf-8", "replace"), e.value_type, C.string_at(e.value, e.value_length)

    def kvs(self):
        return [self.kv(i) for i in range(self.requirements.kv_count)]

    def find_tensor(self, name: str):
        i = eb.lib().emelb_gguf_find_tensor(self._h, name.encode())
        return None if i < 0 else self.tensor(i)

    def get(self, key: str, default=None):
        i = eb.lib().emelb_gguf_find_kv(self._h, key.encode())
        if i < 0:
            return default
        _k, t, payload = self.kv(i)
        return decode_value(t, payload)

    def upload(self, backend: eb.Backend, tensor_index: int, tensor_id: int) -> int:
        """The tensor's bytes -> HBM; returns the device address."""
        dev = _P()
        err = eb.lib().emelb_gguf_upload(backend.handle, self._h, tensor_index, tensor_id, C.byref(dev))
        if err != OK:
            raise GgufError("gguf upload", err)
        return dev.value

    def upload_all(self, backend: eb.Backend, first_tensor_id: int = 0) -> None:
        """Every tensor of the file -> HBM in one pipelined pass; tensor i gets id first_tensor_id + i."""
        err = eb.lib().emelb_gguf_upload_all(backend.handle, self._h, first_tensor_id)
        if err != OK:
            raise GgufError("gguf upload_all", err)

    def upload_rows(self, backend: eb.Backend, tensor_index: int, tensor_id: int, first_row: int, rows: int):
        """Rows [first_row, first_row + rows) -> HBM; returns (address in the image, device address)."""
        host, dev = _P(), _P()
        err = eb.lib().emelb_gguf_upload_rows(backend.handle, self._h, tensor_index, tensor_id, first_row, rows,
                                              C.byref(host), C.byref(dev))
        if err != OK:
            raise GgufError("gguf upload_rows", err)
        return host.value, dev.value


_LAYER_TENSORS = {el.ATTN_NORM: "attn_norm", el.ATTN_Q: "attn_q", el.ATTN_K: "attn_k", el.ATTN_V: "attn_v",
                  el.ATTN_OUT: "attn_output", el.FFN_NORM: "ffn_norm", el.FFN_GATE: "ffn_gate", el.FFN_UP: "ffn_up",
                  el.FFN_DOWN: "ffn_down"}
_GLOBAL_TENSORS = {el.TOKEN_EMBD: "token_embd.weight", el.OUTPUT_NORM: "output_norm.weight", el.OUTPUT: "output.weight"}
_NORMS = (el.ATTN_NORM, el.FFN_NORM, el.OUTPUT_NORM)


def llama_config(f: File, n_ctx: int | None = None, kv_block: int = 16, shard_rank: int = 0,
                 shard_count: int = 1) -> el.Config:
    """Hyper-parameters under the `llama.` keys (src/emel/model/llama/detail.cpp:14-41);
    the vocabulary size falls back to the embedding table's row count."""
    def need(key):
        v = f.get(key)
        if v is None:
            raise GgufError(f"gguf key {key}", MODEL_INVALID)
        return v
    if f.get("general.architecture", "llama") != "llama":
        raise GgufError("gguf architecture", MODEL_INVALID)
    n_embd, n_head = int(need("llama.embedding_length")), int(need("llama.attention.head_count"))
    n_head_kv = int(f.get("llama.attention.head_count_kv", n_head))
    if n_head <= 0 or n_embd % n_head != 0:
        raise GgufError("gguf llama.attention.head_count", MODEL_INVALID)
    head_dim = n_embd // n_head
    embd = f.find_tensor(_GLOBAL_TENSORS[el.TOKEN_EMBD])
    if embd is None:
        raise GgufError("gguf tensor token_embd.weight", MODEL_INVALID)
    n_vocab = int(f.get("llama.vocab_size", embd["dims"][1]))
    ctx = int(need("llama.context_length")) if n_ctx is None else int(n_ctx)
    return el.config(n_layer=int(need("llama.block_count")), n_embd=n_embd, n_head=n_head, n_head_kv=n_head_kv,
                     head_dim=head_dim, n_ff=int(need("llama.feed_forward_length")), n_vocab=n_vocab, n_ctx=ctx,
                     rope_freq_base=float(f.get("llama.rope.freq_base", 10000.0)),
                     rms_eps=float(f.get("llama.attention.layer_norm_rms_epsilon", 1e-5)),
                     rope_dim=int(f.get("llama.rope.dimension_count", head_dim)), kv_block=kv_block,
                     shard_rank=shard_rank, shard_count=shard_count)


def layer_extents(f: File, n_layer: int):
    """One list of (tensor_id, file_offset, byte_size) per layer: the nine `blk.<layer>.*` tensors of the decoder, in
    role order -- the extents a streaming window is bound with.  tensor_id is the tensor's index in the file."""
    layers = []
    for layer in range(n_layer):
        weights = []
        for stem in _LAYER_TENSORS.values():
            t = f.find_tensor(f"blk.{layer}.{stem}.weight")
            if t is None:
                raise GgufError(f"gguf tensor blk.{layer}.{stem}.weight", MODEL_INVALID)
            weights.append((t["index"], t["file_offset"], t["data_size"]))
        layers.append(weights)
    return layers


def load_llama_streamed(backend: eb.Backend, f: File, budget_bytes: int, window_slots: int = 4, prefetch_depth: int = 2,
                        n_ctx: int | None = None, first_tensor_id: int = 0, staged_only: bool = False):
    """A decoder whose layers stay in the file mapping and cross to HBM through a streaming window of
    `window_slots` layer slots (budget_bytes is the HBM the layers may take; a model that fits it is loaded
    whole by load_llama instead).  The embedding table, the output norm and the output projection are uploaded
    as usual.  Returns (session, window); close the session before the window."""
    from . import window as ew
    cfg = llama_config(f, n_ctx)
    layers = layer_extents(f, cfg.n_layer)
    first = f.tensor(0)
    base = first["data"] - first["file_offset"]
    size = max(t["file_offset"] + t["data_size"] for t in f.tensors())
    win = ew.LayerWindow(backend)
    if staged_only:
        win.set_staged_only(True)
    if not win.bind(base, layers, budget_bytes, window_slots, prefetch_depth, source_bytes=size):
        err = win.last_error
        win.close()
        raise GgufError("layer window bind", err)
    if not win.bound["streaming_active"]:
        win.close()
        return load_llama(backend, f, n_ctx, first_tensor_id), None
    sess = el.Session(backend, cfg)
    shapes = el.matrix_shapes(cfg)
    try:
        if not sess.set_window(win):
            raise GgufError("layer window attach", MODEL_INVALID)
        for role, name in _GLOBAL_TENSORS.items():
            t = f.find_tensor(name)
            if t is None:
                raise GgufError(f"gguf tensor {name}", MODEL_INVALID)
            f.upload(backend, t["index"], first_tensor_id + t["index"])
            ok = sess.bind_norm(-1, role, t["data"]) if role in _NORMS else sess.bind_matrix(-1, role, t["data"], t["type"])
            if not ok:
                raise GgufError(f"gguf bind {name}", MODEL_INVALID)
        for layer in range(cfg.n_layer):
            for role, stem in _LAYER_TENSORS.items():
                t = f.find_tensor(f"blk.{layer}.{stem}.weight")
                if role in _NORMS:
                    ok = t["type"] == eb.F32 and sess.bind_norm(layer, role, t["data"])
                else:
                    ok = (t["dims"][0], t["dims"][1]) == shapes[role] and sess.bind_matrix(layer, role, t["data"], t["type"])
                if not ok:
                    raise GgufError(f"gguf bind blk.{layer}.{stem}.weight", MODEL_INVALID)
    except Exception:
        sess.close()
        win.close()
        raise
    return sess, win


def load_llama(backend: eb.Backend, f: File, n_ctx: int | None = None, first_tensor_id: int = 0,
               shard_rank: int = 0, shard_count: int = 1) -> el.Session:
    """Uploads every tensor the decoder needs from the mapping to HBM and binds it by its
    address in the image.  Tensor ids are first_tensor_id + the tensor's index in the file.
    In a row-sharded session only this rank's row interval of each matrix is uploaded
    (the embedding table and the norm weights are whole on every rank)."""
    cfg = llama_config(f, n_ctx, shard_rank=shard_rank, shard_count=shard_count)
    sess = el.Session(backend, cfg)
    shapes = el.matrix_shapes(cfg)

    whole = shard_count <= 1     # unsharded: the whole file goes up in one pipelined pass

    def bind(layer, role, name):
        t = f.find_tensor(name)
        if t is None:
            raise GgufError(f"gguf tensor {name}", MODEL_INVALID)
        tid = first_tensor_id + t["index"]
        if role in _NORMS:
            if not whole:
                f.upload(backend, t["index"], tid)
            ok = t["type"] == eb.F32 and t["dims"][0] == cfg.n_embd and sess.bind_norm(layer, role, t["data"])
        elif shard_count > 1 and role != el.TOKEN_EMBD:
            k, m = shapes[role]
            ok = t["dims"][0] == k and t["dims"][1] == m * shard_count
            if ok:
                host, _dev = f.upload_rows(backend, t["index"], tid, shard_rank * m, m)
                ok = sess.bind_matrix(layer, role, host, t["type"])
        else:
            if not whole:
                f.upload(backend, t["index"], tid)
            ok = (t["dims"][0], t["dims"][1]) == shapes[role] and sess.bind_matrix(layer, role, t["data"], t["type"])
        if not ok:
            raise GgufError(f"gguf bind {name}", MODEL_INVALID)

    try:
        if whole:
            f.upload_all(backend, first_tensor_id)
        for role, name in _GLOBAL_TENSORS.items():
            bind(-1, role, name)
        for layer in range(cfg.n_layer):
            for role, stem in _LAYER_TENSORS.items():
                bind(layer, role, f"blk.{layer}.{stem}.weight")
    except Exception:
        sess.close()
        raise
    return sess
