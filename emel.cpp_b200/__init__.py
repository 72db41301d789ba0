"""emel.cpp_b200 — Python host side over the C-ABI library (libemelb.so).

The library is the product: hand-written sm_100a kernels behind the entry
points of include/emelb.h.  This module only loads it and mirrors, for tests
and the benchmark, the calling convention of the reference's kernel actor:
`process_event(op) -> bool` with the reason kept in `last_error`
(src/emel/kernel/any.hpp:76-80, src/emel/kernel/x86_64/sm.hpp:1198-1211,
1327-1331).  There is no CPU fallback: without the built library every entry
point raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libemelb.so")

# dtype codes (src/emel/kernel/events.hpp:78-123)
F32, F16, Q4_0, Q8_0, Q4_K, Q6_K, Q8_K, I32 = 0, 1, 2, 8, 12, 14, 15, 26
BLOCK_ELEMS = {Q4_0: 32, Q8_0: 32, Q4_K: 256, Q6_K: 256, Q8_K: 256}
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34, Q4_K: 144, Q6_K: 210, Q8_K: 292}
# error bitmask (src/emel/kernel/errors.hpp:7-13)
OK, INVALID_REQUEST, UNSUPPORTED_OP, INTERNAL_ERROR, UNTRACKED = 0, 1, 2, 4, 8
OP_MUL_MAT, OP_MUL_MAT_ARGMAX, OP_FLASH_ATTN_EXT, OP_RMS_NORM, OP_ROPE, OP_GLU = 1, 2, 3, 4, 5, 6
LIFECYCLE = {0: "unbound", 1: "resident", 2: "evicted", 3: "internal_error", 4: "mmap_resident"}


class View(C.Structure):
    """tensor_view (src/emel/kernel/events.hpp:125-137)."""
    _fields_ = [("data", C.c_void_p), ("type", C.c_uint8), ("ne", C.c_uint64 * 4), ("nb", C.c_uint64 * 4)]


class Op(C.Structure):
    """Generic op fields + index_out (src/emel/kernel/events.hpp:178-189, 220-223)."""
    _fields_ = [("src0", View), ("src1", View), ("src2", View), ("dst", View),
                ("op_params", C.c_uint8 * 64), ("op_params_size", C.c_uint32),
                ("index_out", C.POINTER(C.c_int32))]


class HeadRangeRequest(C.Structure):
    """emelb_head_range_request: kernel::attention's head-range event (src/emel/kernel/attention/events.hpp:18-31)."""
    _fields_ = [("query", C.c_void_p), ("query_count", C.c_uint64), ("key_cache", C.c_void_p), ("key_count", C.c_uint64),
                ("value_cache", C.c_void_p), ("value_count", C.c_uint64), ("output", C.c_void_p), ("output_count", C.c_uint64),
                ("layer_offset", C.c_uint64), ("hidden_dim", C.c_int32), ("head_dim", C.c_int32), ("head_begin", C.c_int32),
                ("head_end", C.c_int32), ("position_capacity", C.c_int32), ("physical_begin", C.c_int32),
                ("valid_positions", C.c_int32)]


class TensorState(C.Structure):
    _fields_ = [("lifecycle_state", C.c_uint8), ("buffer", C.c_void_p), ("buffer_bytes", C.c_uint64),
                ("host", C.c_void_p), ("tensor_type", C.c_int32)]


class Diag(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "optimized_flash_dispatch_calls", "shared_flash_dispatch_calls", "optimized_q4_dispatch_calls",
        "optimized_q4_vector_dispatch_calls", "optimized_q6_dispatch_calls", "optimized_q6_vector_dispatch_calls",
        "optimized_q6_vector_argmax_dispatch_calls", "optimized_q8_0_dispatch_calls", "optimized_q4_0_dispatch_calls",
        "rejected_dispatch_calls", "kernel_launches", "h2d_bytes", "d2h_bytes")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


class BackendError(RuntimeError):
    pass


_lib = None

# every symbol include/emelb.h declares: (name, argtypes)
_P = C.c_void_p
_SIGNATURES = {
    "emelb_create": [C.c_int, C.POINTER(_P)],
    "emelb_destroy": [_P],
    "emelb_sync": [_P],
    "emelb_get_stream": [_P, C.POINTER(_P)],
    "emelb_diagnostics": [_P, C.POINTER(Diag)],
    "emelb_set_attention_mode": [_P, C.c_int],
    "emelb_set_upload_route": [_P, C.c_int32, C.c_int32],
    "emelb_set_peer_wait_ms": [_P, C.c_uint32],
    "emelb_selftest_wait_timeout": [_P, C.c_uint32],
    "emelb_residency_upload": [_P, C.c_int32, _P, C.c_uint64, C.c_int32, C.POINTER(_P)],
    "emelb_residency_evict": [_P, C.c_int32],
    "emelb_residency_state": [_P, C.c_int32, C.POINTER(TensorState)],
    "emelb_device_alloc": [_P, C.c_uint64, C.POINTER(_P)],
    "emelb_device_free": [_P, _P],
    "emelb_copy_to_device": [_P, _P, _P, C.c_uint64],
    "emelb_copy_to_host": [_P, _P, _P, C.c_uint64],
    "emelb_can_run": [_P, C.c_uint32, C.POINTER(Op)],
    "emelb_mul_mat": [_P, C.POINTER(Op)],
    "emelb_mul_mat_argmax": [_P, C.POINTER(Op)],
    "emelb_prepare_rhs": [_P, C.POINTER(View), C.c_int32],
    "emelb_mul_mat_prepared": [_P, C.POINTER(Op)],
    "emelb_flash_attn_ext": [_P, C.POINTER(Op)],
    "emelb_rms_norm": [_P, C.POINTER(Op)],
    "emelb_rope": [_P, C.POINTER(Op)],
    "emelb_glu": [_P, C.POINTER(Op)],
    "emelb_attention_head_range_can_run": [C.POINTER(HeadRangeRequest)],
    "emelb_attention_head_range": [_P, C.POINTER(HeadRangeRequest)],
    "emelb_quantize": [_P, C.POINTER(View), C.POINTER(View)],
    "emelb_dequantize": [_P, C.POINTER(View), C.POINTER(View)],
    "emelb_graph_begin": [_P],
    "emelb_graph_end": [_P, C.POINTER(_P)],
    "emelb_graph_launch": [_P, _P],
    "emelb_graph_destroy": [_P, _P],
    "emelb_mul_mat_vec_noalloc": [C.c_int, _P, C.c_int32, _P, C.c_uint64, C.c_uint64, _P, _P, C.c_char_p, C.c_uint64],
    "emelb_synth_fill": [_P, _P, C.c_int32, C.c_uint64, C.c_uint64, C.c_float, C.c_uint64],
    "emelb_comm_unique_id": [_P, C.c_uint64],
    "emelb_comm_init": [_P, C.c_int32, C.c_int32, _P, C.c_uint64],
    "emelb_mul_mat_prepared_group": [_P, C.POINTER(Op), C.c_uint32],
    "emelb_flash_attn_batch": [_P, _P, _P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_float],
    "emelb_comm_destroy": [_P],
    "emelb_all_gather_rows": [_P, _P, C.c_uint64, C.c_uint64],
    "emelb_row_slice": [C.POINTER(Op), C.c_uint32, C.c_uint32, C.POINTER(Op), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)],
}


def declared_symbols():
    from . import gguf as _gguf, llama as _llama, window as _window
    return sorted(list(_SIGNATURES) + list(_llama.SIGNATURES) + list(_gguf.SIGNATURES) + list(_window.SIGNATURES))


def lib():
    """The loaded C-ABI library; raises when it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise BackendError(f"{LIB_PATH} is missing: build it with `python emel.cpp_b200/build.py` "
                               "(this backend has no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        for name, args in _SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = C.c_uint32
            fn.argtypes = args
        from . import gguf as _gguf, llama as _llama, window as _window
        _llama.register(_lib)
        _gguf.register(_lib)
        _window.register(_lib)
    return _lib


def row_bytes(t: int, k: int) -> int:
    return k // BLOCK_ELEMS[t] * BLOCK_BYTES[t]


def ptr(a) -> int:
    """Address of a numpy array, a torch tensor, or a raw integer address."""
    if hasattr(a, "ctypes"):
        return a.ctypes.data
    if hasattr(a, "data_ptr"):
        return a.data_ptr()
    return int(a) if a is not None else 0


def dense_view(data, t: int, ne) -> View:
    ne = list(ne) + [1] * (4 - len(ne))
    v = View()
    v.data = ptr(data)
    v.type = t
    stride = {F32: 4, F16: 2, I32: 4}[t]
    for i in range(4):
        v.ne[i] = ne[i]
        v.nb[i] = stride
        stride *= ne[i]
    return v


def quant_view(data, t: int, k: int, m: int) -> View:
    """{k, m} rows of native blocks, the layout the reference's guards require."""
    v = View()
    v.data = ptr(data)
    v.type = t
    rb = row_bytes(t, k)
    v.ne[0], v.ne[1], v.ne[2], v.ne[3] = k, m, 1, 1
    v.nb[0], v.nb[1], v.nb[2], v.nb[3] = 1, rb, rb * m, rb * m
    return v


def mul_mat_op(w, t, k, m, x, n, y, index_out=None, src1_type=F32) -> Op:
    op = Op()
    op.src0 = quant_view(w, t, k, m)
    if src1_type == F32:
        op.src1 = dense_view(x, F32, [n, k])
    else:  # pre-quantized vector form
        rb = row_bytes(src1_type, k)
        v = View()
        v.data, v.type = ptr(x), src1_type
        v.ne[0], v.ne[1], v.ne[2], v.ne[3] = 1, k, 1, 1
        v.nb[0], v.nb[1], v.nb[2], v.nb[3] = 1, rb, rb, rb
        op.src1 = v
    op.dst = dense_view(y, F32, [n, m] if index_out is None else [1, 1])
    if index_out is not None:
        op.index_out = C.cast(ptr(index_out), C.POINTER(C.c_int32))
    return op


def flash_op(q, kc, vc, dst, head_dim, heads, kv_heads, tokens, capacity, scale=None, masked_total=None) -> Op:
    """Request of make_flash_attn_request (src/emel/text/generator/detail.hpp:3232-3279)."""
    import struct
    op = Op()
    op.src0 = dense_view(q, F32, [head_dim, 1, heads])
    for name, buf in (("src1", kc), ("src2", vc)):
        v = View()
        v.data, v.type = ptr(buf), F16
        v.ne[0], v.ne[1], v.ne[2], v.ne[3] = head_dim, tokens, kv_heads, 1
        v.nb[0], v.nb[1] = 2, 2 * head_dim
        v.nb[2] = 2 * capacity * head_dim
        v.nb[3] = v.nb[2] * kv_heads
        setattr(op, name, v)
    op.dst = dense_view(dst, F32, [head_dim, 1, heads])
    if scale is not None:
        raw = struct.pack("<f", scale) + (struct.pack("<I", masked_total) if masked_total is not None else b"")
        for i, b in enumerate(raw):
            op.op_params[i] = b
        op.op_params_size = len(raw)
    return op


def head_range_request(query, key_cache, value_cache, output, layer_offset, hidden_dim, head_dim, head_begin, head_end,
                       position_capacity, physical_begin, valid_positions, counts=None) -> "HeadRangeRequest":
    """kernel::attention's head_range_request (src/emel/kernel/attention/events.hpp:18-31); counts default to the
    arrays' element counts."""
    r = HeadRangeRequest()
    sizes = counts or [getattr(a, "size", 0) for a in (query, key_cache, value_cache, output)]
    r.query, r.key_cache, r.value_cache, r.output = ptr(query), ptr(key_cache), ptr(value_cache), ptr(output)
    r.query_count, r.key_count, r.value_count, r.output_count = sizes
    r.layer_offset, r.hidden_dim, r.head_dim = layer_offset, hidden_dim, head_dim
    r.head_begin, r.head_end, r.position_capacity = head_begin, head_end, position_capacity
    r.physical_begin, r.valid_positions = physical_begin, valid_positions
    return r


def strided_view(data, t: int, ne, nb) -> View:
    """A view with explicit byte strides (any valid layout)."""
    v = View()
    v.data, v.type = ptr(data), t
    for i in range(4):
        v.ne[i] = ne[i] if i < len(ne) else 1
        v.nb[i] = nb[i] if i < len(nb) else (nb[-1] * ne[len(nb) - 1] if i == len(nb) else v.nb[i - 1] * v.ne[i - 1])
    return v


def rms_norm_op(src: View, dst: View, eps: float) -> Op:
    """op_rms_norm request: op_params = {f32 eps} (src/emel/kernel/detail.hpp:4547-4553)."""
    import struct
    op = Op()
    op.src0, op.dst = src, dst
    for i, b in enumerate(struct.pack("<f", eps)):
        op.op_params[i] = b
    op.op_params_size = 4
    return op


def rope_op(src: View, positions: View, dst: View, n_dims: int, mode: int = 0, freq_base: float = 10000.0,
            freq_scale: float = 1.0, ext_factor: float = 0.0, attn_factor: float = 1.0) -> Op:
    """op_rope request with ggml's parameter layout (src/emel/kernel/detail.hpp:4650-4678)."""
    import struct
    op = Op()
    op.src0, op.src1, op.dst = src, positions, dst
    raw = struct.pack("<5i6f", 0, n_dims, mode, 0, 0, freq_base, freq_scale, ext_factor, attn_factor, 0.0, 0.0)
    for i, b in enumerate(raw):
        op.op_params[i] = b
    op.op_params_size = len(raw)
    return op


class Backend:
    """One backend context = one kernel actor lane."""

    def __init__(self, device: int = 0):
        self._h = _P()
        err = lib().emelb_create(device, C.byref(self._h))
        if err != OK:
            raise BackendError(f"emelb_create failed with error mask {err}")
        self.device = device
        self.last_error = OK

    # -- lifetime
    def close(self):
        if self._h:
            lib().emelb_destroy(self._h)
            self._h = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def _ret(self, err: int) -> bool:
        self.last_error = err
        return err == OK

    def sync(self) -> bool:
        return self._ret(lib().emelb_sync(self._h))

    def stream(self) -> int:
        s = _P()
        lib().emelb_get_stream(self._h, C.byref(s))
        return s.value or 0

    def diagnostics(self) -> dict:
        d = Diag()
        lib().emelb_diagnostics(self._h, C.byref(d))
        return d.as_dict()

    def set_attention_mode(self, mode: int) -> bool:
        return self._ret(lib().emelb_set_attention_mode(self._h, mode))

    def rms_norm(self, op: Op) -> bool:
        return self._ret(lib().emelb_rms_norm(self._h, C.byref(op)))

    def rope(self, op: Op) -> bool:
        return self._ret(lib().emelb_rope(self._h, C.byref(op)))

    def attention_head_range(self, request: "HeadRangeRequest") -> bool:
        return self._ret(lib().emelb_attention_head_range(self._h, C.byref(request)))

    def glu(self, op: Op) -> bool:
        return self._ret(lib().emelb_glu(self._h, C.byref(op)))

    def set_peer_wait_ms(self, limit_ms: int) -> bool:
        return self._ret(lib().emelb_set_peer_wait_ms(self._h, limit_ms))

    def selftest_wait_timeout(self, limit_ms: int) -> bool:
        """Enqueue a peer join nobody answers; the following sync() must then report a failure."""
        return self._ret(lib().emelb_selftest_wait_timeout(self._h, limit_ms))

    def set_upload_route(self, route: str = "ring", threads: int = 0) -> bool:
        """route: "ring" (page-locked staging ring, the default), "plain" or "register"; threads 0 = automatic."""
        code = {"ring": 0, "plain": 1, "register": 2}[route]
        return self._ret(lib().emelb_set_upload_route(self._h, code, threads))

    # -- residency
    def upload(self, tensor_id: int, host, nbytes: int | None = None, tensor_type: int = 0) -> int:
        nbytes = int(host.nbytes) if nbytes is None else nbytes
        dev = _P()
        if not self._ret(lib().emelb_residency_upload(self._h, tensor_id, ptr(host), nbytes, tensor_type, C.byref(dev))):
            raise BackendError(f"residency upload failed with error mask {self.last_error}")
        return dev.value

    def evict(self, tensor_id: int) -> bool:
        return self._ret(lib().emelb_residency_evict(self._h, tensor_id))

    def state(self, tensor_id: int) -> TensorState:
        s = TensorState()
        lib().emelb_residency_state(self._h, tensor_id, C.byref(s))
        return s

    def alloc(self, nbytes: int) -> int:
        dev = _P()
        if not self._ret(lib().emelb_device_alloc(self._h, nbytes, C.byref(dev))):
            raise BackendError(f"device alloc of {nbytes} bytes failed with error mask {self.last_error}")
        return dev.value

    def free(self, dev: int) -> bool:
        return self._ret(lib().emelb_device_free(self._h, dev))

    def to_device(self, dev: int, host, nbytes: int | None = None) -> bool:
        return self._ret(lib().emelb_copy_to_device(self._h, dev, ptr(host), int(host.nbytes) if nbytes is None else nbytes))

    def to_host(self, host, dev: int, nbytes: int | None = None) -> bool:
        return self._ret(lib().emelb_copy_to_host(self._h, ptr(host), dev, int(host.nbytes) if nbytes is None else nbytes))

    # -- ops: `bool accepted`, reason in last_error
    def can_run(self, code: int, op: Op) -> bool:
        return lib().emelb_can_run(self._h, code, C.byref(op)) == OK

    def mul_mat(self, op: Op) -> bool:
        return self._ret(lib().emelb_mul_mat(self._h, C.byref(op)))

    def mul_mat_argmax(self, op: Op) -> bool:
        return self._ret(lib().emelb_mul_mat_argmax(self._h, C.byref(op)))

    def prepare_rhs(self, src1: View, weight_type: int) -> bool:
        return self._ret(lib().emelb_prepare_rhs(self._h, C.byref(src1), weight_type))

    def mul_mat_prepared(self, op: Op) -> bool:
        return self._ret(lib().emelb_mul_mat_prepared(self._h, C.byref(op)))

    def mul_mat_prepared_group(self, ops) -> bool:
        """Several products against the prepared column; one launch when the grouped kernel takes them."""
        arr = (Op * len(ops))(*ops)
        return self._ret(lib().emelb_mul_mat_prepared_group(self._h, arr, len(ops)))

    def flash_attn_ext(self, op: Op) -> bool:
        return self._ret(lib().emelb_flash_attn_ext(self._h, C.byref(op)))

    def flash_attn_batch(self, q_dev, k_dev, v_dev, dst_dev, head_dim, heads, kv_heads, batch, pos0, cache_head_stride, scale) -> bool:
        """Causal attention of `batch` prompt tokens over the f16 cache; device pointers, token-fastest q / dst."""
        return self._ret(lib().emelb_flash_attn_batch(self._h, q_dev, k_dev, v_dev, dst_dev, head_dim, heads, kv_heads, batch,
                                                      pos0, cache_head_stride, scale))

    def quantize(self, src: View, dst: View) -> bool:
        return self._ret(lib().emelb_quantize(self._h, C.byref(src), C.byref(dst)))

    def dequantize(self, src: View, dst: View) -> bool:
        return self._ret(lib().emelb_dequantize(self._h, C.byref(src), C.byref(dst)))

    # -- stream capture of device-resident call sequences
    def graph_begin(self) -> bool:
        return self._ret(lib().emelb_graph_begin(self._h))

    def graph_end(self) -> int:
        g = _P()
        if not self._ret(lib().emelb_graph_end(self._h, C.byref(g))):
            raise BackendError(f"graph capture failed with error mask {self.last_error}")
        return g.value

    def graph_launch(self, graph: int) -> bool:
        return self._ret(lib().emelb_graph_launch(self._h, graph))

    def graph_destroy(self, graph: int) -> bool:
        return self._ret(lib().emelb_graph_destroy(self._h, graph))

    def synth_fill(self, dev: int, t: int, elems: int, seed: int, sigma: float, offset: int = 0) -> bool:
        """N(0, sigma) synthetic data, f32 or block-encoded on the device."""
        return self._ret(lib().emelb_synth_fill(self._h, dev, t, elems, seed, sigma, offset))


    # ---- row-shard exchange (one rank per GPU)
    def comm_init(self, rank: int, world: int, comm_id: bytes) -> bool:
        """Join the exchange group; comm_id comes from comm_unique_id() on rank 0, broadcast by the caller."""
        buf = (C.c_uint8 * COMM_ID_BYTES).from_buffer_copy(comm_id)
        return self._ret(lib().emelb_comm_init(self._h, rank, world, C.addressof(buf), COMM_ID_BYTES))

    def comm_destroy(self) -> bool:
        return self._ret(lib().emelb_comm_destroy(self._h))

    def all_gather_rows(self, dst_dev: int, rows_per_rank: int, row_floats: int = 1) -> bool:
        """Join the ranks' row intervals of a full f32 result (own interval already in place)."""
        return self._ret(lib().emelb_all_gather_rows(self._h, dst_dev, rows_per_rank, row_floats))


COMM_ID_BYTES = 128


def comm_unique_id() -> bytes:
    buf = (C.c_uint8 * COMM_ID_BYTES)()
    err = lib().emelb_comm_unique_id(C.addressof(buf), COMM_ID_BYTES)
    if err != OK:
        raise BackendError(f"emelb_comm_unique_id failed with error mask {err}")
    return bytes(buf)


def mul_mat_vec_noalloc(device: int, stream: int, weight_type: int, weights_dev: int, k: int, m: int, x_dev: int, y_dev: int):
    """Context-free mat-vec that allocates nothing (fixed scratch inside the library; K <= 32768).
    Returns (error mask, message)."""
    buf = C.create_string_buffer(256)
    err = lib().emelb_mul_mat_vec_noalloc(device, stream, weight_type, weights_dev, k, m, x_dev, y_dev, buf, 256)
    return err, buf.value.decode()


def row_slice(op: Op, lane: int, lanes: int):
    out, b, c = Op(), C.c_uint64(), C.c_uint64()
    err = lib().emelb_row_slice(C.byref(op), lane, lanes, C.byref(out), C.byref(b), C.byref(c))
    if err != OK:
        raise BackendError(f"row_slice rejected: {err}")
    return out, b.value, c.value
