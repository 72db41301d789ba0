"""ctypes bindings for the two CPU checkers.  TEST INFRASTRUCTURE ONLY.

`port`  — oracle/libemel_oracle.so, the plain-C restatement (emel_oracle.c).
`ref`   — oracle/_ref/libemel_ref.so, the reference's own kernel headers
          compiled in place (ref_shim.cpp); None when it was never built.

Only tests/, the smoke check and the bench's CPU-baseline legs import this
module; the product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K, Q8_K = 0, 1, 2, 8, 12, 14, 15
OP_MUL_MAT, OP_MUL_MAT_ARGMAX, OP_FLASH_ATTN_EXT = 1, 2, 3

BLOCK_ELEMS = {Q4_0: 32, Q8_0: 32, Q4_K: 256, Q6_K: 256, Q8_K: 256}
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34, Q4_K: 144, Q6_K: 210, Q8_K: 292}
ELEM_SIZE = {F32: 4, F16: 2}


class View(C.Structure):
    _fields_ = [("data", C.c_void_p), ("type", C.c_uint8), ("ne", C.c_uint64 * 4), ("nb", C.c_uint64 * 4)]


class Op(C.Structure):
    _fields_ = [("src0", View), ("src1", View), ("src2", View), ("dst", View),
                ("op_params", C.c_uint8 * 64), ("op_params_size", C.c_uint32),
                ("index_out", C.POINTER(C.c_int32))]


def row_bytes(t: int, k: int) -> int:
    return k // BLOCK_ELEMS[t] * BLOCK_BYTES[t]


def ptr(a) -> int:
    return a.ctypes.data if isinstance(a, np.ndarray) else int(a)


def dense_view(data, t: int, ne) -> View:
    ne = list(ne) + [1] * (4 - len(ne))
    v = View()
    v.data = ptr(data)
    v.type = t
    es = ELEM_SIZE[t]
    stride = es
    for i in range(4):
        v.ne[i] = ne[i]
        v.nb[i] = stride
        stride *= ne[i]
    return v


def quant_view(data, t: int, k: int, m: int) -> View:
    """make_quantized_src of the reference tests: {k, m} rows of native blocks."""
    v = View()
    v.data = ptr(data)
    v.type = t
    rb = row_bytes(t, k)
    v.ne[0], v.ne[1], v.ne[2], v.ne[3] = k, m, 1, 1
    v.nb[0], v.nb[1], v.nb[2], v.nb[3] = 1, rb, rb * m, rb * m
    return v


def mul_mat_op(w, t, k, m, x, n, y, index_out=None) -> Op:
    op = Op()
    op.src0 = quant_view(w, t, k, m)
    op.src1 = dense_view(x, F32, [n, k])
    op.dst = dense_view(y, F32, [n, m] if index_out is None else [1, 1])
    if index_out is not None:
        op.index_out = C.cast(ptr(index_out), C.POINTER(C.c_int32))
    return op


def flash_op(q, kc, vc, dst, head_dim, heads, kv_heads, tokens, capacity, scale=None, masked_total=None) -> Op:
    """Request shape of make_flash_attn_request (text/generator/detail.hpp:3232-3279)."""
    op = Op()
    op.src0 = dense_view(q, F32, [head_dim, 1, heads])
    for name, buf in (("src1", kc), ("src2", vc)):
        v = View()
        v.data = ptr(buf)
        v.type = F16
        v.ne[0], v.ne[1], v.ne[2], v.ne[3] = head_dim, tokens, kv_heads, 1
        v.nb[0], v.nb[1] = 2, 2 * head_dim
        v.nb[2] = 2 * capacity * head_dim
        v.nb[3] = v.nb[2] * kv_heads
        setattr(op, name, v)
    op.dst = dense_view(dst, F32, [head_dim, 1, heads])
    if scale is not None:
        raw = np.array([scale], np.float32).tobytes()
        n = 4
        if masked_total is not None:
            raw += np.array([masked_total], np.uint32).tobytes()
            n = 8
        for i, b in enumerate(raw):
            op.op_params[i] = b
        op.op_params_size = n
    return op


# where the reference checkout lies when it is present: EMEL_REFERENCE_DIR, else a `reference` directory beside
# this repository (the Makefile's default too)
REFERENCE_DIR = os.environ.get("EMEL_REFERENCE_DIR") or os.path.abspath(os.path.join(HERE, "..", "..", "reference"))


def _load(path):
    return C.CDLL(path) if os.path.exists(path) else None


def build(force: bool = False) -> None:
    """Compile both checkers (the reference one only where its checkout exists)."""
    if force or not os.path.exists(os.path.join(HERE, "libemel_oracle.so")) or \
            (os.path.isdir(os.path.join(REFERENCE_DIR, "src", "emel", "kernel")) and
             not os.path.exists(os.path.join(HERE, "_ref", "libemel_ref.so"))):
        subprocess.run(["make", "-C", HERE, f"REFERENCE={REFERENCE_DIR}"] + (["-B"] if force else []), check=True,
                       stdout=subprocess.DEVNULL)


class _Lib:
    """Uniform wrapper: same method names over the port and the reference build."""

    def __init__(self, lib, prefix):
        self.lib, self.p = lib, prefix
        g = lambda n: getattr(lib, prefix + n)
        g("fp16_to_fp32").restype = C.c_float
        g("fp16_to_fp32").argtypes = [C.c_uint16]
        g("fp32_to_fp16").restype = C.c_uint16
        g("fp32_to_fp16").argtypes = [C.c_float]
        for n in ("quantize_q8_k", "quantize_q8_0"):
            g(n).restype = None
            g(n).argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_int64]
        g("quantize_q4_0").restype = None
        g("quantize_q4_0").argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        g("dequantize_row").restype = C.c_int
        g("dequantize_row").argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]

    def f(self, name):
        return getattr(self.lib, self.p + name)

    # -- scalars
    def fp16_to_fp32(self, h):
        return self.f("fp16_to_fp32")(int(h))

    def fp32_to_fp16(self, x):
        return self.f("fp32_to_fp16")(float(x))

    # -- quantizers: x is f32 [k, n] token-fastest (or a vector); column j
    def quantize(self, t, x, k, n=1, col=0):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(row_bytes(t, k), np.uint8)
        fn = self.f("quantize_q8_k" if t == Q8_K else "quantize_q8_0")
        fn(x.ctypes.data + 4 * col, n, out.ctypes.data, k)
        return out

    def quantize_q4_0(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(row_bytes(Q4_0, x.size), np.uint8)
        self.f("quantize_q4_0")(x.ctypes.data, out.ctypes.data, x.size)
        return out

    def dequantize(self, t, blocks, k, m=1):
        blocks = np.ascontiguousarray(blocks, np.uint8)
        out = np.zeros((m, k), np.float32)
        rb = row_bytes(t, k)
        for i in range(m):
            assert self.f("dequantize_row")(t, blocks.ctypes.data + i * rb, out[i].ctypes.data, k)
        return out


class Port(_Lib):
    def __init__(self, lib):
        super().__init__(lib, "orc_")
        for n in ("can_run_mul_mat", "mul_mat", "mul_mat_argmax", "can_run_flash_attn", "flash_attn"):
            self.f(n).restype = C.c_int
            self.f(n).argtypes = [C.POINTER(Op)]
        self.f("flash_attn_f64").restype = C.c_int
        self.f("flash_attn_f64").argtypes = [C.POINTER(Op), C.c_void_p]
        self.f("row_dot").restype = C.c_float
        self.f("row_dot").argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_uint64]
        self.f("encode_rows").restype = C.c_int
        self.f("encode_rows").argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64]
        self.f("row_slice").restype = None
        self.f("row_slice").argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]

    def can_run(self, code, op):
        if code == OP_FLASH_ATTN_EXT:
            return bool(self.f("can_run_flash_attn")(C.byref(op)))
        if code == OP_MUL_MAT:
            return bool(self.f("can_run_mul_mat")(C.byref(op)))
        raise ValueError(code)

    def mul_mat(self, op):
        return bool(self.f("mul_mat")(C.byref(op)))

    def mul_mat_argmax(self, op):
        return bool(self.f("mul_mat_argmax")(C.byref(op)))

    def flash_attn(self, op):
        return bool(self.f("flash_attn")(C.byref(op)))

    def flash_attn_f64(self, op, heads, head_dim):
        out = np.zeros((heads, head_dim), np.float64)
        assert self.f("flash_attn_f64")(C.byref(op), out.ctypes.data)
        return out

    def row_dot(self, t, lhs, rhs, blocks):
        return self.f("row_dot")(t, ptr(lhs), ptr(rhs), blocks)

    def encode_rows(self, t, x, k, m):
        """Weight encoder: f32 [m, k] -> native blocks (own design for Q4_K/Q6_K)."""
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(m * row_bytes(t, k), np.uint8)
        assert self.f("encode_rows")(t, x.ctypes.data, out.ctypes.data, k, m)
        return out

    def row_slice(self, rows, lane, lanes):
        b, c = C.c_uint64(), C.c_uint64()
        self.f("row_slice")(rows, lane, lanes, C.byref(b), C.byref(c))
        return b.value, c.value


class Ref(_Lib):
    def __init__(self, lib):
        super().__init__(lib, "ref_")
        self.f("can_run").restype = C.c_int
        self.f("can_run").argtypes = [C.c_uint32, C.POINTER(Op)]
        for n in ("mul_mat_scalar", "mul_mat_avx2", "mul_mat_argmax", "flash_attn_scalar", "flash_attn_avx2", "rms_norm", "rope"):
            self.f(n).restype = C.c_int
            self.f(n).argtypes = [C.POINTER(Op)]
        self.f("mul_mat_avx2_lanes").restype = C.c_int
        self.f("mul_mat_avx2_lanes").argtypes = [C.POINTER(Op), C.c_uint32]
        for n in ("row_dot_scalar", "row_dot_avx2"):
            self.f(n).restype = C.c_float
            self.f(n).argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_uint64]

        self.f("gguf_probe").restype = C.c_uint32
        self.f("gguf_probe").argtypes = [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]
        self.f("gguf_parse").restype = C.c_uint32
        self.f("gguf_parse").argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]

    def can_run(self, code, op):
        return bool(self.f("can_run")(code, C.byref(op)))

    def head_range_can_run(self, request):
        fn = self.f("head_range_can_run")
        fn.restype, fn.argtypes = C.c_int, [C.c_void_p]
        return bool(fn(C.addressof(request)))

    def head_range(self, request):
        fn = self.f("head_range")
        fn.restype, fn.argtypes = C.c_int, [C.c_void_p]
        return bool(fn(C.addressof(request)))

    def rms_norm(self, op):
        return bool(self.f("rms_norm")(C.byref(op)))

    def rope(self, op):
        return bool(self.f("rope")(C.byref(op)))

    def gguf_probe(self, image: bytes):
        """-> (error, (tensor_count, kv_count, max_key_bytes, max_value_bytes, tensor_data_bytes))"""
        buf = np.frombuffer(image, np.uint8) if len(image) else np.zeros(0, np.uint8)
        req4, total = (C.c_uint32 * 4)(), C.c_uint64(0)
        err = self.f("gguf_probe")(buf.ctypes.data if len(image) else None, len(image), req4, C.byref(total))
        return err, (req4[0], req4[1], req4[2], req4[3], total.value)

    def gguf_parse(self, image: bytes):
        """-> (error, [(key, value type, payload)], [tensor record dicts]) through probe + parse"""
        err, req = self.gguf_probe(image)
        if err != 0:
            return err, [], []
        buf = np.frombuffer(image, np.uint8)
        arena = np.zeros(max(1, req[1] * (req[2] + req[3])), np.uint8)
        kv = np.zeros((max(1, req[1]), 5), np.uint32)
        ten = np.zeros((max(1, req[0]), 11), np.uint64)
        err = self.f("gguf_parse")(buf.ctypes.data, len(image), arena.ctypes.data, kv.ctypes.data, ten.ctypes.data)
        if err != 0:
            return err, [], []
        a = arena.tobytes()
        kvs = [(a[int(r[0]):int(r[0] + r[1])], int(r[4]), a[int(r[2]):int(r[2]) + int(r[3])]) for r in kv[:req[1]]]
        tensors = [{"name": image[int(r[0]):int(r[0] + r[1])], "type": int(np.int64(r[2])), "n_dims": int(r[3]),
                    "dims": tuple(int(x) for x in r[4:8]), "data_offset": int(r[8]), "file_offset": int(r[9]),
                    "data_size": int(r[10])} for r in ten[:req[0]]]
        return 0, kvs, tensors

    def mul_mat(self, op, route="scalar", lanes=1):
        if route == "scalar":
            return bool(self.f("mul_mat_scalar")(C.byref(op)))
        if lanes > 1:
            return bool(self.f("mul_mat_avx2_lanes")(C.byref(op), lanes))
        return bool(self.f("mul_mat_avx2")(C.byref(op)))

    def mul_mat_argmax(self, op):
        return bool(self.f("mul_mat_argmax")(C.byref(op)))

    def flash_attn(self, op, route="scalar"):
        return bool(self.f("flash_attn_" + route)(C.byref(op)))

    def row_dot(self, t, lhs, rhs, blocks, route="scalar"):
        return self.f("row_dot_" + route)(t, ptr(lhs), ptr(rhs), blocks)


_port = None
_ref = None


def port() -> Port:
    global _port
    if _port is None:
        build()
        _port = Port(C.CDLL(os.path.join(HERE, "libemel_oracle.so")))
    return _port


def ref():
    """The reference build, or None when oracle/_ref was never built."""
    global _ref
    if _ref is None:
        lib = _load(os.path.join(HERE, "_ref", "libemel_ref.so"))
        _ref = Ref(lib) if lib is not None else False
    return _ref or None


def rel_l2(a, b) -> float:
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / (den if den > 0 else 1.0))


# ---------------------------------------------------------------- decoder restatement (llama_oracle.c)
class LConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_vocab",
                                         "n_ctx", "rope_dim", "rope_neox", "kv_block")] + \
               [("rope_freq_base", C.c_float), ("rms_eps", C.c_float)]


class CpuLlama:
    """The reference generator's decode loop restated on the CPU.  `kernels` picks who does the
    matrix products and attention: "ref-avx2" / "ref-scalar" (the reference's own kernels from
    oracle/_ref) or "port" (emel_oracle.c)."""

    def __init__(self, cfg: dict, kernels: str = "port"):
        lib = port().lib
        r = ref()
        if kernels.startswith("ref") and r is None:
            raise RuntimeError("oracle/_ref is not built")
        if kernels == "ref-avx2":
            mm, fa = r.lib.ref_mul_mat_avx2, r.lib.ref_flash_attn_avx2
        elif kernels == "ref-scalar":
            mm, fa = r.lib.ref_mul_mat_scalar, r.lib.ref_flash_attn_scalar
        else:
            mm, fa = lib.orc_mul_mat, lib.orc_flash_attn
        self.cfg = LConfig(cfg["n_layer"], cfg["n_embd"], cfg["n_head"], cfg["n_head_kv"], cfg["head_dim"], cfg["n_ff"],
                           cfg["n_vocab"], cfg["n_ctx"], cfg.get("rope_dim", cfg["head_dim"]), cfg.get("rope_neox", 0),
                           cfg.get("kv_block", 16), cfg.get("rope_freq_base", 500000.0), cfg.get("rms_eps", 1e-5))
        lib.orc_llama_create.restype = C.c_void_p
        lib.orc_llama_create.argtypes = [C.POINTER(LConfig), C.c_void_p, C.c_void_p]
        lib.orc_llama_bind.restype = C.c_int
        lib.orc_llama_bind.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int]
        lib.orc_llama_decode.restype = C.c_int
        lib.orc_llama_decode.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        lib.orc_llama_destroy.argtypes = [C.c_void_p]
        self.lib = lib
        self.h = lib.orc_llama_create(C.byref(self.cfg), C.cast(mm, C.c_void_p), C.cast(fa, C.c_void_p))
        self.keep = []

    def bind(self, layer, role, data, t):
        self.keep.append(data)
        assert self.lib.orc_llama_bind(self.h, layer, role, ptr(data), t)

    def decode(self, token, position, want_logits=True):
        logits = np.zeros(self.cfg.n_vocab, np.float32) if want_logits else None
        assert self.lib.orc_llama_decode(self.h, token, position, logits.ctypes.data if want_logits else None)
        return logits

    def close(self):
        if self.h:
            self.lib.orc_llama_destroy(self.h)
            self.h = None


def cpu_rms_norm(x, w, eps):
    lib = port().lib
    out = np.zeros_like(x)
    lib.orc_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p]
    lib.orc_rms_norm(x.ctypes.data, w.ctypes.data, eps, x.size, out.ctypes.data)
    return out


def cpu_rope(vec, heads, head_dim, n_rot, neox, position, base):
    lib = port().lib
    out = np.ascontiguousarray(vec, np.float32).copy()
    lib.orc_rope.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
    lib.orc_rope(out.ctypes.data, heads, head_dim, n_rot, neox, position, base)
    return out


def cpu_swiglu(gate, up):
    lib = port().lib
    out = np.zeros_like(gate)
    lib.orc_swiglu.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    lib.orc_swiglu(gate.ctypes.data, up.ctypes.data, gate.size, out.ctypes.data)
    return out
