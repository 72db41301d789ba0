"""numpy restatement of the reference's row operators beside the matrix product:
op_rms_norm, op_rope (adjacent-pair and half-split pairing) and the op_glu guard.
TEST INFRASTRUCTURE ONLY, like the rest of this directory.

Each function takes the same request struct (bindings.Op) the compiled checkers
take and reads / writes the caller's buffers through the views' byte strides.
Pinned against the reference's own code (oracle/_ref) by tests/test_row_ops.py.
"""
from __future__ import annotations

import ctypes as C
import math
import struct

import numpy as np

from . import bindings as ob

I32 = 26  # ggml's dtype code for int32 (src/emel/kernel/events.hpp dtype table)
OP_RMS_NORM, OP_ROPE, OP_GLU = 4, 5, 6
ELEM = {ob.F32: 4, ob.F16: 2, I32: 4}


def _param(op, slot, fmt):
    """read_op_param_{i32,f32} (src/emel/kernel/detail.hpp:4525-4543): slot must lie inside op_params_size."""
    if op.op_params_size > 64 or (slot + 1) * 4 > op.op_params_size:
        return None
    return struct.unpack_from(fmt, bytes(op.op_params), slot * 4)[0]


def _layout_ok(v):
    """has_valid_tensor_layout (src/emel/kernel/detail.hpp:1720-1736): a known element size and either no explicit
    strides (nb[0] == 0: dense is implied) or nb[0] a positive multiple of the element size and no dimension
    longer than one with a zero stride."""
    es = ELEM.get(v.type)
    if es is None:
        return False
    if v.nb[0] == 0:
        return True
    return v.nb[0] >= es and v.nb[0] % es == 0 and not any(v.ne[i] > 1 and v.nb[i] == 0 for i in range(4))


def _strides(v):
    """tensor_stride_bytes (src/emel/kernel/detail.hpp:1710-1718)."""
    if v.nb[0] == 0:
        s, out = ELEM[v.type], []
        for i in range(4):
            out.append(s)
            s *= v.ne[i]
        return out
    return [v.nb[i] for i in range(4)]


def _array(v, dtype):
    """The view as a numpy array indexed [i3, i2, i1, i0] over the caller's memory."""
    nb = _strides(v)
    span = sum((v.ne[i] - 1) * nb[i] for i in range(4)) + ELEM[v.type]
    raw = np.ctypeslib.as_array(C.cast(v.data, C.POINTER(C.c_uint8)), shape=(span,))
    base = raw[:ELEM[v.type]].view(dtype)
    return np.lib.stride_tricks.as_strided(base, shape=(v.ne[3], v.ne[2], v.ne[1], v.ne[0]),
                                           strides=(nb[3], nb[2], nb[1], nb[0]), writeable=True)


def _same_shape(a, b):
    return all(a.ne[i] == b.ne[i] for i in range(4))


def _validate(op, srcs):
    """validate_dispatch_request (src/emel/kernel/detail.hpp:1919-1927): the named sources and dst have data and
    a known type."""
    views = [getattr(op, s) for s in srcs] + [op.dst]
    count = lambda v: v.ne[0] * v.ne[1] * v.ne[2] * v.ne[3]
    return op.op_params_size <= 64 and all(v.data and v.type in ELEM and _layout_ok(v) and count(v) > 0 for v in views)


def can_run_rms_norm(op) -> bool:
    """can_run_norm_row_op (src/emel/kernel/detail.hpp:4555-4565)."""
    if not _validate(op, ["src0"]):
        return False
    eps = _param(op, 0, "<f")
    return bool(op.src0.ne[0] > 0 and _same_shape(op.src0, op.dst) and op.src0.type == ob.F32 and op.dst.type == ob.F32 and
                _layout_ok(op.src0) and _layout_ok(op.dst) and eps is not None and math.isfinite(eps) and eps >= 0.0)


def rope_params(op):
    vals = [_param(op, 1, "<i"), _param(op, 2, "<i")] + [_param(op, s, "<f") for s in (5, 6, 7, 8)]
    return None if any(v is None for v in vals) else vals


def can_run_rope(op) -> bool:
    """can_run_rope (src/emel/kernel/detail.hpp:4680-4704)."""
    if not _validate(op, ["src0"]) or not op.src1.data:  # positions are not a "required src1" of the dispatch check
        return False
    p = rope_params(op)
    if p is None:
        return False
    n_dims, _mode, base, scale, ext, attn = p
    return bool(_same_shape(op.src0, op.dst) and op.src0.ne[0] > 0 and op.src0.type == ob.F32 and op.dst.type == ob.F32 and
                op.src1.type == I32 and not op.src2.data and _layout_ok(op.src0) and _layout_ok(op.src1) and
                _layout_ok(op.dst) and op.src1.ne[0] == op.src0.ne[2] and n_dims > 0 and n_dims % 2 == 0 and
                n_dims <= op.src0.ne[0] and ext == 0.0 and math.isfinite(base) and base > 0.0 and
                math.isfinite(scale) and scale > 0.0 and math.isfinite(attn))


def can_run(code, op) -> bool:
    if code == OP_RMS_NORM:
        return can_run_rms_norm(op)
    if code == OP_ROPE:
        return can_run_rope(op)
    if code == OP_GLU:
        return False  # no branch of can_execute_scalar takes op_glu (src/emel/kernel/detail.hpp:5166-5203)
    raise ValueError(code)


def rms_norm(op) -> bool:
    """run_rms_norm (src/emel/kernel/detail.hpp:4567-4602): per row, the f32 squares are summed in ascending
    order in f64, mean = f32(sum / cols), scale = 1 / sqrt(mean + eps) in f32, y = x * scale."""
    if not can_run_rms_norm(op):
        return False
    eps = np.float32(_param(op, 0, "<f"))
    x, y = _array(op.src0, np.float32), _array(op.dst, np.float32)
    cols = op.src0.ne[0]
    for i3 in range(op.src0.ne[3]):
        for i2 in range(op.src0.ne[2]):
            for i1 in range(op.src0.ne[1]):
                row = x[i3, i2, i1].astype(np.float32)
                sq = (row * row).astype(np.float64)
                total = 0.0
                for v in sq:  # ascending order; np.sum would pair the terms
                    total += float(v)
                mean = np.float32(total / float(cols))
                scale = np.float32(1.0) / np.sqrt(np.float32(mean + eps), dtype=np.float32)
                y[i3, i2, i1] = row * scale
    return True


def rope(op) -> bool:
    """run_rope_as (src/emel/kernel/detail.hpp:4706-4765): theta starts at the position and is multiplied by
    pow(freq_base, -2 / n_dims) pair after pair, all in f32; the angle is theta * freq_scale and the rotation
    x0' = x0 cos - x1 sin, x1' = x0 sin + x1 cos with cos / sin already multiplied by attn_factor.  mode 0
    pairs (2p, 2p+1), mode 2 pairs (p, p + n_dims / 2); columns past n_dims are copied.
    cos / sin / pow go through f64 here and the products are rounded one by one, so against the compiled reference
    (libm's f32 functions, products the compiler may fuse) results agree to a few units in the last place only."""
    if not can_run_rope(op):
        return False
    n_dims, mode, base, fscale, _ext, attn = rope_params(op)
    if mode not in (0, 2):
        return False
    half = n_dims // 2
    theta_scale = np.float32(math.pow(np.float32(base), np.float32(-2.0) / np.float32(n_dims)))
    x, y = _array(op.src0, np.float32), _array(op.dst, np.float32)
    pos = _array(op.src1, np.int32)
    f32 = np.float32
    for i3 in range(op.src0.ne[3]):
        for i2 in range(op.src0.ne[2]):
            theta0 = f32(pos[0, 0, 0, i2])
            for i1 in range(op.src0.ne[1]):
                row = x[i3, i2, i1].astype(np.float32)
                out = row.copy()
                theta = theta0
                for p in range(half):
                    ang = f32(theta * f32(fscale))
                    c = f32(f32(math.cos(float(ang))) * f32(attn))
                    s = f32(f32(math.sin(float(ang))) * f32(attn))
                    a, b = (p, p + half) if mode == 2 else (2 * p, 2 * p + 1)
                    x0, x1 = row[a], row[b]
                    out[a] = f32(f32(x0 * c) - f32(x1 * s))
                    out[b] = f32(f32(x0 * s) + f32(x1 * c))
                    theta = f32(theta * theta_scale)
                y[i3, i2, i1] = out
    return True


# ---- kernel::attention's head-range event (src/emel/kernel/attention/actions.hpp:15-96), scalar route
def f32_to_bf16_bits(x):
    """ggml's round-to-nearest-even with NaN quieting (src/emel/kernel/detail.hpp:3944-3952), vectorised."""
    u = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7fffffff) > 0x7f800000
    r = ((u + (0x7fff + ((u >> 16) & 1))) >> 16) & 0xffff
    return np.where(nan, ((u >> 16) | 64) & 0xffff, r).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.asarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def head_range_can_run(query, key, value, output, layer_offset, hidden_dim, head_dim, head_begin, head_end, capacity,
                       physical_begin, valid):
    """guard_request_shape_supported (src/emel/kernel/attention/guards.hpp:28-90) for numpy arrays (which are aligned
    and cannot overlap unless they share memory)."""
    if (hidden_dim <= 0 or head_dim <= 0 or head_begin < 0 or head_end <= head_begin or capacity <= 0 or physical_begin < 0 or
            physical_begin >= capacity or valid <= 0 or valid > capacity):
        return False
    if head_end > hidden_dim // head_dim or head_dim > 8192 or capacity > 8192:
        return False
    need = layer_offset + capacity * hidden_dim
    if query.size < hidden_dim or key.size < need or value.size < need or output.size < (head_end - head_begin) * head_dim:
        return False
    return not (np.shares_memory(output, query) or np.shares_memory(output, key) or np.shares_memory(output, value))


def head_range_attention(query, key, value, output, layer_offset, hidden_dim, head_dim, head_begin, head_end, capacity,
                         physical_begin, valid):
    """effect_execute_head_range.  Sums whose order the reference fixes are taken with cumsum (sequential); the
    exponentials go through f64 exp rounded to f32, which is not glibc's expf to the last bit, so against the compiled
    reference the result agrees to about 1e-6 relative only."""
    if not head_range_can_run(query, key, value, output, layer_offset, hidden_dim, head_dim, head_begin, head_end, capacity,
                              physical_begin, valid):
        return False
    f32 = np.float32
    scale = f32(1.0) / np.sqrt(f32(head_dim), dtype=np.float32)
    phys = (physical_begin + np.arange(valid)) % capacity
    for head in range(head_begin, head_end):
        ho = head * head_dim
        q = bf16_bits_to_f32(f32_to_bf16_bits(query[ho:ho + head_dim]))
        scores = np.full(capacity, -np.inf, np.float32)
        rows = layer_offset + phys[:, None] * hidden_dim + ho + np.arange(head_dim)[None, :]
        k = bf16_bits_to_f32(key[rows])
        prod = (k * q[None, :]).astype(np.float32).astype(np.float64)
        scores[phys] = np.cumsum(prod, axis=1)[:, -1].astype(np.float32) * scale
        mx = scores.max()
        with np.errstate(over="ignore", under="ignore"):
            e = np.exp((scores - mx).astype(np.float64)).astype(np.float32)
        total = np.cumsum(e.astype(np.float64))[-1]
        w = bf16_bits_to_f32(f32_to_bf16_bits(e * f32(1.0 / total)))
        v = bf16_bits_to_f32(value[rows])
        acc = np.cumsum((v * w[phys][:, None]).astype(np.float32).astype(np.float64), axis=0)[-1]
        output[(head - head_begin) * head_dim:(head - head_begin + 1) * head_dim] = acc.astype(np.float32)
    return True
