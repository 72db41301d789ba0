"""op_rms_norm / op_rope / op_glu: the guards of the C-ABI against the reference's, and the numpy
restatement (oracle/row_ops.py) against the reference's compiled code.  CPU only."""
import ctypes as C

import numpy as np
import pytest

import emel_cpp_b200 as eb
from oracle import bindings as ob
from oracle import row_ops
from tests.test_cabi import as_eb

I32 = row_ops.I32
ROPE_ULPS = 8  # numpy restatement vs compiled reference: f64 vs f32 libm calls, unfused vs fused products


def to_ob(op: eb.Op) -> ob.Op:
    out = ob.Op()
    C.memmove(C.byref(out), C.byref(op), C.sizeof(eb.Op))
    return out


def rms_request(x, y, eps=1e-5, params_size=None):
    op = eb.rms_norm_op(eb.dense_view(x, eb.F32, list(x.shape[::-1])), eb.dense_view(y, eb.F32, list(y.shape[::-1])), eps)
    if params_size is not None:
        op.op_params_size = params_size
    return op


def rope_request(x, pos, y, n_dims, mode=0, **kw):
    pv = eb.View()
    pv.data, pv.type = pos.ctypes.data, I32
    pv.ne[0], pv.ne[1], pv.ne[2], pv.ne[3] = pos.size, 1, 1, 1
    pv.nb[0], pv.nb[1], pv.nb[2], pv.nb[3] = 4, 4 * pos.size, 4 * pos.size, 4 * pos.size
    return eb.rope_op(eb.dense_view(x, eb.F32, list(x.shape[::-1])), pv, eb.dense_view(y, eb.F32, list(y.shape[::-1])), n_dims,
                      mode, **kw)


def guard_cases():
    keep = []

    def arr(*shape, dtype=np.float32):
        a = np.ones(shape, dtype)
        keep.append(a)
        return a

    cases = []
    x, y = arr(3, 64), arr(3, 64)
    cases.append(("rms ok", eb.OP_RMS_NORM, rms_request(x, y)))
    cases.append(("rms no params", eb.OP_RMS_NORM, rms_request(x, y, params_size=0)))
    cases.append(("rms short params", eb.OP_RMS_NORM, rms_request(x, y, params_size=3)))
    cases.append(("rms negative eps", eb.OP_RMS_NORM, rms_request(x, y, eps=-1.0)))
    cases.append(("rms nan eps", eb.OP_RMS_NORM, rms_request(x, y, eps=float("nan"))))
    cases.append(("rms zero eps", eb.OP_RMS_NORM, rms_request(x, y, eps=0.0)))
    cases.append(("rms shape mismatch", eb.OP_RMS_NORM, rms_request(x, arr(2, 64))))
    op = rms_request(x, y)
    op.dst.type = eb.F16
    cases.append(("rms f16 dst", eb.OP_RMS_NORM, op))
    op = rms_request(x, y)
    op.src0.data = None
    cases.append(("rms null src", eb.OP_RMS_NORM, op))
    op = rms_request(x, y)
    op.src0.nb[0] = 6
    cases.append(("rms misaligned stride", eb.OP_RMS_NORM, op))
    op = rms_request(x, y)
    op.src0.nb[1] = 0
    cases.append(("rms zero row stride", eb.OP_RMS_NORM, op))
    op = rms_request(x, y)
    op.op_params_size = 65
    cases.append(("rms params too long", eb.OP_RMS_NORM, op))
    wide = arr(3, 128)
    op = rms_request(x, y)
    op.src0.data, op.src0.nb[1], op.src0.nb[2], op.src0.nb[3] = wide.ctypes.data, 512, 1536, 1536
    cases.append(("rms strided rows", eb.OP_RMS_NORM, op))

    q, qo, pos = arr(1, 5, 4, 64), arr(1, 5, 4, 64), np.arange(5, dtype=np.int32)
    keep.append(pos)
    cases.append(("rope ok", eb.OP_ROPE, rope_request(q, pos, qo, 64)))
    cases.append(("rope neox", eb.OP_ROPE, rope_request(q, pos, qo, 32, 2)))
    cases.append(("rope timestep mode passes the guard", eb.OP_ROPE, rope_request(q, pos, qo, 64, 4)))
    cases.append(("rope odd dims", eb.OP_ROPE, rope_request(q, pos, qo, 63)))
    cases.append(("rope dims too wide", eb.OP_ROPE, rope_request(q, pos, qo, 66)))
    cases.append(("rope zero dims", eb.OP_ROPE, rope_request(q, pos, qo, 0)))
    cases.append(("rope ext factor", eb.OP_ROPE, rope_request(q, pos, qo, 64, ext_factor=0.5)))
    cases.append(("rope bad base", eb.OP_ROPE, rope_request(q, pos, qo, 64, freq_base=0.0)))
    cases.append(("rope inf scale", eb.OP_ROPE, rope_request(q, pos, qo, 64, freq_scale=float("inf"))))
    cases.append(("rope nan attn", eb.OP_ROPE, rope_request(q, pos, qo, 64, attn_factor=float("nan"))))
    cases.append(("rope wrong position count", eb.OP_ROPE, rope_request(q, pos[:4], qo, 64)))
    op = rope_request(q, pos, qo, 64)
    op.src1.type = eb.F32
    cases.append(("rope f32 positions", eb.OP_ROPE, op))
    op = rope_request(q, pos, qo, 64)
    op.src2.data = q.ctypes.data
    cases.append(("rope with frequency factors", eb.OP_ROPE, op))
    op = rope_request(q, pos, qo, 64)
    op.op_params_size = 32
    cases.append(("rope short params", eb.OP_ROPE, op))
    op = rope_request(q, pos, qo, 64)
    op.src1.data = None
    cases.append(("rope null positions", eb.OP_ROPE, op))
    op = rope_request(q, pos, qo, 64)
    op.src1.ne[1] = 0
    cases.append(("rope positions with an empty dimension", eb.OP_ROPE, op))

    g = arr(2, 64)
    op = eb.Op()
    op.src0, op.src1, op.dst = eb.dense_view(g, eb.F32, [64, 2]), eb.dense_view(g, eb.F32, [64, 2]), eb.dense_view(g, eb.F32, [64, 2])
    cases.append(("glu", eb.OP_GLU, op))
    return cases, keep


def test_guards_match_the_checker():
    cases, _keep = guard_cases()
    ref = ob.ref()
    verdicts = {}
    for name, code, op in cases:
        got = eb.lib().emelb_can_run(None, code, C.byref(op)) == eb.OK
        want = row_ops.can_run(code, to_ob(op))
        assert got == want, name
        if ref is not None:
            assert ref.can_run(code, to_ob(op)) == want, name
        verdicts[name] = got
    assert verdicts["rms ok"] and verdicts["rms strided rows"] and verdicts["rms zero eps"]
    assert verdicts["rope ok"] and verdicts["rope neox"]
    assert not verdicts["glu"] and not verdicts["rope ext factor"] and not verdicts["rms negative eps"]
    assert sum(verdicts.values()) >= 6


def rows(seed, *shape):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(shape) * rng.choice([1e-3, 1.0, 40.0], size=shape[:-1] + (1,))).astype(np.float32)


@pytest.mark.parametrize("shape", [(1, 256), (7, 4096), (2, 3, 5, 100)])
def test_rms_norm_restatement_is_the_reference(ref, shape):
    x = rows(11, *shape)
    a, b = np.zeros_like(x), np.zeros_like(x)
    assert ref.rms_norm(to_ob(rms_request(x, a, 1e-5)))
    assert row_ops.rms_norm(to_ob(rms_request(x, b, 1e-5)))
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def ulps(a, b):
    scale = np.spacing(np.maximum(np.abs(a), np.abs(b)).max(axis=-1, keepdims=True).astype(np.float32))
    return float((np.abs(a.astype(np.float64) - b.astype(np.float64)) / scale).max())


@pytest.mark.parametrize("mode,n_dims", [(0, 128), (2, 128), (0, 64), (2, 96)])
def test_rope_restatement_tracks_the_reference(ref, mode, n_dims):
    x = rows(5, 1, 6, 4, 128)
    pos = np.array([0, 1, 17, 511, 4095, 8191], np.int32)
    a, b = np.zeros_like(x), np.zeros_like(x)
    kw = dict(freq_base=500000.0, freq_scale=1.0 if mode == 0 else 0.5, attn_factor=1.0 if mode == 0 else 1.25)
    assert ref.rope(to_ob(rope_request(x, pos, a, n_dims, mode, **kw)))
    assert row_ops.rope(to_ob(rope_request(x, pos, b, n_dims, mode, **kw)))
    assert ulps(a, b) <= ROPE_ULPS, ulps(a, b)
    assert np.array_equal(a[..., n_dims:], x[..., n_dims:])
