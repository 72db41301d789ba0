"""op_rms_norm and op_rope through the C-ABI against the CPU checker: the reference's own code where
oracle/_ref is present, else the numpy restatement.

Bars: op_rms_norm bit for bit (same f64 sum order, same f32 steps).  op_rope within ROPE_ULPS units in the
last place of the row's largest magnitude: the angles are the reference's floats bit for bit, but the device's
cosf / sinf and the compiler's choice to fuse x0 * c - x1 * s differ from the host's by an ulp or two.
"""
import ctypes as C

import numpy as np
import pytest

import emel_cpp_b200 as eb
from oracle import bindings as ob
from oracle import row_ops
from tests.test_row_ops import rms_request, rope_request, rows, to_ob, ulps

pytestmark = pytest.mark.gpu

ROPE_ULPS = 8


@pytest.fixture(scope="module")
def be():
    b = eb.Backend(0)
    yield b
    b.close()


def cpu(name, op):
    r = ob.ref()
    return getattr(r, name)(to_ob(op)) if r is not None else getattr(row_ops, name)(to_ob(op))


@pytest.mark.parametrize("shape", [(1, 256), (1, 4096), (512, 4096), (3, 8192), (2, 3, 5, 100), (1, 32768)])
def test_rms_norm_bit_exact(be, shape):
    x = rows(3, *shape)
    got, want = np.zeros_like(x), np.zeros_like(x)
    assert be.rms_norm(rms_request(x, got, 1e-5)), be.last_error
    assert cpu("rms_norm", rms_request(x, want, 1e-5))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), float(np.abs(got - want).max())


def test_rms_norm_strided_views(be):
    """Rows taken out of wider buffers on both sides: only the viewed elements are read and written."""
    src = rows(9, 6, 160)
    dst = np.full((6, 192), 7.0, np.float32)
    want = dst.copy()

    def request(out):
        op = rms_request(src[:, :128].copy(), np.zeros((6, 128), np.float32), 1e-6)
        op.src0.data, op.src0.nb[1], op.src0.nb[2], op.src0.nb[3] = src.ctypes.data, 640, 3840, 3840
        op.dst.data, op.dst.nb[1], op.dst.nb[2], op.dst.nb[3] = out.ctypes.data, 768, 4608, 4608
        return op

    assert be.rms_norm(request(dst)), be.last_error
    assert cpu("rms_norm", request(want))
    assert np.array_equal(dst.view(np.uint32), want.view(np.uint32))
    assert np.all(dst[:, 128:] == 7.0)


def test_rms_norm_device_resident(be):
    import torch
    x = rows(4, 16, 4096)
    want = np.zeros_like(x)
    xd = torch.from_numpy(x).cuda()
    yd = torch.zeros_like(xd)
    op = rms_request(x, want, 1e-5)
    op.src0.data, op.dst.data = xd.data_ptr(), yd.data_ptr()
    assert be.rms_norm(op), be.last_error
    be.sync()
    assert cpu("rms_norm", rms_request(x, want, 1e-5))
    assert np.array_equal(yd.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("mode,n_dims,heads,tokens", [(0, 128, 32, 1), (0, 128, 8, 64), (2, 128, 8, 5), (2, 64, 4, 3), (0, 96, 2, 7)])
def test_rope_matches_the_reference(be, mode, n_dims, heads, tokens):
    x = rows(5, 1, tokens, heads, 128)
    pos = (np.arange(tokens, dtype=np.int32) * 131 + (8191 - 131 * (tokens - 1))).astype(np.int32)
    got, want = np.zeros_like(x), np.zeros_like(x)
    kw = dict(freq_base=500000.0, freq_scale=1.0 if mode == 0 else 0.5, attn_factor=1.0 if mode == 0 else 1.25)
    assert be.rope(rope_request(x, pos, got, n_dims, mode, **kw)), be.last_error
    assert cpu("rope", rope_request(x, pos, want, n_dims, mode, **kw))
    assert ulps(got, want) <= ROPE_ULPS, ulps(got, want)
    assert np.array_equal(got[..., n_dims:], x[..., n_dims:])


def test_rope_rejects_what_the_reference_rejects(be):
    x = rows(5, 1, 2, 2, 64)
    pos = np.arange(2, dtype=np.int32)
    y = np.zeros_like(x)
    assert not be.rope(rope_request(x, pos, y, 63))
    assert be.last_error == eb.INVALID_REQUEST
    assert not be.rope(rope_request(x, pos, y, 64, ext_factor=1.0))
    # the timestep-embedding variant passes the guard but is not on this path
    assert not be.rope(rope_request(x, pos, y, 64, 4))
    assert be.last_error == eb.UNSUPPORTED_OP
    assert not np.any(y)


def test_glu_is_rejected_like_the_reference(be):
    g = np.ones((2, 64), np.float32)
    op = eb.Op()
    op.src0, op.src1, op.dst = eb.dense_view(g, eb.F32, [64, 2]), eb.dense_view(g, eb.F32, [64, 2]), eb.dense_view(g, eb.F32, [64, 2])
    assert not be.glu(op)
    assert be.last_error == eb.INVALID_REQUEST
