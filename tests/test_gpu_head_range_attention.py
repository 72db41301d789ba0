"""kernel::attention's head-range event through the C-ABI against the CPU checker.

Bar: bit for bit against the reference's own code (oracle/_ref, its scalar route: the oracle build has no global
-mavx2) -- every sum whose order the reference fixes is sequential in the kernel, and expf has glibc's bits.  Where
that build is absent, the numpy restatement is the checker, within 2e-6 relative (its exp is not glibc's expf).
"""
import numpy as np
import pytest

import emel_cpp_b200 as eb
from oracle import bindings as ob
from oracle import row_ops
from tests.test_head_range_attention import make_case, request

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    b = eb.Backend(0)
    yield b
    b.close()


def check(be, q, k, v, layer_offset, hidden, head_dim, h0, h1, cap, begin, valid):
    got = np.zeros((h1 - h0) * head_dim, np.float32)
    want = np.zeros_like(got)
    assert be.attention_head_range(request(q, k, v, got, layer_offset, hidden, head_dim, h0, h1, cap, begin, valid)), be.last_error
    ref = ob.ref()
    if ref is not None:
        assert ref.head_range(request(q, k, v, want, layer_offset, hidden, head_dim, h0, h1, cap, begin, valid))
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), float(np.abs(got - want).max())
    else:
        assert row_ops.head_range_attention(q, k, v, want, layer_offset, hidden, head_dim, h0, h1, cap, begin, valid)
        assert np.abs(got - want).max() <= 2e-6 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("begin,valid", [(0, 1), (0, 40), (35, 17), (39, 40), (7, 8)])
def test_ring_buffer_positions(be, begin, valid):
    q, k, v = make_case(5)
    check(be, q, k, v, 40 * 256, 256, 64, 1, 4, 40, begin, valid)


@pytest.mark.parametrize("hidden,head_dim,cap,h0,h1", [(512, 128, 750, 0, 4), (1024, 64, 1500, 3, 16), (96, 32, 9, 0, 3), (2048, 128, 300, 8, 16)])
def test_shapes(be, hidden, head_dim, cap, h0, h1):
    q, k, v = make_case(9, hidden=hidden, head_dim=head_dim, capacity=cap, layers=1)
    check(be, q, k, v, 0, hidden, head_dim, h0, h1, cap, cap // 3, cap - 2)


def test_device_resident_operands(be):
    import torch
    q, k, v = make_case(11, hidden=512, head_dim=64, capacity=200, layers=1)
    want = np.zeros(8 * 64, np.float32)
    qd, kd, vd = torch.from_numpy(q).cuda(), torch.from_numpy(k.view(np.int16)).cuda(), torch.from_numpy(v.view(np.int16)).cuda()
    od = torch.zeros(8 * 64, dtype=torch.float32, device="cuda")
    r = eb.head_range_request(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), od.data_ptr(), 0, 512, 64, 0, 8, 200, 150, 120,
                              counts=[512, 200 * 512, 200 * 512, 8 * 64])
    assert be.attention_head_range(r), be.last_error
    assert be.sync()
    ref = ob.ref()
    if ref is not None:
        assert ref.head_range(request(q, k, v, want, 0, 512, 64, 0, 8, 200, 150, 120))
        assert np.array_equal(od.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_rejects_what_the_reference_rejects(be):
    q, k, v = make_case(1)
    out = np.zeros(256, np.float32)
    assert not be.attention_head_range(request(q, k, v, out, 40 * 256, 256, 64, 1, 5, 40, 0, 10))    # head past hidden
    assert be.last_error == eb.INVALID_REQUEST
    assert not be.attention_head_range(request(q, k, v, out, 40 * 256, 256, 64, 1, 4, 40, 0, 41))    # too many positions
    assert not np.any(out)
