"""The allocation-free mat-vec entry point (emelb_mul_mat_vec_noalloc).

It exists for callers that may not call cudaMalloc (latency-bound serving loops, hooks where
allocation is forbidden, processes whose device memory belongs to another pool): its scratch is
a fixed array inside the library.  Checked here: same bits as the context-based emelb_mul_mat on
two calls in a row (the second with different activations and a different K, so stale scratch
would show), no change in free device memory across the calls, and a clear refusal beyond the
fixed maximum K.  This file sorts last so that a run stopping at the first failure has already
run every other test.
"""
import numpy as np
import pytest

import emel_cpp_b200 as eb
from tests import synth

pytestmark = pytest.mark.gpu


def test_noalloc_matches_context_entry_point_twice():
    import torch
    be = eb.Backend(0)
    try:
        # the fixed maximum K = 32768 back to back with small K (stale scratch beyond the used part would show),
        # every weight type, K-quant shapes that take the streaming kernel (K % 2048 == 0) and the generic one
        cases = [(eb.Q4_K, 4096, 300, 1), (eb.Q4_K, 2048, 77, 2), (eb.Q8_0, 4096, 64, 3), (eb.Q6_K, 1280, 9, 4),
                 (eb.Q6_K, 32768, 8, 5), (eb.Q4_K, 2048, 12, 6), (eb.Q8_0, 32768, 8, 7), (eb.Q4_0, 4096, 33, 8),
                 (eb.Q6_K, 4096, 40, 9), (eb.Q4_K, 32768, 16, 10), (eb.Q8_0, 64, 5, 11)]
        bufs = []
        for t, k, m, seed in cases:
            wd, xd, y0, y1 = be.alloc(m * eb.row_bytes(t, k)), be.alloc(4 * k), be.alloc(4 * m), be.alloc(4 * m)
            assert be.synth_fill(wd, t, m * k, 10 + seed, 0.02, 0) and be.synth_fill(xd, eb.F32, k, 20 + seed, 1.0, 0)
            bufs.append((t, k, m, wd, xd, y0, y1))
        assert be.sync()
        # first call on this device happens here, outside any capture; it may do its one-time set-up
        t, k, m, wd, xd, y0, y1 = bufs[0]
        err, msg = eb.mul_mat_vec_noalloc(0, be.stream(), t, wd, k, m, xd, y1)
        assert err == eb.OK, msg
        assert be.sync()
        free_before = torch.cuda.mem_get_info(0)[0]
        for t, k, m, wd, xd, y0, y1 in bufs:                     # calls in a row share one scratch array
            assert be.mul_mat(eb.mul_mat_op(wd, t, k, m, xd, 1, y0)), be.last_error
            err, msg = eb.mul_mat_vec_noalloc(0, be.stream(), t, wd, k, m, xd, y1)
            assert err == eb.OK, msg
        assert be.sync()
        assert torch.cuda.mem_get_info(0)[0] == free_before      # nothing was allocated or freed
        for t, k, m, wd, xd, y0, y1 in bufs:
            a, b = np.zeros(m, np.float32), np.zeros(m, np.float32)
            assert be.to_host(a, y0) and be.to_host(b, y1)
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), (t, k, m)
            assert np.isfinite(a).all() and a.std() > 0
        # and once against the reference's own CPU kernel (x86 route), directly
        from oracle import bindings as ob
        checker = ob.ref()
        t, k, m, wd, xd, y0, y1 = bufs[0]
        w, x, got = np.zeros(m * eb.row_bytes(t, k), np.uint8), np.zeros((k, 1), np.float32), np.zeros(m, np.float32)
        assert be.to_host(w, wd) and be.to_host(x, xd) and be.to_host(got, y1)
        want = np.zeros((m, 1), np.float32)
        if checker is not None:
            assert checker.mul_mat(ob.mul_mat_op(w, t, k, m, x, 1, want), route="avx2")
            assert np.array_equal(got.view(np.uint32), want[:, 0].view(np.uint32))
        else:
            assert ob.port().mul_mat(ob.mul_mat_op(w, t, k, m, x, 1, want))
            assert ob.rel_l2(got, want[:, 0]) <= 1e-5
    finally:
        be.close()


def test_noalloc_leaves_the_callers_current_device_alone():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs a second device to tell the difference")
    be = eb.Backend(1)
    try:
        t, k, m = eb.Q4_K, 2048, 8
        wd, xd, yd = be.alloc(m * eb.row_bytes(t, k)), be.alloc(4 * k), be.alloc(4 * m)
        assert be.synth_fill(wd, t, m * k, 3, 0.02, 0) and be.synth_fill(xd, eb.F32, k, 4, 1.0, 0) and be.sync()
        torch.cuda.set_device(0)
        err, msg = eb.mul_mat_vec_noalloc(1, be.stream(), t, wd, k, m, xd, yd)
        assert err == eb.OK, msg
        assert torch.cuda.current_device() == 0
        from cuda.bindings import runtime as rt   # the runtime's own view of the calling thread's device
        assert rt.cudaGetDevice()[1] == 0
        assert be.sync()
    finally:
        be.close()


def test_noalloc_refuses_beyond_its_fixed_maximum():
    err, msg = eb.mul_mat_vec_noalloc(0, 0, eb.Q8_0, 1 << 20, 32768 + 32, 4, 1 << 20, 1 << 20)
    assert err == eb.INVALID_REQUEST and "32768" in msg
    err, msg = eb.mul_mat_vec_noalloc(0, 0, eb.F32, 1 << 20, 4096, 4, 1 << 20, 1 << 20)
    assert err == eb.INVALID_REQUEST and msg
    err, msg = eb.mul_mat_vec_noalloc(0, 0, eb.Q4_K, 0, 4096, 4, 1 << 20, 1 << 20)
    assert err == eb.INVALID_REQUEST and msg
