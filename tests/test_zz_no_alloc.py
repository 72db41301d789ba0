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
        cases = [(eb.Q4_K, 4096, 300, 1), (eb.Q4_K, 2048, 77, 2), (eb.Q8_0, 4096, 64, 3), (eb.Q6_K, 1280, 9, 4)]
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
    finally:
        be.close()


def test_noalloc_refuses_beyond_its_fixed_maximum():
    err, msg = eb.mul_mat_vec_noalloc(0, 0, eb.Q8_0, 1 << 20, 32768 + 32, 4, 1 << 20, 1 << 20)
    assert err == eb.INVALID_REQUEST and "32768" in msg
    err, msg = eb.mul_mat_vec_noalloc(0, 0, eb.F32, 1 << 20, 4096, 4, 1 << 20, 1 << 20)
    assert err == eb.INVALID_REQUEST and msg
    err, msg = eb.mul_mat_vec_noalloc(0, 0, eb.Q4_K, 0, 4096, 4, 1 << 20, 1 << 20)
    assert err == eb.INVALID_REQUEST and msg
