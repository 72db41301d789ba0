"""A device-side wait that runs out, made on purpose and without a fault: a two-rank peer-store join whose
second rank never answers (both ranks' buffers are the context's own staging memory).  The kernel gives up
after the limit, raises the status word and returns; emelb_sync reports the failure once and the context
keeps working."""
import time

import numpy as np
import pytest

import emel_cpp_b200 as eb
from oracle import bindings as ob
from tests import synth

pytestmark = pytest.mark.gpu


def test_wait_runs_out_sync_reports_it_and_the_context_survives(port, checker):
    be = eb.Backend(0)
    try:
        k, m = 2048, 64
        w = synth.encoded_weights(port, eb.Q4_K, 5, m, k)
        x = synth.activations_f32(6, k)
        y = np.zeros((m, 1), np.float32)
        assert be.mul_mat(eb.mul_mat_op(w, eb.Q4_K, k, m, x, 1, y)) and be.sync()
        want = y.copy()

        t0 = time.perf_counter()
        assert be.selftest_wait_timeout(40), be.last_error
        assert not be.sync() and be.last_error == eb.INTERNAL_ERROR        # the wait ran out: reported here
        dt = time.perf_counter() - t0
        assert 0.03 <= dt < 5.0, dt                                        # it waited about the limit, not forever
        assert be.sync()                                                   # reported once, then cleared

        y[:] = 0
        assert be.mul_mat(eb.mul_mat_op(w, eb.Q4_K, k, m, x, 1, y)) and be.sync()
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32))     # the context still computes
        assert not be.selftest_wait_timeout(0) and be.last_error == eb.INVALID_REQUEST
        assert be.set_peer_wait_ms(2000) and not be.set_peer_wait_ms(0)
    finally:
        be.close()
