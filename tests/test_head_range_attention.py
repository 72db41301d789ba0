"""kernel::attention's head-range event: the C-ABI guard against the reference's, and the numpy restatement against
the reference's compiled code.  CPU only."""
import ctypes as C

import numpy as np
import pytest

import emel_cpp_b200 as eb
from oracle import bindings as ob
from oracle import row_ops


def make_case(seed, hidden=256, head_dim=64, capacity=40, layers=2):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal(hidden).astype(np.float32)
    k = row_ops.f32_to_bf16_bits(rng.standard_normal(layers * capacity * hidden).astype(np.float32) * 0.5)
    v = row_ops.f32_to_bf16_bits(rng.standard_normal(layers * capacity * hidden).astype(np.float32))
    return q, k, v


def request(q, k, v, out, layer_offset, hidden, head_dim, h0, h1, cap, begin, valid, counts=None):
    return eb.head_range_request(q, k, v, out, layer_offset, hidden, head_dim, h0, h1, cap, begin, valid, counts)


def guard_cases():
    q, k, v = make_case(1)
    out = np.zeros(256, np.float32)
    base = dict(layer_offset=40 * 256, hidden=256, head_dim=64, h0=1, h1=4, cap=40, begin=35, valid=17)
    cases = [("ok", dict(base)), ("wraps", dict(base, begin=39, valid=40)), ("one head", dict(base, h0=3, h1=4)),
             ("empty head range", dict(base, h0=2, h1=2)), ("head past hidden", dict(base, h1=5)),
             ("begin at capacity", dict(base, begin=40)), ("too many positions", dict(base, valid=41)),
             ("no positions", dict(base, valid=0)), ("negative begin", dict(base, begin=-1)),
             ("zero head_dim", dict(base, head_dim=0)), ("cache too short", dict(base, layer_offset=2 * 40 * 256)),
             ("capacity over the limit", dict(base, cap=8193, layer_offset=0))]
    reqs = [(name, request(q, k, v, out, **kw)) for name, kw in cases]
    short_q = request(q, k, v, out, **base)
    short_q.query_count = 255
    reqs.append(("query too short", short_q))
    small_out = request(q, k, v, out, **base)
    small_out.output_count = 3 * 64 - 1
    reqs.append(("output too short", small_out))
    null_k = request(q, k, v, out, **base)
    null_k.key_cache = None
    reqs.append(("null key cache", null_k))
    overlap = request(q, k, v, q, **base)          # output over the query
    overlap.output_count = 256
    reqs.append(("output overlaps the query", overlap))
    odd = request(q, k, v, out, **base)
    odd.key_cache = k.ctypes.data + 1
    reqs.append(("misaligned key cache", odd))
    return reqs, (q, k, v, out)


def test_guard_matches_the_reference():
    reqs, _keep = guard_cases()
    ref = ob.ref()
    verdicts = {}
    for name, r in reqs:
        got = eb.lib().emelb_attention_head_range_can_run(C.byref(r)) == eb.OK
        if ref is not None:
            assert got == ref.head_range_can_run(r), name
        verdicts[name] = got
    assert verdicts["ok"] and verdicts["wraps"] and verdicts["one head"]
    assert sum(verdicts.values()) == 3, verdicts


@pytest.mark.parametrize("begin,valid", [(0, 1), (0, 40), (35, 17), (39, 40), (7, 8)])
def test_restatement_tracks_the_reference(ref, begin, valid):
    q, k, v = make_case(5)
    a, b = np.zeros(3 * 64, np.float32), np.zeros(3 * 64, np.float32)
    assert ref.head_range(request(q, k, v, a, 40 * 256, 256, 64, 1, 4, 40, begin, valid))
    assert row_ops.head_range_attention(q, k, v, b, 40 * 256, 256, 64, 1, 4, 40, begin, valid)
    assert np.abs(a - b).max() <= 2e-6 * max(1.0, np.abs(a).max())
