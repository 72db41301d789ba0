"""The layer-window oracle against the expectations of the reference's own tests
(tests/model/tensor/window/lifecycle_tests.cpp, streaming_tests.cpp; fixture numbers from
window_test_fixture.hpp:21-24 and 219-223), and the package's host-side plan against the oracle."""
import random

import emel_cpp_b200  # noqa: F401  (makes the package importable)
from emel_cpp_b200 import window as ew
from oracle import window_oracle as wo

LAYERS, WEIGHTS, WEIGHT_BYTES, HEADER = 6, 2, 8192, 4096


def fixture_layers():
    """stream_file: 6 layers of 2 weights of 8192 bytes behind a 4096-byte header."""
    layers, off = [], HEADER
    for l in range(LAYERS):
        ws = []
        for w in range(WEIGHTS):
            ws.append((l * WEIGHTS + w, off, WEIGHT_BYTES))
            off += WEIGHT_BYTES
        layers.append(ws)
    return layers, off


STREAMING_BUDGET = 5 * 2 * WEIGHT_BYTES
ARENA = 8 * 2 * 8192


def test_reference_bind_expectations():
    layers, size = fixture_layers()
    # "streaming bind activates slots and reports source": 4 slots, depth 2
    assert wo.bind_decision(size, layers, STREAMING_BUDGET, 4, 2, ARENA) == (wo.NONE, True)
    # "passthrough activates without slots for fitting budgets" / "accepts zero slot fields"
    assert wo.bind_decision(size, layers, 0, 4, 2, ARENA) == (wo.NONE, False)
    assert wo.bind_decision(size, layers, 0, 0, 0, ARENA) == (wo.NONE, False)
    # "rejects invalid bind requests": a 64 KiB stage chunk
    assert wo.bind_decision(size, layers, 0, 4, 2, ARENA, chunk=64 * 1024)[0] == wo.INVALID_REQUEST
    # "rejects extents outside the mapped source"
    bad = [list(ws) for ws in layers]
    bad[-1][-1] = (bad[-1][-1][0], size - 16, 64)
    assert wo.bind_decision(size, bad, 0, 4, 2, ARENA)[0] == wo.INVALID_REQUEST
    # "rejects invalid streaming slot configuration": one slot cannot form a ring
    assert wo.bind_decision(size, layers, STREAMING_BUDGET, 1, 0, ARENA)[0] == wo.INVALID_REQUEST
    # "rejects undersized slot storage explicitly" / "rejects null slot storage explicitly"
    assert wo.bind_decision(size, layers, STREAMING_BUDGET, 4, 2, 64)[0] == wo.SLOT_STORAGE_TOO_SMALL
    assert wo.bind_decision(size, layers, STREAMING_BUDGET, 4, 2, 1 << 20, storage_null=True)[0] == wo.SLOT_STORAGE_TOO_SMALL
    # "rejects rebind while bound"
    assert wo.bind_decision(size, layers, STREAMING_BUDGET, 4, 2, ARENA, already_bound=True)[0] == wo.ALREADY_BOUND
    # "rejects sources past the mapping cap before slot sizing": two layers spanning a 2^62 source
    huge = 1 << 62
    assert wo.bind_decision(huge, [[(0, 0, huge)], [(1, 0, huge)]], 64 * 1024, 8, 2, ARENA)[0] == wo.SOURCE_MAP_FAILED
    # a budget that holds fewer than the slots asked for
    assert wo.bind_decision(size, layers, 3 * 2 * WEIGHT_BYTES, 4, 2, ARENA)[0] == wo.BUDGET_TOO_SMALL


def test_reference_ring_expectations():
    # "streams every layer" and "ring eviction preserves content across passes": every acquire succeeds and the slot
    # then holds the layer asked for
    ring = wo.Ring(LAYERS, 4, 2)
    assert ring.loads == [(0, 0), (1, 1)]            # primed with prefetch_depth layers
    for _pass in range(2):
        for l in range(LAYERS):
            assert ring.acquire(l) == wo.NONE
            assert ring.layer[l % 4] == l
    # "cold acquire far from the prefetch ring"
    ring = wo.Ring(LAYERS, 4, 2)
    assert ring.acquire(5) == wo.NONE and ring.layer[5 % 4] == 5 and ring.cold == 1
    assert ring.acquire(0) == wo.NONE and ring.layer[0] == 0
    # out of range
    assert ring.acquire(LAYERS) == wo.LAYER_OUT_OF_RANGE and ring.acquire(-1) == wo.LAYER_OUT_OF_RANGE
    # "resubmits a failed slot load and reports slot_copy_failed": every load fails -> one resubmit, then the error
    ring = wo.Ring(LAYERS, 4, 2, fail=range(100))
    before = len(ring.loads)
    assert ring.acquire(0) == wo.SLOT_COPY_FAILED and len(ring.loads) == before + 1
    # a failed prefetch followed by a load that works is not an error
    ring = wo.Ring(LAYERS, 4, 2, fail=[0])
    assert ring.acquire(0) == wo.NONE


def test_steady_state_is_all_prefetched():
    # sequential passes: after the first acquires every layer is in (or on the way to) its slot when asked for,
    # unless the pass wrap aliases the slot of the layer in use (layers % slots != 0)
    for n, slots, depth in [(32, 4, 2), (32, 8, 7), (80, 4, 3), (6, 3, 1)]:
        ring = wo.Ring(n, slots, depth)
        for _pass in range(3):
            for l in range(n):
                assert ring.acquire(l) == wo.NONE
        if n % slots == 0:
            assert ring.cold == 0
            assert len(ring.loads) == 3 * n + depth


def test_package_plan_matches_oracle():
    rng = random.Random(7)
    for _ in range(50):
        layers, off = [], rng.randrange(0, 5000)
        for _l in range(rng.randrange(1, 9)):
            ws = []
            for _w in range(rng.randrange(1, 13)):
                size = rng.randrange(1, 70000)
                ws.append((len(ws), off, size))
                off += size + rng.randrange(0, 100)
            layers.append(ws)
        plan, cap = wo.scan_layers(layers)
        offs, sizes, cap2 = ew.plan_layers(layers)
        assert cap == cap2 and sizes == [d["slot_bytes"] for d in plan] and offs == [d["slot_offsets"] for d in plan]
        assert all(o % 64 == 0 for os_ in offs for o in os_)
    assert [ew.slot_of(l, 4) for l in range(6)] == [0, 1, 2, 3, 0, 1]
    # the error bits are the reference's (src/emel/model/tensor/window/errors.hpp:9-21)
    assert (ew.INVALID_REQUEST, ew.NOT_BOUND, ew.ALREADY_BOUND, ew.SOURCE_MAP_FAILED, ew.BUDGET_TOO_SMALL, ew.LAYER_OUT_OF_RANGE,
            ew.SLOT_COPY_FAILED, ew.NOT_STREAMING, ew.INTERNAL_ERROR, ew.SLOT_STORAGE_TOO_SMALL) == tuple(1 << i for i in range(10))


def test_library_request_check_matches_oracle():
    """emelb_window_check (no GPU): the reference test cases and random requests, every decision and the plan
    sizes against the oracle."""
    layers, size = fixture_layers()
    aligned_addr = 1 << 20          # any non-null, 64-byte aligned address: the check never touches it
    cases = [
        dict(budget=STREAMING_BUDGET, slots=4, depth=2, storage=ARENA),
        dict(budget=0, slots=4, depth=2, storage=ARENA),
        dict(budget=0, slots=0, depth=0, storage=0),
        dict(budget=0, slots=4, depth=2, storage=ARENA, chunk=64 * 1024),
        dict(budget=STREAMING_BUDGET, slots=1, depth=0, storage=ARENA),
        dict(budget=STREAMING_BUDGET, slots=4, depth=4, storage=ARENA),
        dict(budget=STREAMING_BUDGET, slots=9, depth=2, storage=ARENA),
        dict(budget=STREAMING_BUDGET, slots=4, depth=2, storage=64),
        dict(budget=STREAMING_BUDGET, slots=4, depth=2, storage=0),
        dict(budget=3 * 2 * WEIGHT_BYTES, slots=4, depth=2, storage=ARENA),
        dict(budget=LAYERS * WEIGHTS * WEIGHT_BYTES, slots=4, depth=2, storage=ARENA),
    ]
    for c in cases:
        chunk = c.get("chunk", wo.DEFAULT_CHUNK)
        err, streaming, cap, total = ew.check_request(size, layers, c["budget"], c["slots"], c["depth"], chunk,
                                                      aligned_addr if c["storage"] else 0, c["storage"])
        want = wo.bind_decision(size, layers, c["budget"], c["slots"], c["depth"], c["storage"],
                                storage_null=c["storage"] == 0, chunk=chunk)
        assert (err, streaming) == want, (c, err, streaming, want)
    # an extent past the end; a misaligned arena; a source past the mapping cap
    bad = [list(ws) for ws in layers]
    bad[-1][-1] = (bad[-1][-1][0], size - 16, 64)
    assert ew.check_request(size, bad, 0, 4, 2)[0] == ew.INVALID_REQUEST
    assert ew.check_request(size, layers, STREAMING_BUDGET, 4, 2, slot_storage=aligned_addr + 8,
                            slot_storage_bytes=ARENA)[0] == ew.SLOT_STORAGE_TOO_SMALL
    huge = 1 << 62
    assert ew.check_request(huge, [[(0, 0, huge)], [(1, 0, huge)]], 64 * 1024, 8, 2, slot_storage=aligned_addr,
                            slot_storage_bytes=ARENA)[0] == ew.SOURCE_MAP_FAILED
    assert ew.check_request(size, [], 0)[0] == ew.INVALID_REQUEST
    assert ew.check_request(size, [[]], 0)[0] == ew.INVALID_REQUEST
    assert ew.check_request(size, [[(i, HEADER, 16) for i in range(13)]], 0)[0] == ew.INVALID_REQUEST   # 13 weights in a layer
    assert ew.check_request(0, layers, 0)[0] == ew.INVALID_REQUEST
    assert ew.check_request(size, layers, 0, file_path=b"")[0] == ew.INVALID_REQUEST
    # random requests
    rng = random.Random(11)
    for _ in range(300):
        lay, off = [], rng.randrange(0, 4096)
        for _l in range(rng.randrange(1, 10)):
            ws = []
            for _w in range(rng.randrange(1, 10)):
                n = rng.randrange(1, 50000)
                ws.append((len(ws), off, n))
                off += n + rng.randrange(0, 64)
            lay.append(ws)
        fsize = off + rng.randrange(0, 100)
        plan, cap = wo.scan_layers(lay)
        total = sum(d["slot_bytes"] for d in plan)
        budget = rng.choice([0, total, total - 1, cap, 2 * cap, 3 * cap, 8 * cap, rng.randrange(1, 2 * total + 2)])
        slots, depth = rng.randrange(0, 11), rng.randrange(0, 11)
        storage = rng.choice([0, 64, cap, slots * cap, 8 * cap])
        err, streaming, cap_got, total_got = ew.check_request(fsize, lay, budget, slots, depth, wo.DEFAULT_CHUNK,
                                                              aligned_addr if storage else 0, storage)
        want = wo.bind_decision(fsize, lay, budget, slots, depth, storage, storage_null=storage == 0)
        assert (err, streaming) == want, (budget, slots, depth, storage, cap, total, err, streaming, want)
        assert (cap_got, total_got) == (cap, total)
