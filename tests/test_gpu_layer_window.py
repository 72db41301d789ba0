"""The layer streaming window on the device (include/emelb_window.h).

The window cases follow the reference's own tests of model::tensor::window
(tests/model/tensor/window/lifecycle_tests.cpp, streaming_tests.cpp): the same synthetic
"model file" (six layers of two 8192-byte weights filled with a per-weight sentinel byte behind
a 4096-byte header), the same budgets and slot counts, the same expected errors -- with the
slots in HBM, read back through the context's stream.  Bind decisions and load counts are also
compared with the oracle's model of the ring.  The session cases decode a model whose layers
are streamed through 2-4 slots and compare with the resident session, bit for bit."""
import os

import numpy as np
import pytest

import emel_cpp_b200 as eb
from emel_cpp_b200 import llama as el
from emel_cpp_b200 import window as ew
from oracle import window_oracle as wo
from tests import synth

pytestmark = pytest.mark.gpu

LAYERS, WEIGHTS, WEIGHT_BYTES, HEADER = 6, 2, 8192, 4096
STREAMING_BUDGET = 5 * 2 * WEIGHT_BYTES


def sentinel(layer, weight):
    return (0x11 + layer * 0x10 + weight) & 0xFF


def stream_image():
    layers, off = [], HEADER
    image = np.zeros(HEADER + LAYERS * WEIGHTS * WEIGHT_BYTES, dtype=np.uint8)
    for l in range(LAYERS):
        ws = []
        for w in range(WEIGHTS):
            image[off:off + WEIGHT_BYTES] = sentinel(l, w)
            ws.append((l * WEIGHTS + w, off, WEIGHT_BYTES))
            off += WEIGHT_BYTES
        layers.append(ws)
    return image, layers


@pytest.fixture(scope="module")
def be():
    b = eb.Backend(0)
    yield b
    b.close()


def slot_content_matches(be, got, layer):
    base, layout = got
    for w, (_tid, _off, size, slot_off) in enumerate(layout):
        host = np.empty(size, dtype=np.uint8)
        assert be.to_host(host, base + slot_off, size)
        if not (host == sentinel(layer, w)).all():
            return False
    return True


@pytest.mark.parametrize("route", ["page-locked", "staged", "file"])
def test_streams_every_layer_with_correct_content(be, route, tmp_path):
    image, layers = stream_image()
    win = ew.LayerWindow(be)
    try:
        source = image
        if route == "staged":
            assert win.set_staged_only(True)
        if route == "file":
            source = os.path.join(tmp_path, "window.bin")
            image.tofile(source)
        assert win.bind(source, layers, STREAMING_BUDGET, 4, 2), win.last_error
        assert win.bound["streaming_active"] and win.bound["window_slots"] == 4 and win.bound["source_base"]
        if route != "file":   # whether a file mapping can be page-locked in place is the platform's business
            assert win.bound["source_page_locked"] == (route != "staged")
        plan, cap = wo.scan_layers(layers)
        for l in range(LAYERS):
            got = win.layer_plan(l)
            assert got["slot_offsets"] == plan[l]["slot_offsets"] and got["slot_bytes"] == plan[l]["slot_bytes"]
            assert got["file_begin"] == plan[l]["file_begin"] and got["file_span"] == plan[l]["file_span"] and got["slot_capacity"] == cap
        # two full passes: every slot is evicted and refilled at least once
        ring = wo.Ring(LAYERS, 4, 2)
        for _pass in range(2):
            for l in range(LAYERS):
                got = win.acquire(l)
                assert got is not None, win.last_error
                assert slot_content_matches(be, got, l), (route, l)
                assert ring.acquire(l) == wo.NONE
        st = win.stats()
        assert st["acquires"] == 2 * LAYERS and st["loads_failed"] == 0
        if win.bound["source_page_locked"]:   # the I/O thread's progress decides which prefetches the staged route skips
            assert st["loads_submitted"] == len(ring.loads)
            assert (st["acquires_resident"], st["acquires_cold"]) == (ring.resident_hits, ring.cold)
        assert st["bytes_copied"] >= LAYERS * WEIGHTS * WEIGHT_BYTES
        # out of range
        assert win.acquire(LAYERS) is None and win.last_error == ew.LAYER_OUT_OF_RANGE
        assert win.acquire(-1) is None and win.last_error == ew.LAYER_OUT_OF_RANGE
        assert win.unbind()
    finally:
        win.close()


@pytest.mark.parametrize("staged", [False, True])
def test_cold_acquire_far_from_the_ring_and_back(be, staged):
    image, layers = stream_image()
    win = ew.LayerWindow(be)
    try:
        win.set_staged_only(staged)
        assert win.bind(image, layers, STREAMING_BUDGET, 4, 2)
        got = win.acquire(5)
        assert got is not None and slot_content_matches(be, got, 5)
        got = win.acquire(0)
        assert got is not None and slot_content_matches(be, got, 0)
        # the same layer twice in a row, then a slot that aliases it (4 slots: layers 0 and 4)
        got = win.acquire(0)
        assert got is not None and slot_content_matches(be, got, 0)
        got = win.acquire(4)
        assert got is not None and slot_content_matches(be, got, 4)
        assert win.unbind()
    finally:
        win.close()


def test_lifecycle_and_bind_decisions(be):
    image, layers = stream_image()
    size = image.nbytes
    win = ew.LayerWindow(be)
    try:
        # unbound: acquire and unbind are rejected
        assert win.acquire(0) is None and win.last_error == ew.NOT_BOUND
        assert not win.unbind() and win.last_error == ew.NOT_BOUND

        def bind(budget, slots=4, depth=2, layers_=layers, chunk=ew.DEFAULT_CHUNK_BYTES, storage="auto"):
            ok = win.bind(image, layers_, budget, slots, depth, stage_chunk_bytes=chunk, slot_storage=storage)
            return (win.last_error, bool(ok and win.bound["streaming_active"]))

        import torch
        arena = torch.empty(8 * 2 * 8192, dtype=torch.uint8, device="cuda:0")
        # a stage chunk below the minimum; an extent past the end of the source
        assert bind(0, chunk=64 * 1024) == wo.bind_decision(size, layers, 0, 4, 2, 0, chunk=64 * 1024) == (ew.INVALID_REQUEST, False)
        bad = [list(ws) for ws in layers]
        bad[-1][-1] = (bad[-1][-1][0], size - 16, 64)
        assert bind(0, layers_=bad) == (ew.INVALID_REQUEST, False)
        # one slot cannot form a ring; a prefetch depth that fills the ring
        assert bind(STREAMING_BUDGET, 1, 0, storage=arena) == wo.bind_decision(size, layers, STREAMING_BUDGET, 1, 0, arena.numel())
        assert bind(STREAMING_BUDGET, 4, 4, storage=arena)[0] == ew.INVALID_REQUEST
        assert bind(STREAMING_BUDGET, 9, 2, storage=arena)[0] == ew.INVALID_REQUEST
        # budget below the slots asked for
        assert bind(3 * 2 * WEIGHT_BYTES, 4, 2, storage=arena) == (ew.BUDGET_TOO_SMALL, False)
        # undersized, missing and host slot storage
        assert bind(STREAMING_BUDGET, storage=arena[:64]) == (ew.SLOT_STORAGE_TOO_SMALL, False)
        assert bind(STREAMING_BUDGET, storage=None) == (ew.SLOT_STORAGE_TOO_SMALL, False)
        assert bind(STREAMING_BUDGET, storage=torch.empty(8 * 2 * 8192, dtype=torch.uint8)) == (ew.SLOT_STORAGE_TOO_SMALL, False)
        # a file that is not there
        assert not win.bind("/nonexistent/emelb_window.bin", layers, STREAMING_BUDGET, 4, 2, source_bytes=size)
        assert win.last_error == ew.SOURCE_MAP_FAILED
        # every rejected bind left the window unbound: passthrough binds with zero slot fields
        assert bind(0, 0, 0, storage=None) == (ew.OK, False)
        assert win.bound["window_slots"] == 0 and win.bound["source_base"]
        assert win.acquire(0) is None and win.last_error == ew.NOT_STREAMING
        assert bind(STREAMING_BUDGET)[0] == ew.ALREADY_BOUND
        assert win.unbind()
        # a budget that holds the whole model is passthrough too
        assert bind(LAYERS * WEIGHTS * WEIGHT_BYTES) == (ew.OK, False)
        assert win.unbind()
        # streaming; a second bind is refused and the first stays usable
        assert bind(STREAMING_BUDGET, storage=arena) == (ew.OK, True)
        assert bind(STREAMING_BUDGET, storage=arena)[0] == ew.ALREADY_BOUND
        got = win.acquire(1)
        assert got is not None and slot_content_matches(be, got, 1)
        assert got[0] == arena.data_ptr() + 1 * win.layer_plan(1)["slot_capacity"]
        assert win.unbind()
    finally:
        win.close()


@pytest.mark.parametrize("staged", [False, True])
def test_failed_loads_are_resubmitted_once(be, staged):
    """The failure is made on the host: the next loads report a failed copy without touching the device."""
    image, layers = stream_image()
    win = ew.LayerWindow(be)
    try:
        win.set_staged_only(staged)
        assert win.fail_next_loads(100)
        assert win.bind(image, layers, STREAMING_BUDGET, 4, 2)    # the primed loads fail
        assert win.acquire(0) is None and win.last_error == ew.SLOT_COPY_FAILED
        # not terminal: with the failures used up the same acquire works
        assert win.fail_next_loads(0)
        got = win.acquire(0)
        assert got is not None and slot_content_matches(be, got, 0)
        # one failed prefetch, then a load that works, is no error
        got = win.acquire(1)
        assert got is not None and slot_content_matches(be, got, 1)
        assert win.fail_next_loads(1)
        got = win.acquire(2)            # layer 2 was prefetched already; the failing load is the prefetch of layer 4
        assert got is not None and slot_content_matches(be, got, 2)
        got = win.acquire(3)
        assert got is not None and slot_content_matches(be, got, 3)
        got = win.acquire(4)
        assert got is not None and slot_content_matches(be, got, 4)
        assert win.stats()["loads_failed"] >= 3
        assert win.unbind()
    finally:
        win.close()


def test_unbind_joins_loads_in_flight_and_rebinds(be):
    image, layers = stream_image()
    for staged in (False, True):
        win = ew.LayerWindow(be)
        try:
            win.set_staged_only(staged)
            assert win.bind(image, layers, STREAMING_BUDGET, 4, 2)
            assert win.unbind()                       # straight after the primed prefetches
            assert win.acquire(0) is None and win.last_error == ew.NOT_BOUND
            assert win.bind(image, layers, STREAMING_BUDGET, 4, 2)
            got = win.acquire(0)
            assert got is not None and slot_content_matches(be, got, 0)
        finally:
            win.close()                               # destroys a bound window: joins and unbinds first


# ---------------------------------------------------------------- a decoder whose layers are streamed

MODEL = dict(n_layer=5, n_embd=512, n_head=8, n_head_kv=2, head_dim=64, n_ff=2048, n_vocab=640, n_ctx=96)
LAYER_ROLES = (el.ATTN_NORM, el.ATTN_Q, el.ATTN_K, el.ATTN_V, el.ATTN_OUT, el.FFN_NORM, el.FFN_GATE, el.FFN_UP, el.FFN_DOWN)
NORMS = (el.ATTN_NORM, el.FFN_NORM, el.OUTPUT_NORM)


def model_image(port, cfg, types, seed):
    """A model "file" in one host buffer: [pad | global tensors | layer 0 | layer 1 ...], every tensor at an odd
    multiple of 32 bytes.  -> (image, {(layer, role): (offset, bytes, type)})"""
    c = el.config(**cfg)
    shapes = el.matrix_shapes(c)
    parts, table, at = [], {}, 4096 + 32

    def put(layer, role, data, t):
        nonlocal at
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        table[(layer, role)] = (at, raw.nbytes, t)
        parts.append((at, raw))
        at += (raw.nbytes + 63) // 64 * 64 + 32

    def matrix(layer, role, scale):
        t = types.get(role, types["default"]) if layer >= 0 else types["embd" if role == el.TOKEN_EMBD else "output"]
        k, m = shapes[role]
        w = synth.rng(seed + 31 * (layer + 2) + role).standard_normal((m, k), dtype=np.float32) * np.float32(scale)
        put(layer, role, port.encode_rows(t, w, k, m), t)

    def norm(layer, role):
        w = (1.0 + 0.1 * synth.rng(seed + 977 * (layer + 2) + role).standard_normal(cfg["n_embd"], dtype=np.float32)).astype(np.float32)
        put(layer, role, w, eb.F32)

    matrix(-1, el.TOKEN_EMBD, 1.0)
    norm(-1, el.OUTPUT_NORM)
    matrix(-1, el.OUTPUT, 0.05)
    for l in range(cfg["n_layer"]):
        for role in LAYER_ROLES:
            if role in NORMS:
                norm(l, role)
            else:
                matrix(l, role, 0.05)
    image = np.zeros(at, dtype=np.uint8)
    for off, raw in parts:
        image[off:off + raw.nbytes] = raw
    return image, table


_NEXT_ID = [9000]
_UPLOADED = []     # tensor ids to evict when a test ends: the residency table is keyed by host address, and numpy hands
                   # the addresses of a freed image to the next one


def bind_tensor(be, sess, image, table, layer, role, upload):
    off, size, t = table[(layer, role)]
    span = image[off:off + size]
    if upload:
        be.upload(_NEXT_ID[0], span, tensor_type=t)
        _UPLOADED.append(_NEXT_ID[0])
        _NEXT_ID[0] += 1
    ok = sess.bind_norm(layer, role, span) if role in NORMS else sess.bind_matrix(layer, role, span, t)
    assert ok, (layer, role, sess.last_error)


def evict_uploaded(be):
    while _UPLOADED:
        be.evict(_UPLOADED.pop())


def resident_session(be, image, table, cfg):
    sess = el.Session(be, el.config(**cfg))
    for (layer, role) in table:
        bind_tensor(be, sess, image, table, layer, role, upload=True)
    return sess


def streamed_session(be, image, table, cfg, slots, depth, staged):
    layers = [[(l * 9 + i, table[(l, role)][0], table[(l, role)][1]) for i, role in enumerate(LAYER_ROLES)] for l in range(cfg["n_layer"])]
    _offs, sizes, cap = ew.plan_layers(layers)
    assert slots * cap < sum(sizes)
    win = ew.LayerWindow(be)
    win.set_staged_only(staged)
    assert win.bind(image, layers, slots * cap, slots, depth), win.last_error
    assert win.bound["streaming_active"]
    sess = el.Session(be, el.config(**cfg))
    assert sess.set_window(win), sess.last_error
    for (layer, role) in table:
        bind_tensor(be, sess, image, table, layer, role, upload=layer < 0)
    return sess, win


@pytest.mark.parametrize("slots,depth,staged,types", [
    (2, 1, False, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}),
    (3, 2, False, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K, el.FFN_DOWN: eb.Q6_K}),
    (4, 2, False, {"embd": eb.Q8_0, "output": eb.Q8_0, "default": eb.Q8_0, el.ATTN_K: eb.Q4_K, el.FFN_DOWN: eb.Q4_0}),
    (3, 1, True, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}),
])
def test_streamed_decoder_matches_the_resident_one(be, port, slots, depth, staged, types):
    image, table = model_image(port, MODEL, types, seed=13)
    resident = resident_session(be, image, table, MODEL)
    image2 = image.copy()        # a second copy: nothing of it is resident except what the streamed session uploads
    sess, win = streamed_session(be, image2, table, MODEL, slots, depth, staged)
    prompt = synth.rng(3).integers(0, MODEL["n_vocab"], size=24).tolist()
    try:
        # the prompt as one batch, then one step with logits, then a device-fed run
        assert resident.prefill(prompt[:-1], 0) and sess.prefill(prompt[:-1], 0), sess.last_error
        a = resident.decode(prompt[-1], len(prompt) - 1, want_logits=True)
        b = sess.decode(prompt[-1], len(prompt) - 1, want_logits=True)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), float(np.abs(a - b).max())
        want = list(resident.generate(prompt[-1], len(prompt) - 1, 20))
        assert list(sess.generate(prompt[-1], len(prompt) - 1, 20)) == want
        # the prompt token by token
        assert resident.set_prefill_batch(0) and sess.set_prefill_batch(0)
        assert resident.prefill(prompt[:-1], 0) and sess.prefill(prompt[:-1], 0), sess.last_error
        assert sess.decode(prompt[-1], len(prompt) - 1) == resident.decode(prompt[-1], len(prompt) - 1)
        # three sequences stepped together
        assert resident.set_sequences(3) and sess.set_sequences(3)
        first, pos = [], []
        for j in range(3):
            p = synth.rng(40 + j).integers(0, MODEL["n_vocab"], size=5 + 2 * j).tolist()
            for s in (resident, sess):
                assert s.select_sequence(j) and s.prefill(p[:-1], 0), s.last_error
            first.append(p[-1])
            pos.append(len(p) - 1)
        assert np.array_equal(sess.generate_batch(first, pos, 6), resident.generate_batch(first, pos, 6))
        ids_a, log_a = resident.decode_batch(first, pos, want_logits=True)
        ids_b, log_b = sess.decode_batch(first, pos, want_logits=True)
        assert list(ids_a) == list(ids_b) and np.array_equal(log_a.view(np.uint32), log_b.view(np.uint32))
        st = win.stats()
        assert st["acquires"] > 0 and st["loads_failed"] == 0 and st["loads_submitted"] >= MODEL["n_layer"]
        assert sess.launches_per_token() > 0
        # a failed slot load is an error of the step, not a crash, and not terminal
        assert win.fail_next_loads(100)
        with pytest.raises(eb.BackendError):
            sess.generate(first[0], pos[0], 2)
        assert win.fail_next_loads(0)
        assert sess.select_sequence(0) and resident.select_sequence(0)
        assert list(sess.generate(first[0], pos[0], 4)) == list(resident.generate(first[0], pos[0], 4))
    finally:
        sess.close()
        win.close()
        resident.close()
        evict_uploaded(be)


def test_window_attach_is_checked(be, port):
    types = {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}
    image, table = model_image(port, MODEL, types, seed=5)
    sess, win = streamed_session(be, image, table, MODEL, 2, 1, False)
    other = ew.LayerWindow(be)
    try:
        assert not sess.set_window(None)                     # streamed tensors are bound through it
        assert not sess.set_window(other)                    # and an unbound window streams nothing
        # a span that is neither resident nor an extent of that layer is refused
        off, size, t = table[(1, el.ATTN_Q)]
        assert not sess.bind_matrix(0, el.ATTN_Q, image[off:off + size], t)
        assert not sess.bind_matrix(1, el.ATTN_Q, image[off + 64:off + 64 + size], t)
        assert sess.bind_matrix(1, el.ATTN_Q, image[off:off + size], t)
    finally:
        sess.close()
        other.close()
        win.close()
        evict_uploaded(be)
