"""CPU restatement of the reference's layer streaming window (test infrastructure only: nothing
the library ships imports this file).

Follows src/emel/model/tensor/window: the slot plan (detail.hpp:128-183), the bind decisions in
the order of the transition table (guards.hpp:13-186; errors.hpp:9-21) and the ring
(guards.hpp:296-470, actions.hpp:218-227 and 394-406), as a model that records which loads an
acquire sequence submits.  Parity unpinned against a running reference: the actor needs the
state-machine library `stateforward/sml.hpp`, which the reference tree does not vendor, so it
cannot be compiled here.  The pins are the reference's own test expectations, read as text
(tests/model/tensor/window/lifecycle_tests.cpp and streaming_tests.cpp with the fixture in
window_test_fixture.hpp:21-24, 177-225): tests/test_window_oracle.py replays them on this model.
"""
from __future__ import annotations

NONE, INVALID_REQUEST, NOT_BOUND, ALREADY_BOUND, SOURCE_MAP_FAILED, BUDGET_TOO_SMALL, LAYER_OUT_OF_RANGE, SLOT_COPY_FAILED, \
    NOT_STREAMING, INTERNAL_ERROR, SLOT_STORAGE_TOO_SMALL = [0] + [1 << i for i in range(10)]

MAX_SLOTS, MAX_LAYERS, MAX_WEIGHTS = 8, 160, 12                       # detail.hpp:17-19
MIN_CHUNK, DEFAULT_CHUNK, MAX_CHUNK = 1 << 20, 8 << 20, 16 << 20      # detail.hpp:21-23
ALIGN = 64                                                            # detail.hpp:24
MAX_MAPPING = 1 << 40                                                 # io::mmap's cap on one mapping


def aligned(n):
    """compute_aligned_bytes, detail.hpp:128-131."""
    return (n + ALIGN - 1) & ~(ALIGN - 1)


def scan_layers(layers):
    """scan_layer_descriptors, detail.hpp:135-167.  layers: per layer a list of
    (tensor_id, file_offset, byte_size).  Returns per layer a dict and the slot capacity."""
    plan, capacity = [], 0
    for weights in layers:
        at, offs, lo, hi = 0, [], None, 0
        for _tid, off, size in weights:
            offs.append(at)
            at += aligned(size)
            lo = off if lo is None or off < lo else lo
            hi = max(hi, off + size)
        plan.append({"slot_offsets": offs, "slot_bytes": at, "file_begin": lo or 0, "file_span": hi - (lo or 0) if weights else 0})
        capacity = max(capacity, at)
    return plan, capacity


def request_valid(file_size, layers, chunk, has_source=True):
    """guard_bind_request_valid, guards.hpp:13-60 (without the actor-wiring checks)."""
    if not has_source or file_size == 0:
        return False
    if len(layers) == 0 or len(layers) > MAX_LAYERS:
        return False
    for weights in layers:
        if len(weights) == 0 or len(weights) > MAX_WEIGHTS:
            return False
    for weights in layers:
        for _tid, off, size in weights:
            if size == 0 or size > file_size or off > file_size - size:
                return False
    return MIN_CHUNK <= chunk <= MAX_CHUNK


def bind_decision(file_size, layers, budget, slots, depth, storage_bytes, storage_aligned=True, storage_null=False,
                  chunk=DEFAULT_CHUNK, already_bound=False, source_ok=True):
    """-> (error, streaming_active).  The order of the bind chain: request, source mapping,
    budget fit (passthrough), streaming configuration, slots against the budget, storage."""
    if already_bound:
        return ALREADY_BOUND, False
    if not request_valid(file_size, layers, chunk):
        return INVALID_REQUEST, False
    if not source_ok or file_size > MAX_MAPPING:
        return SOURCE_MAP_FAILED, False
    plan, capacity = scan_layers(layers)
    total = sum(d["slot_bytes"] for d in plan)
    if budget == 0 or total <= budget:                                   # guards.hpp:83-90
        return NONE, False
    if not (2 <= slots <= MAX_SLOTS and 0 < depth < slots):             # guards.hpp:94-108
        return INVALID_REQUEST, False
    if slots * capacity > budget:                                        # guards.hpp:124-131
        return BUDGET_TOO_SMALL, False
    if storage_null or storage_bytes < slots * capacity or not storage_aligned:   # guards.hpp:135-149
        return SLOT_STORAGE_TOO_SMALL, False
    return NONE, True


class Ring:
    """The residency ring of a streaming bind: which layer each slot holds and which loads are
    submitted, for loads that always succeed unless `fail` names their ordinal."""

    def __init__(self, n_layers, slots, depth, fail=()):
        self.n, self.slots, self.depth = n_layers, slots, depth
        self.layer = [-1] * slots      # window_slot.layer
        self.failed = [False] * slots
        self.loads = []                # (layer, slot) in submission order
        self.fail = set(fail)
        self.resident_hits = self.cold = 0
        for l in range(min(depth, n_layers)):   # effect_prime_window, actions.hpp:218-227
            self._submit(l)

    def _submit(self, layer):
        slot = layer % self.slots      # compute_slot_for_layer, detail.hpp:123-126
        self.layer[slot] = layer
        self.failed[slot] = len(self.loads) in self.fail
        self.loads.append((layer, slot))

    def acquire(self, layer):
        """-> error bits.  guards.hpp:296-470: out of range; resident or loading -> wait;
        unscheduled -> submit; failed -> one more submit; then advance."""
        if layer < 0 or layer >= self.n:
            return LAYER_OUT_OF_RANGE
        slot = layer % self.slots
        if self.layer[slot] == layer:
            self.resident_hits += 1
        else:
            self.cold += 1
            self._submit(layer)
        if self.failed[slot]:
            self._submit(layer)
        if self.failed[slot]:
            return SLOT_COPY_FAILED
        ahead = (layer + self.depth) % self.n          # guards.hpp:433-452
        target = ahead % self.slots
        if target != slot and self.layer[target] != ahead:
            self._submit(ahead)
        return NONE
