"""Layer streaming window bindings (include/emelb_window.h): the reference's
model::tensor::window requests (src/emel/model/tensor/window/events.hpp:26-70)
with the slots in HBM and the source in host memory."""
from __future__ import annotations

import ctypes as C
import os

import emel_cpp_b200 as eb

_P = C.c_void_p

# src/emel/model/tensor/window/errors.hpp:9-21
OK, INVALID_REQUEST, NOT_BOUND, ALREADY_BOUND, SOURCE_MAP_FAILED, BUDGET_TOO_SMALL, LAYER_OUT_OF_RANGE, SLOT_COPY_FAILED, \
    NOT_STREAMING, INTERNAL_ERROR, SLOT_STORAGE_TOO_SMALL = [0] + [1 << i for i in range(10)]

# src/emel/model/tensor/window/detail.hpp:17-25
MAX_SLOTS, MAX_LAYERS, MAX_WEIGHTS_PER_LAYER = 8, 160, 12
MIN_CHUNK_BYTES, DEFAULT_CHUNK_BYTES, MAX_CHUNK_BYTES = 1 << 20, 8 << 20, 16 << 20
SLOT_ALIGNMENT = 64


class Extent(C.Structure):
    _fields_ = [("tensor_id", C.c_int32), ("file_offset", C.c_uint64), ("byte_size", C.c_uint64), ("slot_offset", C.c_uint64)]


class Layer(C.Structure):
    _fields_ = [("weights", Extent * MAX_WEIGHTS_PER_LAYER), ("weight_count", C.c_uint32), ("file_begin", C.c_uint64),
                ("file_span", C.c_uint64), ("slot_bytes", C.c_uint64)]


class Request(C.Structure):
    _fields_ = [("file_path", C.c_char_p), ("file_size_bytes", C.c_uint64), ("source", _P), ("extents", C.POINTER(Extent)),
                ("extent_count", C.c_uint64), ("layer_weight_counts", C.POINTER(C.c_uint16)), ("layer_count", C.c_uint64),
                ("budget_bytes", C.c_uint64), ("slot_storage", _P), ("slot_storage_bytes", C.c_uint64),
                ("window_slots", C.c_uint32), ("prefetch_depth", C.c_uint32), ("stage_chunk_bytes", C.c_uint64)]


class Bound(C.Structure):
    _fields_ = [("streaming_active", C.c_int32), ("source_base", _P), ("source_bytes", C.c_uint64),
                ("window_slots", C.c_uint32), ("source_page_locked", C.c_int32)]


class Stats(C.Structure):
    _fields_ = [("loads_submitted", C.c_uint64), ("loads_failed", C.c_uint64), ("bytes_copied", C.c_uint64),
                ("acquires", C.c_uint64), ("acquires_resident", C.c_uint64), ("acquires_cold", C.c_uint64)]

    def as_dict(self):
        return {name: int(getattr(self, name)) for name, _ in self._fields_}


SIGNATURES = {
    "emelb_window_create": [_P, C.POINTER(_P)],
    "emelb_window_destroy": [_P],
    "emelb_window_bind": [_P, C.POINTER(Request), C.POINTER(Bound)],
    "emelb_window_check": [C.POINTER(Request), C.POINTER(C.c_int32), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)],
    "emelb_window_acquire": [_P, C.c_int32, C.POINTER(_P), C.POINTER(C.POINTER(Layer))],
    "emelb_window_unbind": [_P],
    "emelb_window_get_stats": [_P, C.POINTER(Stats)],
    "emelb_window_layer_plan": [_P, C.c_int32, C.POINTER(C.POINTER(Layer)), C.POINTER(C.c_uint64)],
    "emelb_window_fail_next_loads": [_P, C.c_int32],
    "emelb_window_set_staged_only": [_P, C.c_int32],
    "emelb_llama_set_window": [_P, _P],
}


def register(lib):
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = C.c_uint32
        fn.argtypes = args


def aligned(n: int) -> int:
    return (n + SLOT_ALIGNMENT - 1) & ~(SLOT_ALIGNMENT - 1)


def plan_layers(layers):
    """The slot plan of scan_layer_descriptors (src/emel/model/tensor/window/detail.hpp:128-167) for
    `layers` = one list of (tensor_id, file_offset, byte_size) per layer: per layer the list of
    slot offsets and its slot_bytes, and the slot capacity (the largest layer)."""
    offsets, sizes = [], []
    for weights in layers:
        at, offs = 0, []
        for _tid, _off, size in weights:
            offs.append(at)
            at += aligned(size)
        offsets.append(offs)
        sizes.append(at)
    return offsets, sizes, max(sizes, default=0)


def check_request(file_size: int, layers, budget_bytes: int, window_slots: int = 0, prefetch_depth: int = 0,
                  stage_chunk_bytes: int = DEFAULT_CHUNK_BYTES, slot_storage: int = 0, slot_storage_bytes: int = 0,
                  file_path: bytes = b"model.gguf"):
    """emelb_window_check: the bind decisions for a request, without a GPU.
    -> (error bits, streaming_active, slot capacity, packed bytes of all layers)"""
    req = Request()
    req.file_path, req.file_size_bytes = file_path, file_size
    flat = [w for weights in layers for w in weights]
    ext = (Extent * max(1, len(flat)))()
    for i, (tid, off, size) in enumerate(flat):
        ext[i].tensor_id, ext[i].file_offset, ext[i].byte_size = tid, off, size
    counts = (C.c_uint16 * max(1, len(layers)))(*[len(w) for w in layers])
    req.extents, req.extent_count = ext, len(flat)
    req.layer_weight_counts, req.layer_count = counts, len(layers)
    req.budget_bytes, req.window_slots, req.prefetch_depth = budget_bytes, window_slots, prefetch_depth
    req.stage_chunk_bytes = stage_chunk_bytes
    req.slot_storage, req.slot_storage_bytes = slot_storage, slot_storage_bytes
    streaming, cap, total = C.c_int32(0), C.c_uint64(0), C.c_uint64(0)
    err = eb.lib().emelb_window_check(C.byref(req), C.byref(streaming), C.byref(cap), C.byref(total))
    return int(err), bool(streaming.value), int(cap.value), int(total.value)


def slot_of(layer: int, window_slots: int) -> int:
    """compute_slot_for_layer, src/emel/model/tensor/window/detail.hpp:123-126."""
    return layer % window_slots


class LayerWindow:
    """One window actor on a backend context.  bind() takes the source (a path, or host memory that is kept alive
    here), the per-layer extents and the budget; slot storage is a device tensor this object allocates unless one is
    passed in."""

    def __init__(self, backend: eb.Backend):
        self.be = backend
        self._h = _P()
        err = eb.lib().emelb_window_create(backend.handle, C.byref(self._h))
        if err != OK:
            raise eb.BackendError(f"emelb_window_create failed with error mask {err}")
        self.last_error = OK
        self._keep = []
        self.bound = None

    @property
    def handle(self):
        return self._h

    def close(self):
        if self._h:
            eb.lib().emelb_window_destroy(self._h)
            self._h = _P()
            self._keep = []

    def set_staged_only(self, on: bool) -> bool:
        self.last_error = eb.lib().emelb_window_set_staged_only(self._h, 1 if on else 0)
        return self.last_error == OK

    def fail_next_loads(self, count: int) -> bool:
        self.last_error = eb.lib().emelb_window_fail_next_loads(self._h, count)
        return self.last_error == OK

    def bind(self, source, layers, budget_bytes: int, window_slots: int = 0, prefetch_depth: int = 0,
             stage_chunk_bytes: int = DEFAULT_CHUNK_BYTES, slot_storage="auto", source_bytes: int | None = None) -> bool:
        """`source`: a path, a numpy / torch host buffer, or an integer address with source_bytes.  `layers`: one
        list of (tensor_id, file_offset, byte_size) per layer.  slot_storage: "auto" allocates
        window_slots x capacity bytes on the backend's GPU when the request will stream; None passes no storage; a
        torch CUDA tensor is passed as it is."""
        import torch
        req = Request()
        keep = []
        if isinstance(source, (str, os.PathLike)):
            path = os.fsencode(source)
            req.file_path = path
            req.file_size_bytes = os.path.getsize(source) if source_bytes is None else source_bytes
            keep.append(path)
        else:
            req.source = eb.ptr(source)
            if source_bytes is None:
                source_bytes = source.nbytes if hasattr(source, "nbytes") else source.numel() * source.element_size()
            req.file_size_bytes = source_bytes
            keep.append(source)
        flat = [w for weights in layers for w in weights]
        ext = (Extent * max(1, len(flat)))()
        for i, (tid, off, size) in enumerate(flat):
            ext[i].tensor_id, ext[i].file_offset, ext[i].byte_size = tid, off, size
        counts = (C.c_uint16 * max(1, len(layers)))(*[len(w) for w in layers])
        req.extents, req.extent_count = ext, len(flat)
        req.layer_weight_counts, req.layer_count = counts, len(layers)
        req.budget_bytes, req.window_slots, req.prefetch_depth = budget_bytes, window_slots, prefetch_depth
        req.stage_chunk_bytes = stage_chunk_bytes
        _offs, sizes, capacity = plan_layers(layers)
        if isinstance(slot_storage, str) and slot_storage == "auto":
            slot_storage = None
            if budget_bytes and sum(sizes) > budget_bytes and 0 < window_slots <= MAX_SLOTS:
                slot_storage = torch.empty(max(1, window_slots * capacity), dtype=torch.uint8, device=f"cuda:{self.be.device}")
        if slot_storage is not None:
            req.slot_storage = slot_storage.data_ptr()
            req.slot_storage_bytes = slot_storage.numel() * slot_storage.element_size()
            keep.append(slot_storage)
        out = Bound()
        self.last_error = eb.lib().emelb_window_bind(self._h, C.byref(req), C.byref(out))
        if self.last_error != OK:
            return False
        self._keep = keep
        self.bound = {"streaming_active": bool(out.streaming_active), "source_base": out.source_base or 0,
                      "source_bytes": int(out.source_bytes), "window_slots": int(out.window_slots),
                      "source_page_locked": bool(out.source_page_locked), "slot_capacity": capacity}
        return True

    def acquire(self, layer: int):
        """-> (device address of the slot, [(tensor_id, file_offset, byte_size, slot_offset), ...]) or None."""
        base, lay = _P(), C.POINTER(Layer)()
        self.last_error = eb.lib().emelb_window_acquire(self._h, layer, C.byref(base), C.byref(lay))
        if self.last_error != OK:
            return None
        d = lay.contents
        return base.value, [(d.weights[i].tensor_id, d.weights[i].file_offset, d.weights[i].byte_size, d.weights[i].slot_offset)
                            for i in range(d.weight_count)]

    def layer_plan(self, layer: int):
        lay, cap = C.POINTER(Layer)(), C.c_uint64(0)
        self.last_error = eb.lib().emelb_window_layer_plan(self._h, layer, C.byref(lay), C.byref(cap))
        if self.last_error != OK:
            return None
        d = lay.contents
        return {"slot_offsets": [int(d.weights[i].slot_offset) for i in range(d.weight_count)], "slot_bytes": int(d.slot_bytes),
                "file_begin": int(d.file_begin), "file_span": int(d.file_span), "slot_capacity": int(cap.value)}

    def unbind(self) -> bool:
        self.last_error = eb.lib().emelb_window_unbind(self._h)
        if self.last_error == OK:
            self._keep = []
            self.bound = None
        return self.last_error == OK

    def stats(self) -> dict:
        s = Stats()
        eb.lib().emelb_window_get_stats(self._h, C.byref(s))
        return s.as_dict()
