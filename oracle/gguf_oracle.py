"""CPU restatement of the reference's GGUF loader.  TEST INFRASTRUCTURE ONLY — the
product parses GGUF in its own C++ (emel.cpp_b200/csrc/gguf.cu) and never imports
this module.

Follows src/emel/gguf/loader/detail.hpp of the reference function by function:
`probe` = probe_requirements (419-543), `parse` = parse_bound_storage (545-733)
with storage sized by the probe.  Pinned against the reference's own known
answers (tests/gguf/loader/lifecycle_tests.cpp:260-348, 373-429) and, image for
image, against those two functions compiled in place (oracle/_ref, ref_shim.cpp:
ref_gguf_probe / ref_gguf_parse) in tests/test_gguf.py.
"""
from __future__ import annotations

NONE, INVALID_REQUEST, MODEL_INVALID, CAPACITY, PARSE_FAILED = 0, 1, 2, 4, 8   # errors.hpp:7-15
U32_MAX, U64_MAX = 0xFFFFFFFF, 0xFFFFFFFFFFFFFFFF
ALIGNMENT_KEY = b"general.alignment"

# detail.hpp:48-84: type -> (elements per block, bytes per block)
LAYOUT = {0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 9: (32, 36),
          10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292),
          16: (256, 66), 17: (256, 74), 18: (256, 98), 19: (256, 50), 20: (32, 18), 21: (256, 110), 22: (256, 82),
          23: (256, 136), 24: (1, 1), 25: (1, 2), 26: (1, 4), 27: (1, 8), 28: (1, 8), 29: (256, 56), 30: (1, 2),
          34: (256, 54), 35: (256, 66), 39: (32, 17)}
SCALAR_SIZE = {0: 1, 1: 1, 7: 1, 2: 2, 3: 2, 4: 4, 5: 4, 6: 4, 10: 8, 11: 8, 12: 8}      # detail.hpp:91-106


class _Fail(Exception):
    def __init__(self, err):
        self.err = err


class _Reader:
    """bounded_reader (detail.hpp:179-248)"""

    def __init__(self, data: bytes):
        self.b, self.off = data, 0

    def can_read(self, n):
        return n <= len(self.b) and self.off <= len(self.b) - n

    def scalar(self, width):
        if not self.can_read(width):
            return None
        v = int.from_bytes(self.b[self.off:self.off + width], "little")
        self.off += width
        return v

    def string(self):
        n = self.scalar(8)
        if n is None or not self.can_read(n):
            return None
        s = self.b[self.off:self.off + n]
        self.off += n
        return s

    def skip(self, n):
        if not self.can_read(n):
            return False
        self.off += n
        return True


def _pad(value, alignment):
    """pad_to_alignment (165-177): None on 64-bit overflow"""
    rem = value % alignment
    out = value if rem == 0 else value + alignment - rem
    return None if out > U64_MAX else out


def _header(r: _Reader):
    """read_header (264-286) -> (tensor_count, kv_count) or None"""
    if not r.can_read(4):
        return None
    magic = r.b[r.off:r.off + 4]
    r.off += 4
    if magic != b"GGUF":
        return None
    version, tensors, kvs = r.scalar(4), r.scalar(8), r.scalar(8)
    if version is None or tensors is None or kvs is None:
        return None
    return (tensors, kvs) if version == 3 else None


def _value(r: _Reader, vtype, key, alignment):
    """scan_value_payload (288-370) -> alignment in force afterwards; raises _Fail"""
    if vtype >= 13:
        raise _Fail(MODEL_INVALID)
    if vtype == 8:
        if r.string() is None:
            raise _Fail(PARSE_FAILED)
        return alignment
    if vtype == 9:
        elem, count = r.scalar(4), None
        if elem is not None:
            count = r.scalar(8)
        if elem is None or count is None:
            raise _Fail(PARSE_FAILED)
        if elem >= 13 or elem == 9:
            raise _Fail(MODEL_INVALID)
        if elem == 8:
            for _ in range(count):
                if r.string() is None:
                    raise _Fail(PARSE_FAILED)
        else:
            payload = count * SCALAR_SIZE[elem]
            if payload > U64_MAX:
                raise _Fail(CAPACITY)
            if not r.skip(payload):
                raise _Fail(PARSE_FAILED)
        return alignment
    if key == ALIGNMENT_KEY:
        if vtype != 4:
            raise _Fail(MODEL_INVALID)
        a = r.scalar(4)
        if a is None:
            raise _Fail(PARSE_FAILED)
        if a == 0 or a & (a - 1):
            raise _Fail(MODEL_INVALID)
        return a
    if not r.skip(SCALAR_SIZE[vtype]):
        raise _Fail(PARSE_FAILED)
    return alignment


def tensor_data_size(dims, n_dims, ttype):
    """compute_tensor_data_size (372-403) and the row-group-packed case (135-163); raises _Fail"""
    if ttype in (41, 42):
        if n_dims < 2 or n_dims > 4 or dims[0] % 256:
            raise _Fail(MODEL_INVALID)
        rows = 1
        for d in range(1, n_dims):
            rows *= dims[d]
            if rows > U64_MAX:
                raise _Fail(CAPACITY)
        groups = rows // 8 + (1 if rows % 8 else 0)
        cells = groups * (dims[0] // 256)
        if cells > U64_MAX or cells * 1152 > U64_MAX:
            raise _Fail(CAPACITY)
        return cells * 1152
    if ttype not in LAYOUT:
        raise _Fail(MODEL_INVALID)
    be, bb = LAYOUT[ttype]
    if (1 if n_dims == 0 else dims[0]) % be:
        raise _Fail(MODEL_INVALID)
    elems = 1
    for d in range(n_dims):
        elems *= dims[d]
        if elems > U64_MAX:
            raise _Fail(CAPACITY)
    size = elems // be * bb
    if size > U64_MAX:
        raise _Fail(CAPACITY)
    return size


def _walk(data: bytes, req: dict, kvs: list | None, tensors: list | None):
    r = _Reader(data)
    head = _header(r)
    if head is None:
        raise _Fail(PARSE_FAILED if len(data) < 4 else MODEL_INVALID)
    n_tensors, n_kv = head
    if n_tensors > U32_MAX or n_kv > U32_MAX:
        raise _Fail(CAPACITY)
    req["tensor_count"], req["kv_count"] = n_tensors, n_kv
    alignment = 32
    for _ in range(n_kv):
        key = r.string()
        vtype = r.scalar(4) if key is not None else None
        if key is None or vtype is None:
            raise _Fail(PARSE_FAILED)
        if len(key) > U32_MAX:
            raise _Fail(CAPACITY)
        start = r.off
        alignment = _value(r, vtype, key, alignment)
        size = r.off - start
        if size > U32_MAX:
            raise _Fail(CAPACITY)
        req["max_key_bytes"] = max(req["max_key_bytes"], len(key))
        req["max_value_bytes"] = max(req["max_value_bytes"], size)
        if kvs is not None:
            kvs.append((key, vtype, data[start:start + size]))
    expected = 0
    for _ in range(n_tensors):
        name = r.string()
        n_dims = r.scalar(4) if name is not None else None
        if name is None or n_dims is None:
            raise _Fail(PARSE_FAILED)
        if len(name) > U32_MAX:
            raise _Fail(CAPACITY)
        if n_dims > 4:
            raise _Fail(MODEL_INVALID)
        dims = [1, 1, 1, 1]
        for d in range(n_dims):
            dims[d] = r.scalar(8)
            if dims[d] is None:
                raise _Fail(PARSE_FAILED)
        ttype = r.scalar(4)
        offset = r.scalar(8) if ttype is not None else None
        if ttype is None or offset is None:
            raise _Fail(PARSE_FAILED)
        size = tensor_data_size(dims, n_dims, ttype)
        if req["tensor_data_bytes"] + size > U64_MAX:
            raise _Fail(CAPACITY)
        req["tensor_data_bytes"] += size
        if offset != expected:
            raise _Fail(PARSE_FAILED)
        padded = _pad(size, alignment)
        if padded is None or expected + padded > U64_MAX:
            raise _Fail(CAPACITY)
        expected += padded
        if tensors is not None:
            tensors.append({"name": name, "type": ttype, "n_dims": n_dims, "dims": tuple(dims),
                            "data_offset": offset, "data_size": size})
    section = _pad(r.off, alignment)
    if section is None or section > len(data):
        raise _Fail(PARSE_FAILED)
    if section + expected > U64_MAX:
        raise _Fail(CAPACITY)
    if section + expected > len(data):
        raise _Fail(PARSE_FAILED)
    return alignment, section


def _new_req():
    return {"tensor_count": 0, "kv_count": 0, "max_key_bytes": 0, "max_value_bytes": 0, "tensor_data_bytes": 0}


def probe(data: bytes):
    """-> (error, requirements dict); the requirements keep what was read before a failure"""
    if data is None or len(data) == 0:
        return INVALID_REQUEST, _new_req()       # guards.hpp:9-11
    req = _new_req()
    try:
        _walk(data, req, None, None)
    except _Fail as f:
        return f.err, req
    return NONE, req


def parse(data: bytes):
    """-> (error, kv entries [(key, type, payload)], tensor records with file_offset)"""
    if data is None or len(data) == 0:
        return INVALID_REQUEST, [], []
    req, kvs, tensors = _new_req(), [], []
    try:
        _alignment, section = _walk(data, req, kvs, tensors)
    except _Fail as f:
        return f.err, [], []
    for t in tensors:
        t["file_offset"] = section + t["data_offset"]
        if t["file_offset"] + t["data_size"] > len(data):
            return PARSE_FAILED, [], []
    return NONE, kvs, tensors
