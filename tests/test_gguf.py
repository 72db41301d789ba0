"""GGUF loader parity on the CPU: the library's parser (include/emelb_gguf.h), the
oracle's restatement (oracle/gguf_oracle.py) and the reference's own functions
compiled in place (oracle/_ref) must give the same error, the same requirements
and the same records for valid and malformed images.  Bar: identical."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

import emel_cpp_b200 as eb
from emel_cpp_b200 import gguf
from oracle import bindings as ob, gguf_oracle as go
from emel_cpp_b200 import gguf_image as gi
from tests.golden.make_gguf_golden import apply, corruptions

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gguf_golden.npz")


def lib_probe(image: bytes):
    err, req = gguf.probe(image)
    return err, req.as_tuple()


def oracle_probe(image: bytes):
    err, req = go.probe(image)
    return err, tuple(req.values())


def lib_parse(image: bytes):
    """-> (error, kv entries, tensor records) in the shape the oracle gives them"""
    try:
        f = gguf.File(image)
    except gguf.GgufError as e:
        return e.err, [], []
    with f:
        kvs = [f.kv(i, raw_key=True) for i in range(f.requirements.kv_count)]
        tensors = [{"name": t["name_bytes"], "type": t["type"], "n_dims": t["n_dims"], "dims": t["dims"],
                    "data_offset": t["data_offset"], "file_offset": t["file_offset"], "data_size": t["data_size"]}
                   for t in f.tensors()]
    return 0, kvs, tensors


def strip(tensors):
    return [{k: t[k] for k in ("name", "type", "n_dims", "dims", "data_offset", "file_offset", "data_size")} for t in tensors]


# ---------------------------------------------------------------- the reference's own known answers
def test_reference_known_answers():
    """tests/gguf/loader/lifecycle_tests.cpp:260-348 (sizes and records of the valid image),
    350-371 (no image), 373-429 (bad magic, bad version, truncation)."""
    image = gi.reference_valid_file()
    for probe in (lib_probe, oracle_probe):
        assert probe(image) == (0, (1, 2, 17, 35, 24))
        assert probe(b"")[0] == gguf.INVALID_REQUEST
        assert probe(b"F" + image[1:])[0] == gguf.MODEL_INVALID
        assert probe(image[:4] + b"\x04" + image[5:])[0] == gguf.MODEL_INVALID
        assert probe(image[:-1])[0] == gguf.PARSE_FAILED
    for parse in (lib_parse, go.parse):
        err, kvs, tensors = parse(image)
        assert err == 0
        assert kvs[0] == (b"general.alignment", gguf.T_UINT32, struct.pack("<I", 32))
        assert kvs[1][0] == b"tokenizer.tokens" and kvs[1][1] == gguf.T_ARRAY and len(kvs[1][2]) == 35
        assert struct.unpack_from("<IQ", kvs[1][2]) == (gguf.T_STRING, 2)
        t = tensors[0]
        assert (t["name"], t["type"], t["n_dims"], t["dims"][:2]) == (b"weights.f32", 0, 2, (2, 3))
        assert (t["data_offset"], t["data_size"]) == (0, 24) and t["file_offset"] == len(image) - 32
        assert parse(image[:-1])[0] == gguf.PARSE_FAILED
    with gguf.File(image) as f:
        assert f.get("tokenizer.tokens") == ["hi", "world"] and f.get("general.alignment") == 32
        assert f.alignment == 32 and f.data_section_offset == len(image) - 32
        rec = f.find_tensor("weights.f32")
        assert C.string_at(rec["data"], rec["data_size"]) == image[rec["file_offset"]:rec["file_offset"] + 24]


def test_packed_row_group_ceiling_does_not_overflow():
    """tests/gguf/loader/lifecycle_tests.cpp:644-656"""
    with pytest.raises(go._Fail) as e:
        go.tensor_data_size([256, 2 ** 64 - 1, 1, 1], 2, 41)
    assert e.value.err == gguf.CAPACITY
    image = b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + gi.tensor_info("p", (256, 2 ** 64 - 1), 41, 0)
    assert lib_probe(image)[0] == gguf.CAPACITY


# ---------------------------------------------------------------- golden fixture (reference outputs)
@pytest.mark.parametrize("name", ["valid", "rich"])
def test_golden_cases(name):
    g = np.load(GOLDEN)
    image = g[name + "_image"].tobytes()
    for probe in (lib_probe, oracle_probe):
        for kind, pos, value, err, *req in g[name + "_cases"].tolist():
            got = probe(apply(image, kind, pos, value))
            if kind == 0 and pos == 0:
                assert got[0] == gguf.INVALID_REQUEST      # the shim applies the request guard the same way
            assert got == (err, tuple(req)), (probe.__name__, kind, pos, value, got, err, req)
    want = g[name + "_tensors"].tolist()
    for parse in (lib_parse, go.parse):
        err, _kvs, tensors = parse(image)
        assert err == 0
        got = [[t["type"], t["n_dims"], *t["dims"], t["data_offset"], t["file_offset"], t["data_size"]] for t in tensors]
        assert got == want


def test_golden_fixture_is_current():
    """The committed fixture holds exactly the images the writer makes today."""
    g = np.load(GOLDEN)
    assert g["valid_image"].tobytes() == gi.reference_valid_file()
    assert g["rich_image"].tobytes() == gi.rich_file(0)


# ---------------------------------------------------------------- three-way agreement, live
def crafted_images():
    """(name, image, expected error or None): one malformation per check of the loader."""
    u32, u64 = (lambda v: struct.pack("<I", v)), (lambda v: struct.pack("<Q", v))
    head = lambda nt, nkv, version=3: b"GGUF" + u32(version) + u64(nt) + u64(nkv)
    f32 = lambda name, dims, off, t=0: gi.tensor_info(name, dims, t, off)
    pad32 = lambda b: b + b"\0" * (gi.pad(len(b), 32) - len(b))
    out = [
        ("three bytes", b"GGU", gguf.PARSE_FAILED),
        ("magic only", b"GGUF", gguf.MODEL_INVALID),
        ("version 2", head(0, 0, 2), gguf.MODEL_INVALID),
        ("empty model", pad32(head(0, 0)), 0),
        ("empty model, unpadded", head(0, 0), gguf.PARSE_FAILED),   # 24 bytes: padding to 32 leaves the image
        ("tensor count over 32 bits", head(1 << 32, 0), gguf.CAPACITY),
        ("kv count over 32 bits", head(0, 1 << 32), gguf.CAPACITY),
        ("kv missing", head(0, 1), gguf.PARSE_FAILED),
        ("value type 13", head(0, 1) + gi.gstr("k") + u32(13), gguf.MODEL_INVALID),
        ("array of arrays", head(0, 1) + gi.gstr("k") + u32(9) + u32(9) + u64(0), gguf.MODEL_INVALID),
        ("array element type 99", head(0, 1) + gi.gstr("k") + u32(9) + u32(99) + u64(0), gguf.MODEL_INVALID),
        ("array payload overflow", head(0, 1) + gi.gstr("k") + u32(9) + u32(10) + u64(1 << 62), gguf.CAPACITY),
        ("array payload short", head(0, 1) + gi.gstr("k") + u32(9) + u32(4) + u64(3) + b"\0" * 11, gguf.PARSE_FAILED),
        ("string length past the end", head(0, 1) + gi.gstr("k") + u32(8) + u64(1 << 63), gguf.PARSE_FAILED),
        ("alignment as u64", head(0, 1) + gi.kv("general.alignment", gi.T_UINT64, 32), gguf.MODEL_INVALID),
        ("alignment zero", head(0, 1) + gi.kv("general.alignment", gi.T_UINT32, 0), gguf.MODEL_INVALID),
        ("alignment 48", head(0, 1) + gi.kv("general.alignment", gi.T_UINT32, 48), gguf.MODEL_INVALID),
        ("alignment as string", pad32(head(0, 1) + gi.kv("general.alignment", gi.T_STRING, "x")), 0),
        ("alignment 1", head(0, 1) + gi.kv("general.alignment", gi.T_UINT32, 1), 0),
        ("alignment 2^31", head(0, 1) + gi.kv("general.alignment", gi.T_UINT32, 1 << 31), gguf.PARSE_FAILED),
        ("five dimensions", head(1, 0) + gi.gstr("t") + u32(5), gguf.MODEL_INVALID),
        ("dimension missing", head(1, 0) + gi.gstr("t") + u32(2) + u64(4), gguf.PARSE_FAILED),
        ("tensor type 4", head(1, 0) + f32("t", (32,), 0, 4), gguf.MODEL_INVALID),
        ("tensor type 31", head(1, 0) + f32("t", (32,), 0, 31), gguf.MODEL_INVALID),
        ("tensor type 43", head(1, 0) + f32("t", (256, 8), 0, 43), gguf.MODEL_INVALID),
        ("row not whole blocks", head(1, 0) + f32("t", (100, 2), 0, 12), gguf.MODEL_INVALID),
        ("no dimensions, block type", head(1, 0) + f32("t", (), 0, 8), gguf.MODEL_INVALID),
        ("element count overflow", head(1, 0) + f32("t", (1 << 40, 1 << 40), 0), gguf.CAPACITY),
        ("byte count overflow", head(1, 0) + f32("t", (1 << 62,), 0), gguf.CAPACITY),
        ("packed, one dimension", head(1, 0) + f32("t", (256,), 0, 41), gguf.MODEL_INVALID),
        ("packed, ragged columns", head(1, 0) + f32("t", (128, 8), 0, 42), gguf.MODEL_INVALID),
        ("offset not the running one", pad32(head(1, 0) + f32("t", (8,), 32)) + b"\0" * 64, gguf.PARSE_FAILED),
        ("second offset unpadded", pad32(head(2, 0) + f32("a", (3,), 0) + f32("b", (3,), 12)) + b"\0" * 64, gguf.PARSE_FAILED),
        ("two tensors", pad32(head(2, 0) + f32("a", (3,), 0) + f32("b", (3,), 32)) + b"\0" * 64, 0),
        ("data one byte short", pad32(head(2, 0) + f32("a", (3,), 0) + f32("b", (3,), 32)) + b"\0" * 63, gguf.PARSE_FAILED),
        ("zero-sized tensor", pad32(head(1, 0) + f32("z", (0, 4), 0)), 0),
        ("total bytes overflow", head(2, 0) + f32("a", (1 << 61,), 0) + f32("b", (1 << 61,), 1 << 63), gguf.CAPACITY),
        ("reference image", gi.reference_valid_file(), 0),
        ("every value type", gi.rich_file(3), 0),
    ]
    return out


def test_crafted_images_three_way():
    ref = ob.ref()
    for name, image, want in crafted_images():
        got = lib_probe(image)
        assert got[0] == want, (name, got)
        assert oracle_probe(image) == got, name
        lp, op = lib_parse(image), go.parse(image)
        assert lp[0] == op[0] == want, name
        assert lp[1] == op[1] and strip(lp[2]) == strip(op[2]), name
        if ref is not None:
            assert ref.gguf_probe(image) == got, name
            rp = ref.gguf_parse(image)
            assert rp[0] == want and rp[1] == lp[1] and strip(rp[2]) == strip(lp[2]), name


def test_random_corruptions_three_way():
    """Seeded byte, bit and length corruptions of a rich image beyond the fixture's set, against
    the oracle and (where built) the reference; records are compared whenever the image still parses."""
    ref = ob.ref()
    rng = np.random.default_rng(11)
    image = gi.rich_file(5)
    head = gguf.File(image).data_section_offset
    still_valid = 0
    for _ in range(1500):
        m = bytearray(image)
        for _k in range(int(rng.integers(1, 4))):
            pos = int(rng.integers(0, head))
            m[pos] = int(rng.integers(0, 256)) if rng.random() < 0.5 else m[pos] ^ (1 << int(rng.integers(0, 8)))
        if rng.random() < 0.2:
            m = m[:int(rng.integers(1, len(m)))]
        m = bytes(m)
        got = lib_probe(m)
        assert got == oracle_probe(m)
        lp = lib_parse(m)
        assert lp[0] == got[0]
        if ref is not None:
            assert ref.gguf_probe(m) == got
        if got[0] == 0:
            still_valid += 1
            op = go.parse(m)
            assert lp[1] == op[1] and strip(lp[2]) == strip(op[2])
            if ref is not None:
                rp = ref.gguf_parse(m)
                assert rp[1] == lp[1] and strip(rp[2]) == strip(lp[2])
    assert 50 < still_valid < 1450


# ---------------------------------------------------------------- handle API (no GPU)
def test_file_mapping_and_lookups(tmp_path):
    image = gi.rich_file(0)
    p = tmp_path / "rich.gguf"
    p.write_bytes(image)
    with gguf.File(str(p)) as f:
        assert f.requirements.as_tuple() == lib_probe(image)[1]
        assert f.alignment == 64
        names = [t["name"] for t in f.tensors()]
        assert names == ["t.f32", "t.f16", "t.q4_k", "t.q6_k", "t.q8_0", "t.q4_0", "t.scalar", "t.packed", "t.i32"]
        for t in f.tensors():
            got = C.string_at(t["data"], t["data_size"])
            assert got == image[t["file_offset"]:t["file_offset"] + t["data_size"]]
            assert t["file_offset"] % 64 == 0
        assert f.find_tensor("t.q4") is None and f.find_tensor("t.q4_k")["type"] == eb.Q4_K
        assert f.get("a.i8") == -3 and f.get("a.u64") == 1 << 40 and f.get("a.f64") == 2.25 and f.get("a.bool") is True
        assert f.get("a.floats") == [0.5, 1.5, 2.5] and f.get("a.strings") == ["", "x", "a longer token"]
        assert f.get("a.empty") == [] and f.get("missing", 7) == 7
        lib = eb.lib()
        rec = gguf.TensorRecord()
        assert lib.emelb_gguf_tensor_at(f.handle, 9, C.byref(rec)) == gguf.INVALID_REQUEST
        assert lib.emelb_gguf_kv_at(f.handle, 16, C.byref(gguf.KvRecord())) == gguf.INVALID_REQUEST
        assert lib.emelb_gguf_upload(None, f.handle, 0, 1, None) == gguf.INVALID_REQUEST
        assert lib.emelb_gguf_upload_rows(None, f.handle, 2, 1, 0, 1, None, None) == gguf.INVALID_REQUEST
    empty = tmp_path / "empty.gguf"
    empty.write_bytes(b"")
    h = C.c_void_p()
    assert eb.lib().emelb_gguf_open_file(str(empty).encode(), C.byref(h)) == gguf.INVALID_REQUEST
    assert eb.lib().emelb_gguf_open_file(str(tmp_path / "absent.gguf").encode(), C.byref(h)) == gguf.INVALID_REQUEST
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(image[:100])
    assert eb.lib().emelb_gguf_open_file(str(bad).encode(), C.byref(h)) == gguf.PARSE_FAILED and not h.value
    assert eb.lib().emelb_gguf_close(None) == gguf.INVALID_REQUEST


def test_layer_extents_feed_a_window_request(tmp_path, port):
    """The extents a streaming window is bound with, taken from a parsed Llama file: nine tensors per layer in role
    order, each inside the file and disjoint, and the window's request check accepts them (no GPU involved)."""
    from emel_cpp_b200 import llama as el, window as ew
    from tests.test_gpu_gguf import CFG, model_file
    cfg = dict(CFG, n_layer=3)
    types = {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K, el.FFN_DOWN: eb.Q6_K}
    image, _plan = model_file(port, 5, types, cfg)
    path = tmp_path / "llama3.gguf"
    path.write_bytes(image)
    with gguf.File(str(path)) as f:
        layers = gguf.layer_extents(f, 3)
        assert [len(ws) for ws in layers] == [9, 9, 9]
        spans = sorted((off, off + size) for ws in layers for _tid, off, size in ws)
        assert all(a1 <= b0 for (_a0, a1), (b0, _b1) in zip(spans, spans[1:]))          # disjoint
        assert spans[0][0] >= f.data_section_offset and spans[-1][1] <= len(image)
        for l, ws in enumerate(layers):
            for (tid, off, size), stem in zip(ws, ("attn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "ffn_norm",
                                                    "ffn_gate", "ffn_up", "ffn_down")):
                t = f.find_tensor(f"blk.{l}.{stem}.weight")
                assert (tid, off, size) == (t["index"], t["file_offset"], t["data_size"])
        _offs, sizes, cap = ew.plan_layers(layers)
        err, streaming, cap_lib, total_lib = ew.check_request(len(image), layers, 2 * cap, 2, 1, slot_storage=1 << 20,
                                                              slot_storage_bytes=2 * cap)
        assert (err, streaming, cap_lib, total_lib) == (ew.OK, True, cap, sum(sizes))
        assert ew.check_request(len(image), layers, sum(sizes), 2, 1)[:2] == (ew.OK, False)     # fits: passthrough
        assert ew.check_request(len(image), layers, cap, 2, 1, slot_storage=1 << 20, slot_storage_bytes=2 * cap)[0] == ew.BUDGET_TOO_SMALL
        with pytest.raises(gguf.GgufError):
            gguf.layer_extents(f, 4)       # the file has three layers
