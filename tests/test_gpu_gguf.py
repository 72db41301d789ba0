"""GGUF file -> HBM -> decode: a Llama model written as a GGUF file, mapped and
uploaded by the library, must decode exactly as the reference's loop does on the
same bytes (bars: greedy ids identical, max |delta logit| <= 1e-3; met bit for bit
on the AVX2 route with reference-order attention)."""
import numpy as np
import pytest

import emel_cpp_b200 as eb
from emel_cpp_b200 import gguf, llama as el
from oracle import bindings as ob
from emel_cpp_b200 import gguf_image as gi
from tests import synth

pytestmark = pytest.mark.gpu

CFG = dict(n_layer=2, n_embd=512, n_head=8, n_head_kv=2, head_dim=64, n_ff=1024, n_vocab=384, n_ctx=64)
ROLE_NAMES = {el.ATTN_Q: "attn_q", el.ATTN_K: "attn_k", el.ATTN_V: "attn_v", el.ATTN_OUT: "attn_output",
              el.FFN_GATE: "ffn_gate", el.FFN_UP: "ffn_up", el.FFN_DOWN: "ffn_down"}
NORM_NAMES = {el.ATTN_NORM: "attn_norm", el.FFN_NORM: "ffn_norm"}


def model_file(port, seed, types, CFG=CFG):
    shapes = el.matrix_shapes(el.config(**CFG))
    matrices, norms, plan = {}, {}, []

    def matrix(name, layer, role, t, scale):
        k, m = shapes[role]
        w = synth.rng(seed + 31 * (layer + 2) + role).standard_normal((m, k), dtype=np.float32) * np.float32(scale)
        matrices[name] = (k, m, t, port.encode_rows(t, w, k, m))
        plan.append((name, layer, role, t))

    def norm(name, layer, role):
        norms[name] = (1.0 + 0.1 * synth.rng(seed + 977 * (layer + 2) + role).standard_normal(CFG["n_embd"])).astype(np.float32)
        plan.append((name, layer, role, eb.F32))

    matrix("token_embd.weight", -1, el.TOKEN_EMBD, types["embd"], 1.0)
    norm("output_norm.weight", -1, el.OUTPUT_NORM)
    matrix("output.weight", -1, el.OUTPUT, types["output"], 0.05)
    for l in range(CFG["n_layer"]):
        for role, stem in NORM_NAMES.items():
            norm(f"blk.{l}.{stem}.weight", l, role)
        for role, stem in ROLE_NAMES.items():
            matrix(f"blk.{l}.{stem}.weight", l, role, types.get(role, types["default"]), 0.05)
    return gi.llama_file(CFG, matrices, norms, alignment=64), plan


@pytest.fixture(scope="module")
def be():
    b = eb.Backend(0)
    yield b
    b.close()


@pytest.mark.parametrize("types", [
    {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K},
    {"embd": eb.Q8_0, "output": eb.Q8_0, "default": eb.Q8_0, el.FFN_DOWN: eb.Q4_0, el.ATTN_V: eb.Q6_K},
])
def test_decode_from_gguf_file_matches_reference_loop(be, port, tmp_path, types):
    image, plan = model_file(port, 21, types)
    path = tmp_path / "tiny-llama.gguf"
    path.write_bytes(image)
    kernels = "ref-avx2" if ob.ref() is not None else "port"
    cpu = ob.CpuLlama(CFG, kernels)
    host = np.frombuffer(image, np.uint8)
    with gguf.File(str(path)) as f:
        assert f.alignment == 64 and f.get("llama.block_count") == CFG["n_layer"]
        cfg = gguf.llama_config(f)
        assert (cfg.n_embd, cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.n_ff, cfg.n_vocab, cfg.n_ctx) == \
            (512, 8, 2, 64, 1024, 384, 64) and cfg.rope_freq_base == 500000.0
        # the CPU loop reads the same bytes from an in-memory copy of the file
        for name, layer, role, t in plan:
            rec = f.find_tensor(name)
            assert rec["type"] == t
            cpu.bind(layer, role, host[rec["file_offset"]:rec["file_offset"] + rec["data_size"]], t)
        sess = gguf.load_llama(be, f, first_tensor_id=5000 + 100 * len(types))
        be.set_attention_mode(2 if ob.ref() is not None else 1)
        try:
            prompt = synth.rng(4).integers(0, CFG["n_vocab"], size=10).tolist()
            for pos, tok in enumerate(prompt[:-1]):
                cpu.decode(tok, pos, want_logits=False)
            assert sess.prefill(prompt[:-1], 0), sess.last_error
            tok_gpu = tok_cpu = prompt[-1]
            worst = 0.0
            for i in range(16):
                pos = len(prompt) - 1 + i
                lg, lc = sess.decode(tok_gpu, pos, want_logits=True), cpu.decode(tok_cpu, pos)
                worst = max(worst, float(np.abs(lg - lc).max()))
                tok_gpu, tok_cpu = int(np.argmax(lg)), int(np.argmax(lc))
                assert tok_gpu == tok_cpu and worst <= 1e-3, (i, worst)
            if ob.ref() is not None:
                assert worst == 0.0, worst
            # every tensor is resident under its id, keyed by its address in the mapping
            rec = f.find_tensor("blk.1.ffn_down.weight")
            st = be.state(5000 + 100 * len(types) + rec["index"])
            assert eb.LIFECYCLE[st.lifecycle_state] == "resident" and st.buffer_bytes == rec["data_size"]
            assert st.host == rec["data"] and st.tensor_type == rec["type"]
        finally:
            be.set_attention_mode(0)
            sess.close()
            cpu.close()
            for t in f.tensors():
                be.evict(5000 + 100 * len(types) + t["index"])


def test_layers_streamed_from_a_gguf_file(be, port, tmp_path):
    """The same file decoded with its layers resident and with its layers left in the mapping and streamed through
    a two-slot window: identical logits and ids."""
    from emel_cpp_b200 import window as ew
    cfg4 = dict(CFG, n_layer=4)
    types = {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K, el.FFN_DOWN: eb.Q6_K}
    image, _plan = model_file(port, 33, types, cfg4)
    path = tmp_path / "tiny-llama-4.gguf"
    path.write_bytes(image)
    prompt = synth.rng(6).integers(0, CFG["n_vocab"], size=12).tolist()
    with gguf.File(str(path)) as f:
        resident = gguf.load_llama(be, f, first_tensor_id=7000)
        try:
            assert resident.prefill(prompt[:-1], 0)
            want_logits = resident.decode(prompt[-1], len(prompt) - 1, want_logits=True)
            want_ids = list(resident.generate(prompt[-1], len(prompt) - 1, 12))
        finally:
            resident.close()
            for t in f.tensors():
                be.evict(7000 + t["index"])
        layers = gguf.layer_extents(f, 4)
        assert [len(w) for w in layers] == [9] * 4
        _offs, sizes, cap = ew.plan_layers(layers)
        # a budget that holds every layer: nothing is streamed, the plain loader's session comes back
        sess, win = gguf.load_llama_streamed(be, f, sum(sizes), 2, 1, first_tensor_id=7000)
        try:
            assert win is None and list(sess.generate(prompt[-1], len(prompt) - 1, 1)) is not None
        finally:
            sess.close()
            for t in f.tensors():
                be.evict(7000 + t["index"])
        for staged in (False, True):
            sess, win = gguf.load_llama_streamed(be, f, 2 * cap, 2, 1, first_tensor_id=7200, staged_only=staged)
            try:
                assert win is not None and win.bound["streaming_active"] and win.bound["window_slots"] == 2
                assert sess.prefill(prompt[:-1], 0), sess.last_error
                got = sess.decode(prompt[-1], len(prompt) - 1, want_logits=True)
                assert np.array_equal(got.view(np.uint32), want_logits.view(np.uint32))
                assert list(sess.generate(prompt[-1], len(prompt) - 1, 12)) == want_ids
                # only the three model-level tensors are resident
                assert eb.LIFECYCLE[be.state(7200 + f.find_tensor("blk.0.attn_q.weight")["index"]).lifecycle_state] != "resident"
                assert eb.LIFECYCLE[be.state(7200 + f.find_tensor("output.weight")["index"]).lifecycle_state] == "resident"
                assert win.stats()["loads_failed"] == 0
            finally:
                sess.close()
                win.close()
                for t in f.tensors():
                    be.evict(7200 + t["index"])
        # a window that cannot hold two layers
        with pytest.raises(gguf.GgufError):
            gguf.load_llama_streamed(be, f, cap, 2, 1, first_tensor_id=7400)


def test_upload_rows_feeds_a_row_sharded_product(be, port, tmp_path):
    """One rank's row interval of a matrix in the file, uploaded alone, gives that interval of the product."""
    k, m = 1024, 24
    w = synth.rng(2).standard_normal((m, k), dtype=np.float32) * np.float32(0.05)
    blocks = port.encode_rows(eb.Q4_K, w, k, m)
    image = gi.build([gi.kv("general.alignment", gi.T_UINT32, 32)], [("pad.f32", (3,), 0, b"\1" * 12),
                                                                     ("w", (k, m), eb.Q4_K, blocks.tobytes())], 32)
    path = tmp_path / "w.gguf"
    path.write_bytes(image)
    x = synth.rng(3).standard_normal(k, dtype=np.float32)
    with gguf.File(str(path)) as f:
        rec = f.find_tensor("w")
        f.upload(be, rec["index"], 7001)
        full = np.zeros(m, np.float32)
        assert be.mul_mat(eb.mul_mat_op(rec["data"], eb.Q4_K, k, m, x, 1, full)), be.last_error
        be.evict(7001)
        host, _dev = f.upload_rows(be, rec["index"], 7002, 8, 8)
        assert host == rec["data"] + 8 * eb.row_bytes(eb.Q4_K, k)
        part = np.zeros(8, np.float32)
        assert be.mul_mat(eb.mul_mat_op(host, eb.Q4_K, k, 8, x, 1, part)), be.last_error
        assert np.array_equal(part, full[8:16])
        with pytest.raises(gguf.GgufError) as e:
            f.upload_rows(be, rec["index"], 7003, 20, 8)       # past the last row
        assert e.value.err == gguf.INVALID_REQUEST
        with pytest.raises(gguf.GgufError):
            f.upload_rows(be, f.find_tensor("pad.f32")["index"], 7003, 0, 1)   # one dimension: no rows to slice
        be.evict(7002)
        # the whole file at once is all or nothing: id 7101 (tensor 1) is taken, so tensor 0 must not stay behind
        f.upload(be, rec["index"], 7101)
        with pytest.raises(gguf.GgufError) as e:
            f.upload_all(be, 7100)
        assert e.value.err == gguf.INVALID_REQUEST
        assert eb.LIFECYCLE[be.state(7100).lifecycle_state] == "unbound"
        be.evict(7101)
        f.upload_all(be, 7100)
        for t in f.tensors():
            st = be.state(7100 + t["index"])
            got = np.empty(t["data_size"], np.uint8)
            assert be.to_host(got, st.buffer, t["data_size"])
            assert got.tobytes() == image[t["file_offset"]:t["file_offset"] + t["data_size"]]
            be.evict(7100 + t["index"])


def test_large_tensor_goes_through_the_staging_ring_unchanged(be, tmp_path):
    """Spans above the direct-copy threshold are cut into chunks filled by several threads (pread from the
    file, or memcpy from a host array): the bytes in HBM must be the file's, whatever the route."""
    import os
    rng = synth.rng(8)
    sizes = [(1 << 20) + 32, 37 * (1 << 20) + 96, 5 * (1 << 20)]      # one direct-sized, two chunked (ragged ends)
    blobs = [rng.integers(0, 256, size=n, dtype=np.uint8) for n in sizes]
    image = gi.build([], [(f"t{i}", (len(b),), 24, b.tobytes()) for i, b in enumerate(blobs)], 32)
    path = tmp_path / "big.gguf"
    path.write_bytes(image)
    for mode in ("ring", "plain", "register"):
        assert be.set_upload_route(mode)
        try:
            with gguf.File(str(path)) as f:
                f.upload_all(be, 7200)
                for i, b in enumerate(blobs):
                    st = be.state(7200 + i)
                    got = np.empty(len(b), np.uint8)
                    assert be.to_host(got, st.buffer, len(b)) and np.array_equal(got, b), (mode, i)
                    be.evict(7200 + i)
        finally:
            assert be.set_upload_route("ring")
    # a plain host array (no file behind it) takes the memcpy-fed ring
    be.upload(7300, blobs[1], tensor_type=24)
    got = np.empty(len(blobs[1]), np.uint8)
    assert be.to_host(got, be.state(7300).buffer, len(got)) and np.array_equal(got, blobs[1])
    be.evict(7300)
