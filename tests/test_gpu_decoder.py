"""The device-resident decode loop against the CPU restatement of the reference
generator's loop (oracle/llama_oracle.c) driving the reference's own kernels.

Bars (north star): greedy tokens identical, max |delta logit| <= 1e-3.  The decode
loop re-quantizes activations to int8 after every step, so it is chaotic at that
scale: the reference's own scalar and AVX2 routes drift apart by > 1e-2 within a few
tokens.  The bound is therefore met the only way it can be, by following one route
(the x86 AVX2 one) rounding for rounding: with the reference-order attention the
logits are compared bit for bit.  The split-KV attention is checked beside it within
the attention tolerance.
"""
import numpy as np
import pytest

import emel_cpp_b200 as eb
from emel_cpp_b200 import llama as el
from oracle import bindings as ob
from tests import synth

pytestmark = pytest.mark.gpu

_NEXT_TENSOR_ID = [1000]     # residency ids stay unique across the models built in this module

TINY = dict(n_layer=3, n_embd=512, n_head=8, n_head_kv=2, head_dim=64, n_ff=2048, n_vocab=640, n_ctx=96)
MIXED = dict(n_layer=2, n_embd=2048, n_head=16, n_head_kv=4, head_dim=128, n_ff=4096, n_vocab=1000, n_ctx=64)


def build_model(be, port, cfg, types, seed):
    """Encodes N(0, 0.02) weights on the host, uploads them, binds both decoders."""
    c = el.config(**cfg)
    sess = el.Session(be, c)
    kernels = "ref-avx2" if ob.ref() is not None else "port"
    cpu = ob.CpuLlama(cfg, kernels)
    shapes = el.matrix_shapes(c)
    tid = _NEXT_TENSOR_ID

    def put_matrix(layer, role, t, scale=0.02):
        k, m = shapes[role]
        w = synth.rng(seed + 31 * (layer + 2) + role).standard_normal((m, k), dtype=np.float32) * np.float32(scale)
        blocks = port.encode_rows(t, w, k, m)
        be.upload(tid[0], blocks, tensor_type=t)
        tid[0] += 1
        assert sess.bind_matrix(layer, role, blocks, t), sess.last_error     # bound by host address of the resident span
        cpu.bind(layer, role, blocks, t)

    def put_norm(layer, role):
        w = (1.0 + 0.1 * synth.rng(seed + 977 * (layer + 2) + role).standard_normal(cfg["n_embd"], dtype=np.float32)).astype(np.float32)
        be.upload(tid[0], w, tensor_type=eb.F32)
        tid[0] += 1
        assert sess.bind_norm(layer, role, w), sess.last_error
        cpu.bind(layer, role, w, eb.F32)

    put_matrix(-1, el.TOKEN_EMBD, types["embd"], scale=1.0)
    put_norm(-1, el.OUTPUT_NORM)
    put_matrix(-1, el.OUTPUT, types["output"], scale=0.05)
    for l in range(cfg["n_layer"]):
        put_norm(l, el.ATTN_NORM)
        put_norm(l, el.FFN_NORM)
        for role in (el.ATTN_Q, el.ATTN_K, el.ATTN_V, el.ATTN_OUT, el.FFN_GATE, el.FFN_UP, el.FFN_DOWN):
            put_matrix(l, role, types.get(role, types["default"]), scale=0.05)
    return sess, cpu


@pytest.fixture(scope="module")
def be():
    b = eb.Backend(0)
    yield b
    b.close()


@pytest.mark.parametrize("cfg,types", [
    (TINY, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}),
    (MIXED, {"embd": eb.Q8_0, "output": eb.Q8_0, "default": eb.Q8_0, el.ATTN_K: eb.Q4_K, el.FFN_DOWN: eb.Q4_0}),
    # Q6_K value and down projections beside Q4_K: Q/K and V run as two fused launches, each with its share of the
    # RoPE / KV-store epilogue; and a Q6_K query projection (three runs of one matrix each)
    (MIXED, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K, el.ATTN_V: eb.Q6_K, el.FFN_DOWN: eb.Q6_K}),
    (MIXED, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K, el.ATTN_K: eb.Q6_K}),
])
def test_greedy_decode_matches_reference_loop(be, port, cfg, types):
    sess, cpu = build_model(be, port, cfg, types, seed=5)
    prompt = synth.rng(9).integers(0, cfg["n_vocab"], size=20).tolist()
    n_new = 24
    be.set_attention_mode(2 if ob.ref() is not None else 1)   # reference order of the route the CPU loop runs
    try:
        # prompt: the CPU loop skips logits except at the last prompt token
        for pos, tok in enumerate(prompt[:-1]):
            cpu.decode(tok, pos, want_logits=False)
        assert sess.prefill(prompt[:-1], 0), sess.last_error
        tok_gpu = tok_cpu = prompt[-1]
        worst = 0.0
        for i in range(n_new):
            pos = len(prompt) - 1 + i
            lg = sess.decode(tok_gpu, pos, want_logits=True)
            lc = cpu.decode(tok_cpu, pos)
            worst = max(worst, float(np.abs(lg - lc).max()))
            tok_gpu, tok_cpu = int(np.argmax(lg)), int(np.argmax(lc))
            assert tok_gpu == tok_cpu, (i, worst)
            assert worst <= 1e-3, (i, worst)
        if ob.ref() is not None:
            assert worst == 0.0, worst       # every rounding of the AVX2 route reproduced
    finally:
        be.set_attention_mode(0)
        sess.close()
        cpu.close()


def test_argmax_route_generate_and_split_kv_attention(be, port):
    """The fused-argmax step and the device-fed generate loop give the same ids as argmax over
    the logits route; the split-KV attention changes logits only within the attention tolerance."""
    sess, cpu = build_model(be, port, TINY, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}, seed=7)
    try:
        prompt = synth.rng(3).integers(0, TINY["n_vocab"], size=12).tolist()
        assert sess.prefill(prompt[:-1], 0)
        ids_logits, tok = [], prompt[-1]
        for i in range(16):
            lg = sess.decode(tok, len(prompt) - 1 + i, want_logits=True)
            tok = int(np.argmax(lg))
            ids_logits.append(tok)
        # same sequence through the argmax route (KV rows are rewritten with identical values)
        ids_argmax, tok = [], prompt[-1]
        for i in range(16):
            tok = sess.decode(tok, len(prompt) - 1 + i)
            ids_argmax.append(tok)
        assert ids_argmax == ids_logits
        assert sess.generate(prompt[-1], len(prompt) - 1, 16).tolist() == ids_logits
        assert sess.launches_per_token() > 0
        # CPU reference (sequential f16-accumulator attention) vs split-KV f32 attention
        for pos, t in enumerate(prompt[:-1]):
            cpu.decode(t, pos, want_logits=False)
        lc = cpu.decode(prompt[-1], len(prompt) - 1)
        lg = sess.decode(prompt[-1], len(prompt) - 1, want_logits=True)
        # the two attention numerics differ by ~1e-3 per call and the loop amplifies differences
        # (int8 re-quantization), so only the overall agreement is checked here
        assert np.isfinite(lg).all()
        assert float(np.dot(lg, lc) / (np.linalg.norm(lg) * np.linalg.norm(lc))) > 0.995
    finally:
        sess.close()
        cpu.close()


def test_decoder_rejects_bad_requests(port):
    # own context: the shared one still maps host spans of arrays earlier tests uploaded and freed, and a
    # new array may be handed one of those addresses
    be = eb.Backend(0)
    c = el.config(**TINY)
    sess = el.Session(be, c)
    try:
        with pytest.raises(eb.BackendError):
            sess.decode(0, 0)                                  # nothing bound
        w = np.zeros(10, np.uint8)
        assert not sess.bind_matrix(0, el.ATTN_Q, w, eb.Q4_K)  # not resident, not a device pointer
        assert not sess.bind_matrix(7, el.ATTN_Q, w, eb.Q4_K)  # no such layer
    finally:
        sess.close()
    bad = dict(TINY, n_embd=500)
    with pytest.raises(eb.BackendError):
        el.Session(be, el.config(**bad))
    be.close()


def _prompt_then_logits(be, sess, prompt, pieces, mode=0):
    """Prefill `prompt[:-1]` in the given pieces (attention mode `mode`), then the logits of the last token
    (always with the split-KV attention, so only the prompt path differs between calls)."""
    be.set_attention_mode(mode)
    pos = 0
    for n in pieces:
        assert sess.prefill(prompt[pos:pos + n], pos), sess.last_error
        pos += n
    be.set_attention_mode(0)
    assert pos == len(prompt) - 1
    return sess.decode(prompt[-1], pos, want_logits=True)


def _rel(a, b):
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


@pytest.mark.parametrize("cfg,types", [
    (TINY, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}),
    (MIXED, {"embd": eb.Q8_0, "output": eb.Q8_0, "default": eb.Q8_0, el.ATTN_K: eb.Q4_K, el.FFN_DOWN: eb.Q4_0}),
])
def test_batched_prompt_one_layer_is_bit_identical(be, port, cfg, types):
    """With one layer the logits after a prompt depend on the prompt only through the layer's K and V rows:
    embedding, norm, quantization, the matrix products (tensor-core kernel for batches of 32 and more Q4_K
    columns, multi-column mat-vec kernels below), RoPE and the f16 store.  Those are the same arithmetic per
    token in the batched path, so the logits must be bit-identical to a token-by-token walk."""
    cfg = dict(cfg, n_layer=1, n_ctx=192)
    sess, cpu = build_model(be, port, cfg, types, seed=13)
    cpu.close()
    try:
        prompt = synth.rng(17).integers(0, cfg["n_vocab"], size=151).tolist()
        assert sess.set_prefill_batch(0)
        l0 = be.diagnostics()["kernel_launches"]
        base = _prompt_then_logits(be, sess, prompt, [150])
        launches_token = be.diagnostics()["kernel_launches"] - l0
        assert sess.set_prefill_batch(2048)
        for batch, pieces in ((None, [150]), ("64", [150]), (None, [1, 2, 33, 100, 14]), ("40", [70, 80])):
            if batch:
                assert sess.set_prefill_batch(int(batch))
            # scrub the cache rows first so that stale rows of the previous walk cannot stand in for missing ones
            junk = synth.rng(5).integers(0, cfg["n_vocab"], size=150).tolist()
            assert sess.prefill(junk, 0)
            l0 = be.diagnostics()["kernel_launches"]
            got = _prompt_then_logits(be, sess, prompt, pieces)
            launches = be.diagnostics()["kernel_launches"] - l0
            assert sess.set_prefill_batch(2048)
            assert np.array_equal(got.view(np.uint32), base.view(np.uint32)), (batch, pieces, float(np.abs(got - base).max()))
            assert launches < launches_token / 3
    finally:
        sess.close()


@pytest.mark.parametrize("cfg,types", [
    (TINY, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}),
    (MIXED, {"embd": eb.Q8_0, "output": eb.Q8_0, "default": eb.Q8_0, el.ATTN_K: eb.Q4_K, el.FFN_DOWN: eb.Q4_0}),
])
def test_batched_prompt_many_layers_within_attention_noise(be, port, cfg, types):
    """With more layers the prompt's attention outputs feed the next layer's int8 quantizers, where a
    difference in the last bits flips roundings (the decoder is chaotic at that scale: the reference's own
    routes drift apart the same way).  The batch attention kernel is held to 2e-5 of the exact softmax on its
    own (test_gpu_attention_batch.py); here the batched walk must stay closer to the token-by-token walk
    than the reference-order attention (f16 accumulators) does."""
    cfg = dict(cfg, n_ctx=192)
    sess, cpu = build_model(be, port, cfg, types, seed=13)
    cpu.close()
    try:
        prompt = synth.rng(17).integers(0, cfg["n_vocab"], size=151).tolist()
        assert sess.set_prefill_batch(0)
        base = _prompt_then_logits(be, sess, prompt, [150])
        ref_order = _prompt_then_logits(be, sess, prompt, [150], mode=2)
        assert sess.set_prefill_batch(2048)
        yard = _rel(ref_order, base)
        for batch, pieces in ((None, [150]), ("64", [150]), (None, [1, 2, 33, 100, 14])):
            if batch:
                assert sess.set_prefill_batch(int(batch))
            got = _prompt_then_logits(be, sess, prompt, pieces)
            assert sess.set_prefill_batch(2048)
            d = _rel(got, base)
            print(pieces, "batched vs token-by-token %.2e, reference-order vs token-by-token %.2e" % (d, yard))
            assert np.isfinite(got).all() and d <= yard and d <= 5e-2, (pieces, d, yard)
    finally:
        sess.close()


def test_batched_prompt_fills_the_context_to_the_last_row(be, port):
    """A prompt that ends on the last but one cache row, batches of 2 and of 61 tokens, and the decode step
    on the last row: bit-identical to the token-by-token walk (one layer), and requests past the context
    are refused before anything runs."""
    cfg = dict(TINY, n_layer=1, n_ctx=64)
    sess, cpu = build_model(be, port, cfg, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}, seed=29)
    cpu.close()
    try:
        prompt = synth.rng(31).integers(0, cfg["n_vocab"], size=64).tolist()
        assert sess.set_prefill_batch(0)
        base = _prompt_then_logits(be, sess, prompt, [63])
        assert sess.set_prefill_batch(2048)
        assert sess.prefill(synth.rng(5).integers(0, cfg["n_vocab"], size=63).tolist(), 0)    # scrub
        got = _prompt_then_logits(be, sess, prompt, [2, 61])
        assert np.array_equal(got.view(np.uint32), base.view(np.uint32))
        assert not sess.prefill(prompt[:2], 63) and sess.last_error == eb.INVALID_REQUEST       # would pass the last row
        assert not sess.prefill([cfg["n_vocab"]], 0) and sess.last_error == eb.INVALID_REQUEST  # no such token
        again = sess.decode(prompt[-1], 63, want_logits=True)                                    # the session still works
        assert np.array_equal(again.view(np.uint32), base.view(np.uint32))
    finally:
        sess.close()
