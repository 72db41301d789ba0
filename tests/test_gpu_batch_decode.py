"""Several sequences decoded together (emelb_llama_decode_batch / generate_batch): every sequence must get
exactly the logits and greedy ids it gets when it is decoded alone in the same session -- the products of a
column follow the one-column kernels block for block, and the attention uses the same split count -- so the
comparison is bit for bit."""
import numpy as np
import pytest

import emel_cpp_b200 as eb
from emel_cpp_b200 import llama as el
from tests import synth
from tests.test_gpu_decoder import MIXED, TINY, build_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    b = eb.Backend(0)
    yield b
    b.close()


def fill_sequences(sess, cfg, n_seq, seed):
    """Different prompts of different lengths, one per sequence -> (last prompt token, its position) per sequence."""
    rng = synth.rng(seed)
    first, pos = [], []
    for j in range(n_seq):
        prompt = rng.integers(0, cfg["n_vocab"], size=6 + 3 * (j % 5)).tolist()
        assert sess.select_sequence(j)
        assert sess.prefill(prompt[:-1], 0), sess.last_error
        first.append(prompt[-1])
        pos.append(len(prompt) - 1)
    return first, pos


@pytest.mark.parametrize("cfg,types,n_seq", [
    (TINY, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}, 5),
    (TINY, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}, 16),
    (MIXED, {"embd": eb.Q8_0, "output": eb.Q8_0, "default": eb.Q8_0, el.ATTN_K: eb.Q4_K, el.FFN_DOWN: eb.Q4_0}, 4),
    (MIXED, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K, el.FFN_DOWN: eb.Q6_K}, 16),
])
def test_each_sequence_decodes_as_it_does_alone(be, port, cfg, types, n_seq):
    sess, cpu = build_model(be, port, cfg, types, seed=21)
    cpu.close()
    n_new = 10
    try:
        assert sess.set_sequences(n_seq), sess.last_error
        first, pos = fill_sequences(sess, cfg, n_seq, seed=4)
        # alone: one sequence at a time through the one-sequence entry points
        alone_logits, alone_ids = [], []
        for j in range(n_seq):
            assert sess.select_sequence(j)
            alone_logits.append(sess.decode(first[j], pos[j], want_logits=True))
            alone_ids.append(list(sess.generate(first[j], pos[j], n_new)))
        # together: the KV rows written above are rewritten with the same values
        ids, logits = sess.decode_batch(first, pos, want_logits=True)
        for j in range(n_seq):
            assert np.array_equal(logits[j].view(np.uint32), alone_logits[j].view(np.uint32)), (j, float(np.abs(logits[j] - alone_logits[j]).max()))
            assert int(ids[j]) == alone_ids[j][0], j
        got = sess.generate_batch(first, pos, n_new)
        assert got.shape == (n_new, n_seq)
        for j in range(n_seq):
            assert list(got[:, j]) == alone_ids[j], (j, list(got[:, j]), alone_ids[j])
        # a subset of the sequences steps alone just as well
        sub = max(1, n_seq // 2)
        got = sess.generate_batch(first[:sub], pos[:sub], 4)
        for j in range(sub):
            assert list(got[:, j]) == alone_ids[j][:4], j
        assert sess.batch_launches_per_step() > 0
    finally:
        sess.close()


def test_batch_requests_are_checked(be, port):
    sess, cpu = build_model(be, port, TINY, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}, seed=2)
    cpu.close()
    try:
        assert not sess.set_sequences(0) and not sess.set_sequences(65)
        assert sess.set_sequences(3)
        assert not sess.select_sequence(3)
        with pytest.raises(eb.BackendError):
            sess.decode_batch([1, 2, 3, 4], [0, 0, 0, 0])            # more sequences than the session holds
        with pytest.raises(eb.BackendError):
            sess.decode_batch([1, TINY["n_vocab"]], [0, 0])          # token out of range
        with pytest.raises(eb.BackendError):
            sess.generate_batch([1, 2], [0, TINY["n_ctx"] - 2], 5)   # would run past the context
        be.set_attention_mode(2)
        try:
            with pytest.raises(eb.BackendError):
                sess.decode_batch([1, 2], [0, 0])
            assert sess.last_error == eb.UNSUPPORTED_OP
        finally:
            be.set_attention_mode(0)
        assert list(sess.decode_batch([1, 2], [0, 0])) == [sess.decode_batch([1], [0])[0], sess.decode_batch([2], [0])[0]]
    finally:
        sess.close()


def test_buffers_grow_with_the_sequence_count(be, port):
    """Batch buffers sized by an earlier, smaller prompt batch or sequence count are sized again."""
    sess, cpu = build_model(be, port, TINY, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}, seed=3)
    cpu.close()
    try:
        assert sess.set_prefill_batch(4)
        assert sess.prefill([5, 6, 7, 8, 9, 10], 0)          # sizes the prompt path's buffers for 4 columns
        assert sess.set_sequences(2)
        first, pos = fill_sequences(sess, TINY, 2, seed=8)
        two = sess.generate_batch(first, pos, 3)
        assert sess.set_sequences(9)                          # clears the caches: fill again, now 9 sequences
        first9, pos9 = fill_sequences(sess, TINY, 9, seed=8)
        assert first9[:2] == first and pos9[:2] == pos
        nine = sess.generate_batch(first9, pos9, 3)
        assert np.array_equal(nine[:, :2], two)
    finally:
        sess.close()
