"""Parity at the shapes the benchmark runs, not just at small ones.

* configuration 4: the tcgen05 Q4_K product with 2048 token columns, K = 4096 -> 14336 rows (up / gate) and
  K = 14336 -> 4096 rows (down: 56 super-blocks per row, many turns of every pipeline ring and barrier phase);
* configuration 2 at 512 tokens: the Q8_0 many-column kernel at 14336 x 4096.
  The GPU computes the whole product; the reference's AVX2 route (8 lanes) computes a sample of the token
  columns — every output element is independent of the other columns — and those are compared bit for bit
  over ALL rows.
* configurations 3/5: one full-width layer of the 8B shape (hidden 4096, 32/8 heads of 128, FFN 14336) decoded
  for a few tokens against the CPU loop over the reference's kernels in the reference-order attention mode,
  logits bit for bit.
"""
import numpy as np
import pytest

import emel_cpp_b200 as eb
from emel_cpp_b200 import llama as el
from oracle import bindings as ob
from tests import synth
from tests.test_gpu_decoder import build_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    b = eb.Backend(0)
    yield b
    b.close()


def sampled_columns(n, count=24):
    """first, last and spread token columns: the edges of the 128-token tiles and a stride through the middle"""
    cols = set(range(4)) | set(range(n - 4, n)) | {127, 128, 129, n // 2 - 1, n // 2}
    step = max(1, n // (count - len(cols)))
    cols |= set(range(0, n, step))
    return np.array(sorted(c for c in cols if 0 <= c < n), np.int64)


_NEXT_ID = [52000]


def product_on_sample(be, checker, t, w, k, m, x, n):
    """w is made resident first (the view then carries its host address, as the reference's tensor records do):
    the staging area is for the activations and the result"""
    tid = _NEXT_ID[0]
    _NEXT_ID[0] += 1
    be.upload(tid, w, tensor_type=t)
    y = np.zeros((m, n), np.float32)
    try:
        assert be.mul_mat(eb.mul_mat_op(w, t, k, m, x, n, y)), be.last_error
        assert be.sync()                   # a bounded wait that ran out would surface here
    finally:
        be.evict(tid)                      # the host span must not outlive the array (its address may be reused)
    cols = sampled_columns(n)
    xs = np.ascontiguousarray(x[:, cols])
    want = np.zeros((m, cols.size), np.float32)
    kw = {"route": "avx2", "lanes": 8} if isinstance(checker, ob.Ref) else {}
    assert checker.mul_mat(ob.mul_mat_op(w, t, k, m, xs, cols.size, want), **kw)
    got = np.ascontiguousarray(y[:, cols])
    assert ob.rel_l2(got, want) <= 1e-5
    if isinstance(checker, ob.Ref) or t in (eb.Q8_0, eb.Q4_0):
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), float(np.abs(got - want).max())
    assert np.isfinite(y).all() and y.std() > 0
    return y


@pytest.mark.parametrize("k,m", [(4096, 14336), (14336, 4096)])
def test_config4_q4_k_2048_tokens(be, checker, k, m):
    n = 2048
    w = synth.random_blocks(eb.Q4_K, 900 + k, m, k)         # arbitrary scale / min / quant codes
    x = synth.activations_f32(901 + k, k, n)
    y = product_on_sample(be, checker, eb.Q4_K, w, k, m, x, n)
    # and the same bits as the one-column route for a few columns (different kernel family)
    for c in (0, 1000, n - 1):
        y1 = np.zeros((m, 1), np.float32)
        assert be.mul_mat(eb.mul_mat_op(w, eb.Q4_K, k, m, np.ascontiguousarray(x[:, c:c + 1]), 1, y1)), be.last_error
        assert np.array_equal(y1[:, 0].view(np.uint32), y[:, c].view(np.uint32)), c
    assert be.sync()


def test_config2_q8_0_512_tokens(be, checker, port):
    k, m, n = 4096, 14336, 512
    w = synth.encoded_weights(port, eb.Q8_0, 3, m, k)
    x = synth.activations_f32(4, k, n)
    product_on_sample(be, checker, eb.Q8_0, w, k, m, x, n)


def test_one_layer_of_the_8b_shape_matches_the_reference_loop(port):
    cfg = dict(n_layer=1, n_embd=4096, n_head=32, n_head_kv=8, head_dim=128, n_ff=14336, n_vocab=1024, n_ctx=32)
    be = eb.Backend(0)
    sess, cpu = build_model(be, port, cfg, {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}, seed=17)
    be.set_attention_mode(2 if ob.ref() is not None else 1)   # reference order of the route the CPU loop runs
    try:
        prompt = synth.rng(19).integers(0, cfg["n_vocab"], size=6).tolist()
        for pos, tok in enumerate(prompt[:-1]):
            cpu.decode(tok, pos, want_logits=False)
        assert sess.prefill(prompt[:-1], 0), sess.last_error
        tok_gpu = tok_cpu = prompt[-1]
        for i in range(4):
            pos = len(prompt) - 1 + i
            lg, lc = sess.decode(tok_gpu, pos, want_logits=True), cpu.decode(tok_cpu, pos)
            assert float(np.abs(lg - lc).max()) <= 1e-3, i
            if ob.ref() is not None:
                assert np.array_equal(lg.view(np.uint32), lc.view(np.uint32)), (i, float(np.abs(lg - lc).max()))
            tok_gpu, tok_cpu = int(np.argmax(lg)), int(np.argmax(lc))
            assert tok_gpu == tok_cpu
    finally:
        be.set_attention_mode(0)
        sess.close()
        cpu.close()
        be.close()
