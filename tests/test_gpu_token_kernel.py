"""One decode token as one persistent kernel (emelb_llama_set_step_mode 1) against the chain of
per-operation launches (mode 0): same session, same tokens, same positions, logits compared bit
for bit.  The chain itself is held to the reference's CPU loop in tests/test_gpu_decoder.py, and
both routes are built from the same arithmetic (Q4_K products in the x86 route's order, the
split-KV attention bodies), so nothing but the scheduling differs between them.

Shapes: head size 128, Q4_K layer matrices, a feed-forward width of three 2048-weight chunks so
that the down projection completes its rows through the block-value table (two chunk pairs, the
second one half full), several query-head quads per KV head, a prompt long enough for several
KV ranges per head.
"""
import numpy as np
import pytest

import emel_cpp_b200 as eb
from emel_cpp_b200 import llama as el
from oracle import bindings as ob
from tests import synth
from tests.test_gpu_decoder import build_model

pytestmark = pytest.mark.gpu

SHAPES = [
    dict(n_layer=3, n_embd=2048, n_head=16, n_head_kv=4, head_dim=128, n_ff=6144, n_vocab=1024, n_ctx=192),
    dict(n_layer=2, n_embd=4096, n_head=32, n_head_kv=4, head_dim=128, n_ff=14336, n_vocab=512, n_ctx=96),
]
ALL_Q4K = {"embd": eb.Q4_K, "output": eb.Q6_K, "default": eb.Q4_K}


@pytest.mark.parametrize("cfg", SHAPES)
def test_one_kernel_step_equals_launch_chain(port, cfg):
    be = eb.Backend(0)
    sess, cpu = build_model(be, port, cfg, ALL_Q4K, seed=11)
    cpu.close()
    try:
        prompt = synth.rng(21).integers(0, cfg["n_vocab"], size=cfg["n_ctx"] // 2).tolist()
        assert sess.prefill(prompt[:-1], 0), sess.last_error
        pos0, n_new = len(prompt) - 1, 12

        def walk(mode):
            assert sess.set_step_mode(mode)
            out, tok = [], prompt[-1]
            for i in range(n_new):
                lg = sess.decode(tok, pos0 + i, want_logits=True)
                out.append(lg)
                tok = int(np.argmax(lg))
            return out, sess.launches_per_token()

        chain, _ = walk(0)
        fused, _ = walk(1)
        for i, (a, b) in enumerate(zip(chain, fused)):
            assert np.isfinite(a).all() and a.std() > 0
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), (i, float(np.abs(a - b).max()))
        # the greedy routes (fused argmax head, device-fed loop) agree as well, and the fused step is a
        # handful of launches instead of seven per layer
        assert sess.set_step_mode(0)
        ids_chain = sess.generate(prompt[-1], pos0, n_new).tolist()
        n_chain = sess.launches_per_token()
        assert sess.set_step_mode(1)
        ids_fused = sess.generate(prompt[-1], pos0, n_new).tolist()
        n_fused = sess.launches_per_token()
        assert ids_fused == ids_chain == [int(np.argmax(l)) for l in chain]
        assert n_fused < n_chain and n_fused <= 8, (n_fused, n_chain)
        assert be.sync()
    finally:
        sess.close()
        be.close()


def test_one_kernel_step_stays_out_of_the_way(port):
    """Sessions the persistent kernel does not take (head size 64 here) run the chain in either mode."""
    cfg = dict(n_layer=2, n_embd=2048, n_head=8, n_head_kv=2, head_dim=64, n_ff=4096, n_vocab=512, n_ctx=64)
    be = eb.Backend(0)
    sess, cpu = build_model(be, port, cfg, ALL_Q4K, seed=13)
    cpu.close()
    try:
        assert sess.prefill([1, 2, 3], 0)
        a = sess.decode(4, 3, want_logits=True)
        assert sess.set_step_mode(1)
        b = sess.decode(4, 3, want_logits=True)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        assert not sess.set_step_mode(2) and sess.last_error == eb.INVALID_REQUEST
    finally:
        sess.close()
        be.close()
