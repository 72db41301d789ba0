"""The CPU restatement of the generator's decode loop (oracle/llama_oracle.c): the same loop
driven by the plain-C kernels and by the reference's own kernels must agree."""
import numpy as np
import pytest

from oracle import bindings as ob
from tests import synth

CFG = dict(n_layer=2, n_embd=512, n_head=8, n_head_kv=2, head_dim=64, n_ff=1024, n_vocab=320, n_ctx=48)
ROLES_K_M = lambda c: {0: (c["n_embd"], c["n_vocab"]), 2: (c["n_embd"], c["n_vocab"]),
                       4: (c["n_embd"], c["n_head"] * c["head_dim"]), 5: (c["n_embd"], c["n_head_kv"] * c["head_dim"]),
                       6: (c["n_embd"], c["n_head_kv"] * c["head_dim"]), 7: (c["n_head"] * c["head_dim"], c["n_embd"]),
                       9: (c["n_embd"], c["n_ff"]), 10: (c["n_embd"], c["n_ff"]), 11: (c["n_ff"], c["n_embd"])}


def make(port, kernels, types):
    m = ob.CpuLlama(CFG, kernels)
    shapes = ROLES_K_M(CFG)
    for layer, roles in [(-1, (0, 2))] + [(l, (4, 5, 6, 7, 9, 10, 11)) for l in range(CFG["n_layer"])]:
        for role in roles:
            k, mm = shapes[role]
            w = synth.rng(100 * (layer + 2) + role).standard_normal((mm, k), dtype=np.float32) * np.float32(1.0 if role == 0 else 0.05)
            m.bind(layer, role, port.encode_rows(types.get(role, types["default"]), w, k, mm), types.get(role, types["default"]))
    for layer, roles in [(-1, (1,))] + [(l, (3, 8)) for l in range(CFG["n_layer"])]:
        for role in roles:
            m.bind(layer, role, (1 + 0.1 * synth.rng(7 * (layer + 2) + role).standard_normal(CFG["n_embd"], dtype=np.float32)).astype(np.float32), ob.F32)
    return m


@pytest.mark.parametrize("types", [{"default": ob.Q4_K, 2: ob.Q6_K}, {"default": ob.Q8_0, 11: ob.Q4_0}])
def test_loop_with_port_kernels_equals_loop_with_reference_kernels(port, ref, types):
    a, b, c = make(port, "port", types), make(port, "ref-scalar", types), make(port, "ref-avx2", types)
    tok = 5
    for pos in range(12):
        la, lb, lc = a.decode(tok, pos), b.decode(tok, pos), c.decode(tok, pos)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))     # same kernels' arithmetic, same loop
        # The reference's AVX2 and scalar routes differ in the last bits of each row sum.  Activations
        # are re-quantized to int8 after every step, so sooner or later one rounding flips and the two
        # routes drift apart by ~1e-2 in the logits (and stay apart through the KV cache): only the
        # first positions are comparable at 1e-5, afterwards only the order of magnitude is.
        assert np.abs(lc - lb).max() <= (1e-5 if pos < 2 else 0.5)
        assert np.isfinite(la).all() and la.std() > 0
        tok = int(np.argmax(la))
    for m in (a, b, c):
        m.close()


def test_elementwise_restatements(port):
    x = synth.rng(1).standard_normal(1024, dtype=np.float32)
    w = (1 + 0.1 * synth.rng(2).standard_normal(1024, dtype=np.float32)).astype(np.float32)
    out = ob.cpu_rms_norm(x, w, 1e-5)
    ref = x * np.float32(1.0 / np.sqrt(np.float32(np.mean(x.astype(np.float64) ** 2)) + np.float32(1e-5))) * w
    np.testing.assert_allclose(out, ref, rtol=1e-6)
    v = synth.rng(3).standard_normal(2 * 64, dtype=np.float32)
    r = ob.cpu_rope(v, 2, 64, 64, 0, 5, 500000.0)
    np.testing.assert_allclose(np.hypot(r[0::2], r[1::2]), np.hypot(v[0::2], v[1::2]), rtol=1e-5)   # rotations keep pair norms
    assert np.array_equal(ob.cpu_rope(v, 2, 64, 64, 0, 0, 500000.0), v)                              # position 0: identity
    g = synth.rng(4).standard_normal(256, dtype=np.float32)
    np.testing.assert_allclose(ob.cpu_swiglu(g, g), g / (1 + np.exp(-g)) * g, rtol=1e-6)
