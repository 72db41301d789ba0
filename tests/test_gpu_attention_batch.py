"""Attention over a batch of prompt tokens (emelb_flash_attn_batch) against an exact
f64 softmax over the same f16 cache.  Tolerance 2e-5 relative to the largest output,
the bar the one-token split-KV kernel is held to."""
import numpy as np
import pytest

import emel_cpp_b200 as eb
from tests import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    b = eb.Backend(0)
    yield b
    b.close()


def exact(q, k, v, heads, kv_heads, pos0, scale):
    """q: [heads*D, B] f32 (token fastest); k, v: [kv_heads, capacity, D] f16 -> [heads*D, B] f64"""
    d = k.shape[2]
    b = q.shape[1]
    rep = heads // kv_heads
    q16 = q.astype(np.float16).astype(np.float64).reshape(heads, d, b)
    out = np.zeros((heads, d, b))
    for h in range(heads):
        kh = h // rep
        for j in range(b):
            t = pos0 + j + 1
            s = k[kh, :t].astype(np.float64) @ q16[h, :, j] * scale
            p = np.exp(s - s.max())
            out[h, :, j] = (p / p.sum()) @ v[kh, :t].astype(np.float64)
    return out.reshape(heads * d, b)


@pytest.mark.parametrize("d,heads,kv_heads,batch,pos0", [
    (64, 8, 2, 1, 0), (64, 8, 2, 11, 0), (64, 8, 2, 40, 0), (64, 8, 2, 150, 0), (64, 8, 2, 33, 37),
    (128, 16, 4, 40, 0), (128, 16, 4, 150, 5), (128, 32, 8, 70, 130), (128, 64, 8, 24, 100),
    (128, 4, 4, 65, 64), (64, 2, 1, 130, 1),
])
def test_batch_attention_matches_exact_softmax(be, d, heads, kv_heads, batch, pos0):
    rng = synth.rng(1000 * d + heads + batch + pos0)
    capacity = pos0 + batch + 9
    q = rng.standard_normal((heads * d, batch), dtype=np.float32) * np.float32(1.5)
    k = rng.standard_normal((kv_heads, capacity, d), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((kv_heads, capacity, d), dtype=np.float32).astype(np.float16)
    k[:, pos0 + batch:] = np.float16(np.nan)       # rows past the batch hold no data and must not be used
    v[:, pos0 + batch:] = np.float16(np.nan)
    scale = 1.0 / np.sqrt(d)
    bufs = [be.alloc(a.nbytes) for a in (q, k, v, q)]
    try:
        for dev, a in zip(bufs[:3], (q, k, v)):
            assert be.to_device(dev, a)
        assert be.flash_attn_batch(bufs[0], bufs[1], bufs[2], bufs[3], d, heads, kv_heads, batch, pos0, capacity * d, scale), be.last_error
        got = np.zeros_like(q)
        assert be.to_host(got, bufs[3])
        want = exact(q, k, v, heads, kv_heads, pos0, scale)
        assert np.isfinite(got).all()
        err = float(np.abs(got - want).max() / np.abs(want).max())
        assert err <= 2e-5, err
    finally:
        for dev in bufs:
            be.free(dev)


def test_batch_attention_rejects_what_it_cannot_take(be):
    buf = be.alloc(1 << 16)
    try:
        host = np.zeros(64, np.float32)
        assert not be.flash_attn_batch(buf, buf, buf, buf, 64, 8, 2, 0, 0, 4096, 0.125)          # empty batch
        assert not be.flash_attn_batch(buf, buf, buf, buf, 64, 8, 2, 4, 0, 3 * 64, 0.125)        # cache shorter than the batch
        assert not be.flash_attn_batch(host.ctypes.data, buf, buf, buf, 64, 8, 2, 1, 0, 64, 0.125)   # host pointer
        assert not be.flash_attn_batch(buf, buf, buf, buf, 80, 8, 2, 1, 0, 80, 0.1) and be.last_error == eb.UNSUPPORTED_OP
        assert not be.flash_attn_batch(buf, buf, buf, buf, 64, 12, 4, 1, 0, 64, 0.125) and be.last_error == eb.UNSUPPORTED_OP
    finally:
        be.free(buf)
