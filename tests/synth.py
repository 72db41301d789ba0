"""Seeded synthetic inputs for the parity tests (shapes and distributions of the
benchmark configurations: weights N(0, 0.02), activations N(0, 1))."""
import numpy as np

from oracle import bindings as ob


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def weights_f32(seed, m, k):
    return (rng(seed).standard_normal((m, k), dtype=np.float32) * np.float32(0.02))


def activations_f32(seed, k, n=1):
    """[k, n] token-fastest, the op_mul_mat src1 layout b[p*n + j]."""
    return rng(seed).standard_normal((k, n), dtype=np.float32)


def encoded_weights(port, t, seed, m, k):
    return port.encode_rows(t, weights_f32(seed, m, k), k, m)


def random_blocks(t, seed, m, k):
    """Random block bytes with sane f16 scales (exponent bounded so products stay finite)."""
    g = rng(seed)
    nblk = m * k // ob.BLOCK_ELEMS[t]
    bb = ob.BLOCK_BYTES[t]
    raw = g.integers(0, 256, size=(nblk, bb), dtype=np.uint8)

    def f16_bits(n):
        # |value| in [2^-10, 2^-3], random sign
        e = g.integers(5, 13, size=n).astype(np.uint16)
        mant = g.integers(0, 1024, size=n).astype(np.uint16)
        sign = g.integers(0, 2, size=n).astype(np.uint16)
        return (sign << 15) | (e << 10) | mant

    def put16(col, vals):
        raw[:, col] = (vals & 0xFF).astype(np.uint8)
        raw[:, col + 1] = (vals >> 8).astype(np.uint8)

    if t in (ob.Q4_0, ob.Q8_0):
        put16(0, f16_bits(nblk))
    elif t == ob.Q4_K:
        put16(0, f16_bits(nblk) & 0x7FFF)
        put16(2, f16_bits(nblk) & 0x7FFF)
    elif t == ob.Q6_K:
        put16(208, f16_bits(nblk))
    return raw.reshape(-1)
