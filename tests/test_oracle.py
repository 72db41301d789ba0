"""Pins the CPU oracle: the plain-C restatement (oracle/emel_oracle.c) against

  * the reference's own known-answer tests and deterministic fixtures
    (tests/kernel/lifecycle_tests.cpp:121-310, tests/kernel/x86_64_tests.cpp:50-145,
    tests/kernel/test_helpers.hpp:324-343), restated here as data;
  * the reference's kernel headers compiled in place (oracle/_ref), bit for bit
    on seeded inputs, wherever that build is present;
  * the committed golden vectors under tests/golden (generated from oracle/_ref).
"""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import bindings as ob
from tests import synth

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "hot_path_golden.npz")


# ---------------------------------------------------------------- fixtures restated
def kat_q4_k_block():
    """tests/kernel/lifecycle_tests.cpp:144-160: d=dmin=1.0, scales 1 / mins 1, quants 0."""
    b = np.zeros(144, np.uint8)
    b[0:2] = [0x00, 0x3C]
    b[2:4] = [0x00, 0x3C]
    b[4:12] = 0x01
    b[12:16] = 0x11
    return b


def kat_q6_k_block():
    """tests/kernel/lifecycle_tests.cpp:162-166: d=1.0, scales 1, ql=qh=0 (every value -32)."""
    b = np.zeros(210, np.uint8)
    b[192:208] = 1
    b[208:210] = [0x00, 0x3C]
    return b


def fill_block(t, salt):
    """Deterministic block patterns of tests/kernel/x86_64_tests.cpp:87-145."""
    i = lambda n: np.arange(n, dtype=np.uint32)
    u8 = lambda v: (v & 0xFF).astype(np.uint8)
    put16 = lambda v: [v & 0xFF, v >> 8]
    if t == ob.Q4_K:
        b = np.zeros(144, np.uint8)
        b[0:2] = put16(0x3C00 + salt % 17)
        b[2:4] = put16(0x3800 + salt % 13)
        b[4:16] = u8((i(12) * (11 + salt)) ^ (0x47 + salt))
        b[16:144] = u8((i(128) * (5 + salt)) ^ ((0x9D - salt) & 0xFFFFFFFF))
        return b
    if t == ob.Q6_K:
        b = np.zeros(210, np.uint8)
        b[0:128] = u8((i(128) * (19 + salt)) ^ (0x6C + salt))
        b[128:192] = u8((i(64) * (7 + salt)) ^ ((0x95 - salt) & 0xFFFFFFFF))
        b[192:208] = ((((i(16) + salt) * 3) % 31).astype(np.int32) - 15).astype(np.int8).view(np.uint8)
        b[208:210] = put16(0x3C00 + salt % 23)
        return b
    if t == ob.Q8_0:
        b = np.zeros(34, np.uint8)
        b[0:2] = put16(0x3C00 + salt % 23)
        b[2:34] = ((((i(32) + salt) * (5 + salt)) % 251).astype(np.int32) - 125).astype(np.int8).view(np.uint8)
        return b
    if t == ob.Q4_0:
        b = np.zeros(18, np.uint8)
        b[0:2] = put16(0x3C00 + salt % 17)
        b[2:18] = u8((i(16) * (7 + salt)) ^ (0x53 + salt))
        return b
    raise ValueError(t)


def rhs_values(n, salt):
    """make_quantized_rhs_values, tests/kernel/x86_64_tests.cpp:50-60."""
    i = np.arange(n, dtype=np.uint64)
    return ((((i + salt) * (7 + salt)) % 41).astype(np.int64) - 20).astype(np.float32) * np.float32(0.03125)


def run_mul_mat(lib, t, w, k, m, x, n=1, **kw):
    y = np.zeros((m, n), np.float32)
    op = ob.mul_mat_op(w, t, k, m, x, n, y)
    assert lib.mul_mat(op, **kw)
    return y


# ---------------------------------------------------------------- known answers
@pytest.mark.parametrize("which", ["port", "ref"])
def test_kat_all_ones_q4_k_q6_k(which, request):
    lib = request.getfixturevalue(which)
    x = np.ones(256, np.float32)
    assert run_mul_mat(lib, ob.Q4_K, kat_q4_k_block(), 256, 1, x)[0, 0] == pytest.approx(-256.0)
    assert run_mul_mat(lib, ob.Q6_K, kat_q6_k_block(), 256, 1, x)[0, 0] == pytest.approx(-8192.0)


@pytest.mark.parametrize("which", ["port", "ref"])
def test_kat_q8_0_and_argmax(which, request):
    """tests/kernel/lifecycle_tests.cpp:207-310."""
    lib = request.getfixturevalue(which)
    port = request.getfixturevalue("port")
    d = port.fp32_to_fp16(1.0 / 127.0)
    unit = 127.0 * port.fp16_to_fp32(d)
    rows = np.zeros((2, 34), np.uint8)
    rows[:, 0], rows[:, 1] = d & 0xFF, d >> 8
    rows[0, 2:] = 127
    x = np.ones(32, np.float32)
    y = run_mul_mat(lib, ob.Q8_0, rows, 32, 2, x)
    assert y[0, 0] == pytest.approx(unit * unit * 32, rel=1e-6)
    assert y[1, 0] == pytest.approx(0.0, abs=1e-6)

    rows[1, 2:] = 63
    best, idx = np.zeros(1, np.float32), np.full(1, -1, np.int32)
    assert lib.mul_mat_argmax(ob.mul_mat_op(rows, ob.Q8_0, 32, 2, x, 1, best, idx))
    assert idx[0] == 0 and best[0] == pytest.approx(unit * unit * 32, rel=1e-6)

    q4 = np.zeros((2, 144), np.uint8)
    q4[0] = kat_q4_k_block()
    best[:], idx[:] = 0, -1
    assert lib.mul_mat_argmax(ob.mul_mat_op(q4, ob.Q4_K, 256, 2, np.ones(256, np.float32), 1, best, idx))
    assert idx[0] == 1 and best[0] == pytest.approx(0.0, abs=1e-6)


@pytest.mark.parametrize("which", ["port", "ref"])
def test_kat_flash_fixture(which, request):
    """tests/kernel/test_helpers.hpp:324-343 with scale 1: scores (1, 0)."""
    lib = request.getfixturevalue(which)
    q = np.array([1, 0, 0, 0], np.float32)
    k = np.array([0x3C00, 0, 0, 0, 0, 0x3C00, 0, 0], np.uint16)
    v = np.array([0x4000, 0, 0, 0, 0, 0x4400, 0, 0], np.uint16)
    dst = np.zeros(4, np.float32)
    op = ob.flash_op(q, k, v, dst, 4, 1, 1, 2, 2, scale=1.0)
    assert lib.flash_attn(op)
    e = np.exp(1.0)
    np.testing.assert_allclose(dst, [2 * e / (e + 1), 4 / (e + 1), 0, 0], atol=1e-3)


# ---------------------------------------------------------------- fp16 conversions
def test_fp16_to_fp32_all_halves(port):
    halves = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    want = halves.view(np.float16).astype(np.float32)
    got = np.array([port.fp16_to_fp32(int(h)) for h in halves], np.float32)
    nan = np.isnan(want)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))
    assert np.all(np.isnan(got[nan]))


def test_fp16_to_fp32_port_equals_ref(port, ref):
    for h in range(0, 65536, 7):
        a, b = port.fp16_to_fp32(h), ref.fp16_to_fp32(h)
        assert np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32) or (np.isnan(a) and np.isnan(b))


def test_fp32_to_fp16_rne_and_specials(port):
    g = synth.rng(11)
    vals = np.concatenate([
        g.standard_normal(4000).astype(np.float32),
        (g.standard_normal(2000) * 1e-6).astype(np.float32),
        (g.standard_normal(2000) * 3e4).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65520.0, 1e9, -1e9, np.inf, -np.inf, 5.96e-8, 2.98e-8, 6.1e-5,
                  0.33325195, 1.0009765625, 1.00048828125, 1.00146484375], np.float32),
    ])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([port.fp32_to_fp16(float(v)) for v in vals], np.uint16)
    assert np.array_equal(got, want)
    assert port.fp32_to_fp16(float("nan")) == 0x7E00  # src/emel/kernel/detail.hpp:391


def test_fp32_to_fp16_port_equals_ref(port, ref):
    g = synth.rng(12)
    for v in np.concatenate([g.standard_normal(3000), g.standard_normal(500) * 1e-5, g.standard_normal(500) * 7e4]):
        assert port.fp32_to_fp16(float(np.float32(v))) == ref.fp32_to_fp16(float(np.float32(v)))


# ---------------------------------------------------------------- quantizers (bit-exact)
def edge_activations(k, n):
    x = synth.activations_f32(5, k, n)
    x[0:256, 0] = 0.0                                 # all-zero block
    x[256:512, 0] = 0.0
    x[300, 0], x[400, 0] = 1.5, -1.5                  # +max first, -max later (sign of first wins)
    if k >= 1024:
        x[512:768, 0] = np.float32(-2.0)              # constant negative
        x[768:1024, 0] = (np.arange(256) - 127.5).astype(np.float32) / 127.0  # half-way products
    return x


@pytest.mark.parametrize("t", [ob.Q8_K, ob.Q8_0])
@pytest.mark.parametrize("k,n", [(256, 1), (1024, 1), (4096, 1), (1024, 3), (2048, 8)])
def test_quantizer_port_equals_ref(port, ref, t, k, n):
    x = edge_activations(k, n) if k >= 512 else synth.activations_f32(3, k, n)
    for col in range(n):
        assert np.array_equal(port.quantize(t, x, k, n, col), ref.quantize(t, x, k, n, col))


def test_q8_k_properties(port):
    k = 2048
    x = edge_activations(k, 1)
    q = port.quantize(ob.Q8_K, x, k).reshape(-1, 292)
    d = q[:, 0:4].copy().view(np.float32).ravel()
    qs = q[:, 4:260].view(np.int8).astype(np.int32)
    bs = q[:, 260:292].copy().view(np.int16).reshape(-1, 16)
    assert np.array_equal(bs, qs.reshape(-1, 16, 16).sum(axis=2))
    assert d[0] == 0 and not q[0].any()               # zero block -> all fields zero
    assert qs[1, 300 - 256] == -127 and qs[1, 400 - 256] == 127   # first max keeps sign, maps to -127
    assert qs.max() <= 127 and qs.min() >= -128
    deq = qs * d[:, None]
    assert np.abs(deq.ravel() - x[:, 0]).max() <= np.abs(d).max() * 0.5 + 1e-6


def test_q4_0_encoder_port_equals_ref(port, ref):
    x = synth.weights_f32(21, 4, 512).ravel()
    assert np.array_equal(port.quantize_q4_0(x), ref.quantize_q4_0(x))


# ---------------------------------------------------------------- dequantizers (bit-exact)
@pytest.mark.parametrize("t", [ob.Q4_K, ob.Q6_K, ob.Q8_0, ob.Q4_0])
def test_dequantize_port_equals_ref(port, ref, t):
    k, m = 1024, 3
    blocks = synth.random_blocks(t, 31 + t, m, k)
    a, b = port.dequantize(t, blocks, k, m), ref.dequantize(t, blocks, k, m)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    fixed = np.concatenate([fill_block(t, s) for s in range(k // ob.BLOCK_ELEMS[t])])
    assert np.array_equal(port.dequantize(t, fixed, k).view(np.uint32), ref.dequantize(t, fixed, k).view(np.uint32))


@pytest.mark.parametrize("t,tol", [(ob.Q4_K, 0.08), (ob.Q6_K, 0.02), (ob.Q8_0, 0.006), (ob.Q4_0, 0.12)])
def test_weight_encoder_round_trip(port, t, tol):
    """Own-design Q4_K/Q6_K encoders (and the reference-owned Q8_0/Q4_0) decode close to the input."""
    k, m = 2048, 4
    w = synth.weights_f32(41, m, k)
    back = port.dequantize(t, port.encode_rows(t, w, k, m), k, m)
    assert ob.rel_l2(back, w) < tol


# ---------------------------------------------------------------- row dots and mul_mat
@pytest.mark.parametrize("t,salt,rsalt", [(ob.Q4_K, 9, 13), (ob.Q6_K, 17, 19), (ob.Q8_0, 3, 5), (ob.Q4_0, 5, 7)])
def test_row_dot_fixtures(port, ref, t, salt, rsalt):
    """SIMD == scalar fixtures (tests/kernel/x86_64_tests.cpp:330-354, 536-654, 896-920), eps 1e-6."""
    nblk = 4 if t in (ob.Q4_K, ob.Q6_K) else 8
    k = nblk * ob.BLOCK_ELEMS[t]
    lhs = np.concatenate([fill_block(t, b + salt) for b in range(nblk)])
    act_t = ob.Q8_K if t in (ob.Q4_K, ob.Q6_K) else ob.Q8_0
    rhs = ref.quantize(act_t, rhs_values(k, rsalt), k)
    scalar = ref.row_dot(t, lhs, rhs, nblk, "scalar")
    assert ref.row_dot(t, lhs, rhs, nblk, "avx2") == pytest.approx(scalar, rel=1e-6)
    assert np.float32(port.row_dot(t, lhs, rhs, nblk)).view(np.uint32) == np.float32(scalar).view(np.uint32)


@pytest.mark.parametrize("t", [ob.Q4_K, ob.Q6_K, ob.Q8_0, ob.Q4_0])
@pytest.mark.parametrize("k,m,n", [(256, 1, 1), (512, 2, 2), (2048, 33, 1), (4096, 16, 3)])
def test_mul_mat_port_equals_ref(port, ref, t, k, m, n):
    w = synth.encoded_weights(port, t, 51, m, k)
    x = synth.activations_f32(52, k, n)
    a = run_mul_mat(port, t, w, k, m, x, n)
    b = run_mul_mat(ref, t, w, k, m, x, n, route="scalar")
    c = run_mul_mat(ref, t, w, k, m, x, n, route="avx2")
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert ob.rel_l2(c, b) < 1e-6
    d = run_mul_mat(ref, t, w, k, m, x, n, route="avx2", lanes=4)
    assert np.array_equal(c.view(np.uint32), d.view(np.uint32))     # sliced == serial, bit-exact


def test_mul_mat_argmax_port_equals_ref(port, ref):
    k, m = 1024, 257
    w4 = synth.encoded_weights(port, ob.Q4_0, 61, m, k)
    for lib in (port, ref):   # no Q4_0 branch in run_mul_mat_argmax (src/emel/kernel/detail.hpp:3621-3731)
        assert not lib.mul_mat_argmax(ob.mul_mat_op(w4, ob.Q4_0, k, m, synth.activations_f32(62, k), 1,
                                                    np.zeros(1, np.float32), np.zeros(1, np.int32)))
    for t in (ob.Q4_K, ob.Q6_K, ob.Q8_0):
        w = synth.encoded_weights(port, t, 61, m, k)
        w = w.reshape(m, -1)
        w[200] = w[7]                                  # duplicate row: lowest index must win a tie
        x = synth.activations_f32(62, k)
        outs = []
        for lib in (port, ref):
            best, idx = np.zeros(1, np.float32), np.zeros(1, np.int32)
            assert lib.mul_mat_argmax(ob.mul_mat_op(w, t, k, m, x, 1, best, idx))
            outs.append((best[0], idx[0]))
        assert outs[0] == outs[1]
        y = run_mul_mat(port, t, w, k, m, x)
        assert outs[0][1] == int(np.argmax(y[:, 0])) and outs[0][0] == y[:, 0].max()


# ---------------------------------------------------------------- request guards
def guard_cases():
    k, m, n = 512, 4, 2
    w = np.zeros(m * ob.row_bytes(ob.Q4_K, k), np.uint8)
    x = np.zeros((k, n), np.float32)
    y = np.zeros((m, n), np.float32)
    keep = [w, x, y]

    def base(t=ob.Q4_K):
        return ob.mul_mat_op(w, t, k, m, x, n, y)

    cases = [("ok", base())]
    for t in (ob.Q6_K, ob.Q8_0, ob.Q4_0):
        ww = np.zeros(m * ob.row_bytes(t, k), np.uint8)
        keep.append(ww)
        cases.append((f"ok_type_{t}", ob.mul_mat_op(ww, t, k, m, x, n, y)))

    def mut(name, f):
        op = base()
        f(op)
        cases.append((name, op))

    mut("null_src0", lambda o: setattr(o.src0, "data", None))
    mut("null_src1", lambda o: setattr(o.src1, "data", None))
    mut("null_dst", lambda o: setattr(o.dst, "data", None))
    mut("k_mismatch", lambda o: o.src1.ne.__setitem__(1, k - 256))
    mut("dst_rows", lambda o: o.dst.ne.__setitem__(1, m + 1))
    mut("dst_cols", lambda o: o.dst.ne.__setitem__(0, n + 1))
    mut("row_stride", lambda o: o.src0.nb.__setitem__(1, o.src0.nb[1] + 16))
    mut("nb0", lambda o: o.src0.nb.__setitem__(0, 2))
    mut("nb2", lambda o: o.src0.nb.__setitem__(2, 0))
    mut("rank", lambda o: o.src0.ne.__setitem__(2, 2))
    mut("src1_f16", lambda o: setattr(o.src1, "type", ob.F16))
    mut("dst_f16", lambda o: setattr(o.dst, "type", ob.F16))
    mut("src1_strided", lambda o: o.src1.nb.__setitem__(1, 4 * n + 4))
    mut("params_size", lambda o: setattr(o, "op_params_size", 65))
    mut("zero_rows", lambda o: (o.src0.ne.__setitem__(1, 0), o.dst.ne.__setitem__(1, 0)))
    mut("k_not_block_multiple", lambda o: (o.src0.ne.__setitem__(0, 300), o.src1.ne.__setitem__(1, 300)))
    big_k = 256 * 129
    bw = np.zeros(ob.row_bytes(ob.Q4_K, big_k), np.uint8)
    bx = np.zeros(big_k, np.float32)
    by = np.zeros(1, np.float32)
    keep += [bw, bx, by]
    cases.append(("k_over_128_blocks", ob.mul_mat_op(bw, ob.Q4_K, big_k, 1, bx, 1, by)))
    ok_k = 256 * 128
    cases.append(("k_at_128_blocks", ob.mul_mat_op(bw, ob.Q4_K, ok_k, 1, bx, 1, by)))
    return cases, keep


def test_mul_mat_guard_matches_reference(port, ref):
    cases, _keep = guard_cases()
    for name, op in cases:
        assert port.can_run(ob.OP_MUL_MAT, op) == ref.can_run(ob.OP_MUL_MAT, op), name
    verdicts = {n: port.can_run(ob.OP_MUL_MAT, o) for n, o in cases}
    assert verdicts["ok"] and verdicts["k_at_128_blocks"]
    assert not verdicts["k_over_128_blocks"] and not verdicts["row_stride"] and not verdicts["null_src0"]


def flash_inputs(seed, hd, heads, kvh, T, cap):
    g = synth.rng(seed)
    q = g.standard_normal((heads, hd), dtype=np.float32)
    k = (g.standard_normal((kvh, cap, hd), dtype=np.float32) * 0.5).astype(np.float16)
    v = (g.standard_normal((kvh, cap, hd), dtype=np.float32)).astype(np.float16)
    return q, k.view(np.uint16), v.view(np.uint16)


def test_flash_guard_matches_reference(port, ref):
    hd, heads, kvh, T, cap = 64, 8, 2, 40, 48
    q, k, v = flash_inputs(71, hd, heads, kvh, T, cap)
    dst = np.zeros((heads, hd), np.float32)
    mk = lambda **kw: ob.flash_op(q, k, v, dst, hd, heads, kvh, T, cap, **kw)
    cases = [("ok", mk(scale=0.125)), ("ok_default_scale", mk()), ("ok_masked", mk(scale=0.125, masked_total=cap))]

    def mut(name, f, **kw):
        op = mk(scale=0.125, **kw)
        f(op)
        cases.append((name, op))

    mut("masked_lt_T", lambda o: None, masked_total=T - 1)
    mut("neg_scale", lambda o: o.op_params.__setitem__(3, 0xBE))
    mut("head_dim_mismatch", lambda o: (o.src1.ne.__setitem__(0, hd - 1), o.src1.nb.__setitem__(1, 2 * (hd - 1))))
    mut("zero_kv_heads", lambda o: (o.src1.ne.__setitem__(2, 0), o.src2.ne.__setitem__(2, 0)))
    mut("null_k", lambda o: setattr(o.src1, "data", None))
    mut("null_v", lambda o: setattr(o.src2, "data", None))
    mut("two_queries", lambda o: (o.src0.ne.__setitem__(1, 2), o.dst.ne.__setitem__(1, 2)))
    mut("heads_not_multiple", lambda o: (o.src1.ne.__setitem__(2, 3), o.src2.ne.__setitem__(2, 3)))
    mut("k_f32", lambda o: setattr(o.src1, "type", ob.F32))
    mut("v_tokens", lambda o: o.src2.ne.__setitem__(1, T + 1))
    for name, op in cases:
        assert port.can_run(ob.OP_FLASH_ATTN_EXT, op) == ref.can_run(ob.OP_FLASH_ATTN_EXT, op), name
    assert port.can_run(ob.OP_FLASH_ATTN_EXT, cases[0][1])
    assert not port.can_run(ob.OP_FLASH_ATTN_EXT, cases[3][1])


# ---------------------------------------------------------------- flash decode attention
@pytest.mark.parametrize("hd,heads,kvh,T,cap", [(64, 12, 12, 104, 104), (128, 8, 2, 300, 320), (128, 32, 8, 769, 784)])
def test_flash_port_vs_ref(port, ref, hd, heads, kvh, T, cap):
    q, k, v = flash_inputs(81, hd, heads, kvh, T, cap)
    outs = {}
    for name, lib, kw in (("port", port, {}), ("scalar", ref, {"route": "scalar"}), ("avx2", ref, {"route": "avx2"})):
        dst = np.zeros((heads, hd), np.float32)
        assert lib.flash_attn(ob.flash_op(q, k, v, dst, hd, heads, kvh, T, cap, scale=1 / np.sqrt(hd), masked_total=cap), **kw)
        outs[name] = dst
    assert np.array_equal(outs["port"].view(np.uint32), outs["scalar"].view(np.uint32))
    # the reference's own tolerance between its routes (tests/kernel/test_helpers.hpp:22-27)
    assert np.abs(outs["avx2"] - outs["scalar"]).max() <= 1e-3
    dst = np.zeros((heads, hd), np.float32)
    truth = port.flash_attn_f64(ob.flash_op(q, k, v, dst, hd, heads, kvh, T, cap, scale=1 / np.sqrt(hd)), heads, hd)
    assert np.abs(outs["scalar"] - truth).max() <= 5e-3


def test_flash_token_major_layout(port, ref):
    """Interleaved KV (nb1 = kv_dim, nb2 = head_dim) as in tests/kernel/lifecycle_tests.cpp:1041-1048."""
    hd, heads, T = 64, 4, 50
    g = synth.rng(91)
    q = g.standard_normal((heads, hd), dtype=np.float32)
    k = g.standard_normal((T, heads, hd), dtype=np.float32).astype(np.float16).view(np.uint16)
    v = g.standard_normal((T, heads, hd), dtype=np.float32).astype(np.float16).view(np.uint16)
    res = []
    for lib in (port, ref):
        dst = np.zeros((heads, hd), np.float32)
        op = ob.flash_op(q, k, v, dst, hd, heads, heads, T, T, scale=0.125)
        for s in (op.src1, op.src2):
            s.nb[1], s.nb[2], s.nb[3] = 2 * heads * hd, 2 * hd, 2 * heads * hd * T
        assert lib.flash_attn(op)
        res.append(dst)
    assert np.array_equal(res[0].view(np.uint32), res[1].view(np.uint32))


# ---------------------------------------------------------------- row slicing
def test_row_slice_tiling(port):
    """Properties of tests/kernel/matmul_tests.cpp:96-175: disjoint, ordered, covering, ragged tail."""
    for rows in (1, 7, 8, 9, 4096, 128256):
        for lanes in (2, 4, 8):
            nxt = 0
            for lane in range(lanes):
                b, c = port.row_slice(rows, lane, lanes)
                assert b == nxt
                nxt += c
            assert nxt == rows
            counts = [port.row_slice(rows, l, lanes)[1] for l in range(lanes)]
            assert max(counts) - min(counts) <= 1


# ---------------------------------------------------------------- committed golden vectors
def test_port_matches_committed_golden(port):
    g = np.load(GOLDEN)
    for t in (ob.Q8_K, ob.Q8_0):
        x = g[f"quant_x_{t}"]
        k, n = x.shape
        for col in range(n):
            assert np.array_equal(port.quantize(t, x, k, n, col), g[f"quant_y_{t}_{col}"])
    for t in (ob.Q4_K, ob.Q6_K, ob.Q8_0, ob.Q4_0):
        w = g[f"w_{t}"]
        k, m, n = (int(v) for v in g[f"shape_{t}"])
        assert np.array_equal(port.dequantize(t, w, k, m).view(np.uint32), g[f"deq_{t}"].view(np.uint32))
        y = run_mul_mat(port, t, w, k, m, g[f"x_{t}"], n)
        assert np.array_equal(y.view(np.uint32), g[f"y_scalar_{t}"].view(np.uint32))
        assert ob.rel_l2(y, g[f"y_avx2_{t}"]) < 1e-6
    hd, heads, kvh, T, cap = (int(v) for v in g["flash_shape"])
    dst = np.zeros((heads, hd), np.float32)
    assert port.flash_attn(ob.flash_op(g["flash_q"], g["flash_k"], g["flash_v"], dst, hd, heads, kvh, T, cap,
                                       scale=float(g["flash_scale"]), masked_total=cap))
    assert np.array_equal(dst.view(np.uint32), g["flash_scalar"].view(np.uint32))
    assert np.abs(dst - g["flash_avx2"]).max() <= 1e-3
