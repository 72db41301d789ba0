"""GPU parity tests: every call goes through the C-ABI (libemelb.so) and is
checked against the CPU oracle on the same seeded inputs.

Bars: activation quantizers and block dequantizers bit-exact; op_mul_mat f32
outputs relative L2 <= 1e-5; argmax identical index; attention within the
reference's own tolerance (abs 1e-3, tests/kernel/test_helpers.hpp:22-27) for
the split-KV kernel and ~bit-level for the reference-order kernel.
"""
import numpy as np
import pytest

import emel_cpp_b200 as eb
from oracle import bindings as ob
from tests import synth
from tests.test_oracle import (GOLDEN, edge_activations, fill_block, flash_inputs, kat_q4_k_block, kat_q6_k_block,
                               rhs_values)

pytestmark = pytest.mark.gpu

GEMV_TOL = 1e-5
WEIGHT_TYPES = [eb.Q4_K, eb.Q6_K, eb.Q8_0, eb.Q4_0]


@pytest.fixture(scope="module")
def be():
    b = eb.Backend(0)
    yield b
    b.close()


def act_type(t):
    return eb.Q8_K if t in (eb.Q4_K, eb.Q6_K) else eb.Q8_0


def gpu_mul_mat(be, t, w, k, m, x, n=1):
    y = np.zeros((m, n), np.float32)
    assert be.mul_mat(eb.mul_mat_op(w, t, k, m, x, n, y)), be.last_error
    return y


def cpu_mul_mat(lib, t, w, k, m, x, n=1, **kw):
    """The reference's x86 route (AVX2/FMA) where oracle/_ref is present, else the C port."""
    y = np.zeros((m, n), np.float32)
    if isinstance(lib, ob.Ref):
        kw.setdefault("route", "avx2")
    assert lib.mul_mat(ob.mul_mat_op(w, t, k, m, x, n, y), **kw)
    return y


def assert_mul_mat_parity(got, want, checker, t):
    """rel-L2 <= 1e-5 always; bit-for-bit against the reference's AVX2 route (which the kernels
    follow block by block) and, for Q8_0/Q4_0, against the scalar order of the C port too."""
    assert ob.rel_l2(got, want) <= GEMV_TOL, ob.rel_l2(got, want)
    if isinstance(checker, ob.Ref) or t in (eb.Q8_0, eb.Q4_0):
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), float(np.abs(got - want).max())


# ------------------------------------------------------------------ quantizers: bit-exact
@pytest.mark.parametrize("t", [eb.Q8_K, eb.Q8_0])
@pytest.mark.parametrize("k,n", [(256, 1), (1024, 1), (4096, 1), (1024, 3), (2048, 8), (14336, 2), (32768, 1)])
def test_quantize_bit_exact(be, checker, t, k, n):
    x = edge_activations(k, n) if k >= 1024 else synth.activations_f32(3, k, n)
    rb = eb.row_bytes(t, k)
    out = np.zeros((n, rb), np.uint8)
    dst = eb.View()
    dst.data, dst.type = out.ctypes.data, t
    dst.ne[0], dst.ne[1], dst.ne[2], dst.ne[3] = k, n, 1, 1
    dst.nb[0], dst.nb[1], dst.nb[2], dst.nb[3] = 1, rb, rb * n, rb * n
    assert be.quantize(eb.dense_view(x, eb.F32, [n, k]), dst), be.last_error
    for col in range(n):
        assert np.array_equal(out[col], checker.quantize(t, x, k, n, col)), (t, k, n, col)


def test_quantize_rejects_bad_requests(be):
    x = np.zeros((300, 1), np.float32)
    out = np.zeros(400, np.uint8)
    dst = eb.View()
    dst.data, dst.type = out.ctypes.data, eb.Q8_K
    dst.ne[0], dst.ne[1], dst.ne[2], dst.ne[3] = 300, 1, 1, 1
    dst.nb[0], dst.nb[1], dst.nb[2], dst.nb[3] = 1, 400, 400, 400
    assert not be.quantize(eb.dense_view(x, eb.F32, [1, 300]), dst)      # K not a block multiple
    assert be.last_error == eb.INVALID_REQUEST


# ------------------------------------------------------------------ dequantizers: bit-exact
@pytest.mark.parametrize("t", WEIGHT_TYPES)
def test_dequantize_bit_exact(be, checker, port, t):
    k, m = 2048, 5
    for blocks in (synth.random_blocks(t, 31 + t, m, k), synth.encoded_weights(port, t, 7, m, k)):
        out = np.zeros((m, k), np.float32)
        assert be.dequantize(eb.quant_view(blocks, t, k, m), eb.dense_view(out, eb.F32, [k, m])), be.last_error
        assert np.array_equal(out.view(np.uint32), checker.dequantize(t, blocks, k, m).view(np.uint32))


# ------------------------------------------------------------------ op_mul_mat
def test_known_answers_through_cabi(be, port):
    """tests/kernel/lifecycle_tests.cpp:121-279."""
    x = np.ones(256, np.float32)
    assert gpu_mul_mat(be, eb.Q4_K, kat_q4_k_block(), 256, 1, x)[0, 0] == pytest.approx(-256.0)
    assert gpu_mul_mat(be, eb.Q6_K, kat_q6_k_block(), 256, 1, x)[0, 0] == pytest.approx(-8192.0)
    d = port.fp32_to_fp16(1.0 / 127.0)
    unit = 127.0 * port.fp16_to_fp32(d)
    rows = np.zeros((2, 34), np.uint8)
    rows[:, 0], rows[:, 1] = d & 0xFF, d >> 8
    rows[0, 2:] = 127
    y = gpu_mul_mat(be, eb.Q8_0, rows, 32, 2, np.ones(32, np.float32))
    assert y[0, 0] == pytest.approx(unit * unit * 32, rel=1e-6) and y[1, 0] == pytest.approx(0.0, abs=1e-6)


@pytest.mark.parametrize("t,salt", [(eb.Q4_K, 29), (eb.Q6_K, 17), (eb.Q8_0, 3), (eb.Q4_0, 5)])
def test_reference_block_fixtures(be, checker, t, salt):
    """The deterministic block patterns of tests/kernel/x86_64_tests.cpp:87-145, n = 2."""
    nblk, m, n = (2, 2, 2) if t in (eb.Q4_K, eb.Q6_K) else (8, 2, 2)
    k = nblk * eb.BLOCK_ELEMS[t]
    w = np.concatenate([fill_block(t, i + salt) for i in range(m * nblk)])
    x = np.stack([rhs_values(k, 13), rhs_values(k, 7)], axis=1).copy()
    got, want = gpu_mul_mat(be, t, w, k, m, x, n), cpu_mul_mat(checker, t, w, k, m, x, n)
    assert_mul_mat_parity(got, want, checker, t)


@pytest.mark.parametrize("t", WEIGHT_TYPES)
@pytest.mark.parametrize("k,m,n", [
    (256, 1, 1), (512, 7, 1), (1280, 33, 2),          # generic kernel (K not a multiple of 2048)
    (2048, 1, 1), (2048, 257, 1), (4096, 1000, 1),    # streaming kernel, ragged row counts
    (4096, 64, 2), (2048, 129, 3), (4096, 40, 8), (2048, 31, 13),
    (14336, 24, 2), (14336, 24, 4), (8192, 19, 7),    # long rows: column copies that fit / do not fit in shared memory
    (2048, 2048, 12), (2048, 4096, 20), (4096, 2048, 16), (2048, 512, 20),   # column groups after the first, many CTAs
    (1024, 70, 9), (4096, 130, 31), (8192, 64, 16), (512, 5, 17), (14336, 100, 16),   # 9..31 columns: Q4_K takes the mma.sync kernel
])
def test_mul_mat_parity(be, checker, port, t, k, m, n):
    w = synth.encoded_weights(port, t, 100 + t, m, k)
    x = synth.activations_f32(200 + t, k, n)
    got, want = gpu_mul_mat(be, t, w, k, m, x, n), cpu_mul_mat(checker, t, w, k, m, x, n)
    assert_mul_mat_parity(got, want, checker, t)


@pytest.mark.parametrize("t", [eb.Q8_0, eb.Q4_0])
@pytest.mark.parametrize("k,m,n", [
    (256, 128, 32), (512, 5, 33), (1024, 300, 130), (2048, 129, 257), (4096, 260, 64), (1280, 384, 200), (14336, 150, 70),
])
def test_mul_mat_many_columns_block32_tensor_core_kernel(be, checker, port, t, k, m, n):
    """32 or more columns of Q8_0 / Q4_0 take the mma.sync kernel (one 32-weight block per instruction, scales
    applied block by block in order): ragged tiles in both directions and the same bits as the mat-vec route."""
    w = synth.encoded_weights(port, t, 500 + m, m, k)
    x = synth.activations_f32(600 + n, k, n)
    got, want = gpu_mul_mat(be, t, w, k, m, x, n), cpu_mul_mat(checker, t, w, k, m, x, n)
    assert_mul_mat_parity(got, want, checker, t)
    x8 = np.ascontiguousarray(x.reshape(k, n)[:, :8])
    got8 = gpu_mul_mat(be, t, w, k, m, x8, 8)
    assert np.array_equal(got.reshape(m, n)[:, :8].view(np.uint32), got8.view(np.uint32))


@pytest.mark.parametrize("k,m,n", [
    (256, 128, 32), (512, 5, 33), (1024, 300, 130), (2048, 129, 257), (4096, 260, 64), (1280, 384, 200),
])
def test_mul_mat_many_columns_tensor_core_kernel(be, checker, port, k, m, n):
    """32 or more columns of Q4_K take the tcgen05 kernel: ragged tiles in both directions, one and
    many super-blocks, and the same bits as the mat-vec route."""
    w = synth.encoded_weights(port, eb.Q4_K, 300 + m, m, k)
    x = synth.activations_f32(400 + n, k, n)
    got, want = gpu_mul_mat(be, eb.Q4_K, w, k, m, x, n), cpu_mul_mat(checker, eb.Q4_K, w, k, m, x, n)
    assert_mul_mat_parity(got, want, checker, eb.Q4_K)
    # the first 8 columns alone run the mat-vec kernels: identical bits
    x8 = np.ascontiguousarray(x.reshape(k, n)[:, :8])
    got8 = gpu_mul_mat(be, eb.Q4_K, w, k, m, x8, 8)
    assert np.array_equal(got.reshape(m, n)[:, :8].view(np.uint32), got8.view(np.uint32))
    assert be.sync()       # a bounded wait that ran out would surface here


@pytest.mark.parametrize("k,m,n", [
    (2048, 128, 32), (2048, 5, 33), (4096, 300, 130), (2048, 129, 257), (4096, 260, 64), (14336, 150, 70), (6144, 70, 9),
    (4096, 64, 17), (2048, 1000, 40),
])
def test_mul_mat_many_columns_q6_k(be, checker, port, k, m, n):
    """Nine or more columns of Q6_K (K a multiple of 2048) take the mma.sync kernel, one instruction per 16-weight
    scale group: ragged tiles in both directions, every column tile width, the same bits as the mat-vec route."""
    w = synth.encoded_weights(port, eb.Q6_K, 700 + m, m, k)
    x = synth.activations_f32(800 + n, k, n)
    got, want = gpu_mul_mat(be, eb.Q6_K, w, k, m, x, n), cpu_mul_mat(checker, eb.Q6_K, w, k, m, x, n)
    assert_mul_mat_parity(got, want, checker, eb.Q6_K)
    x8 = np.ascontiguousarray(x.reshape(k, n)[:, :8])
    got8 = gpu_mul_mat(be, eb.Q6_K, w, k, m, x8, 8)
    assert np.array_equal(got.reshape(m, n)[:, :8].view(np.uint32), got8.view(np.uint32))


@pytest.mark.parametrize("n", [48, 12])
def test_mul_mat_many_columns_q6_k_random_block_bytes(be, checker, n):
    """Arbitrary block bytes: every 6-bit code and every int8 scale, -128 included."""
    k, m = 4096, 96
    w = synth.random_blocks(eb.Q6_K, 910, m, k)
    x = synth.activations_f32(911, k, n)
    got, want = gpu_mul_mat(be, eb.Q6_K, w, k, m, x, n), cpu_mul_mat(checker, eb.Q6_K, w, k, m, x, n)
    assert_mul_mat_parity(got, want, checker, eb.Q6_K)


@pytest.mark.parametrize("n", [96, 16, 23])
def test_mul_mat_many_columns_random_block_bytes(be, checker, n):
    """Arbitrary scale/min bits (all 6-bit values, extreme nibbles) through the tcgen05 kernel (96 columns) and
    the mma.sync kernel (16 and 23 columns)."""
    k, m = 1024, 192
    rng = synth.rng(77)
    w = rng.integers(0, 256, size=m * eb.row_bytes(eb.Q4_K, k), dtype=np.uint8)
    blocks = w.reshape(-1, eb.BLOCK_BYTES[eb.Q4_K])
    blocks[:, 1] = rng.integers(0x18, 0x30, size=blocks.shape[0])     # sane f16 exponents for d and dmin
    blocks[:, 3] = rng.integers(0x18, 0x30, size=blocks.shape[0])
    x = synth.activations_f32(78, k, n)
    got, want = gpu_mul_mat(be, eb.Q4_K, w, k, m, x, n), cpu_mul_mat(checker, eb.Q4_K, w, k, m, x, n)
    assert_mul_mat_parity(got, want, checker, eb.Q4_K)


@pytest.mark.parametrize("t", WEIGHT_TYPES)
def test_mul_mat_random_block_bytes(be, checker, t):
    """Arbitrary block bytes (all scale/min/quant codes), not just encoder output."""
    k, m = 4096, 48
    w = synth.random_blocks(t, 300 + t, m, k)
    x = synth.activations_f32(301, k)
    got, want = gpu_mul_mat(be, t, w, k, m, x), cpu_mul_mat(checker, t, w, k, m, x)
    assert_mul_mat_parity(got, want, checker, t)


@pytest.mark.parametrize("t", [eb.Q4_K, eb.Q8_0])
def test_max_block_count(be, checker, port, t):
    """K at the reference's block limit (128 K-blocks / 1024 32-blocks)."""
    k, m = 32768, 9
    w = synth.encoded_weights(port, t, 400, m, k)
    x = synth.activations_f32(401, k)
    assert_mul_mat_parity(gpu_mul_mat(be, t, w, k, m, x), cpu_mul_mat(checker, t, w, k, m, x), checker, t)
    k2 = k + eb.BLOCK_ELEMS[t]
    w2 = np.zeros(eb.row_bytes(t, k2), np.uint8)
    assert not be.mul_mat(eb.mul_mat_op(w2, t, k2, 1, np.zeros(k2, np.float32), 1, np.zeros(1, np.float32)))
    assert be.last_error == eb.INVALID_REQUEST


def test_config1_q4_k_4096(be, checker, port):
    """Configuration 1: 4096x4096 Q4_K, x ~ N(0,1) quantized to Q8_K."""
    k = m = 4096
    w = synth.encoded_weights(port, eb.Q4_K, 1, m, k)
    x = synth.activations_f32(2, k)
    got = gpu_mul_mat(be, eb.Q4_K, w, k, m, x)
    assert_mul_mat_parity(got, cpu_mul_mat(checker, eb.Q4_K, w, k, m, x), checker, eb.Q4_K)


@pytest.mark.parametrize("n", [1, 8, 64])
def test_config2_q8_0_sweep(be, checker, port, n):
    """Configuration 2: 14336x4096 Q8_0, token batch n (512 is covered by the GEMM tests)."""
    k, m = 4096, 14336
    w = synth.encoded_weights(port, eb.Q8_0, 3, m, k)
    x = synth.activations_f32(4, k, n)
    got = gpu_mul_mat(be, eb.Q8_0, w, k, m, x, n)
    kw = {"lanes": 8} if isinstance(checker, ob.Ref) else {}
    assert_mul_mat_parity(got, cpu_mul_mat(checker, eb.Q8_0, w, k, m, x, n, **kw), checker, eb.Q8_0)


def test_resident_weights_by_host_pointer(be, checker, port):
    """A view may carry the host (mmap) address of an uploaded span; bytes are unchanged on the device."""
    k, m = 2048, 300
    w = synth.encoded_weights(port, eb.Q6_K, 5, m, k)
    dev = be.upload(77, w, tensor_type=eb.Q6_K)
    st = be.state(77)
    assert eb.LIFECYCLE[st.lifecycle_state] == "resident" and st.buffer == dev and st.buffer_bytes == w.nbytes
    back = np.zeros_like(w)
    assert be.to_host(back, dev) and np.array_equal(back, w)
    x = synth.activations_f32(6, k)
    want = cpu_mul_mat(checker, eb.Q6_K, w, k, m, x)
    before = be.diagnostics()["h2d_bytes"]
    got_host_key = gpu_mul_mat(be, eb.Q6_K, w, k, m, x)
    assert be.diagnostics()["h2d_bytes"] - before == x.nbytes      # only the activations moved
    got_dev_ptr = gpu_mul_mat(be, eb.Q6_K, dev, k, m, x)
    assert np.array_equal(got_host_key, got_dev_ptr) and ob.rel_l2(got_host_key, want) <= GEMV_TOL
    # a row slice of a resident span resolves too
    full = eb.mul_mat_op(w, eb.Q6_K, k, m, x, 1, np.zeros((m, 1), np.float32))
    y = np.zeros((m, 1), np.float32)
    full.dst.data = y.ctypes.data
    for lane in range(4):
        s, _, _ = eb.row_slice(full, lane, 4)
        assert be.mul_mat(s)
    assert np.array_equal(y, got_host_key)                          # sliced == unsliced, bit-exact
    assert be.evict(77) and eb.LIFECYCLE[be.state(77).lifecycle_state] == "evicted"
    assert not be.evict(77)
    assert eb.LIFECYCLE[be.state(12345).lifecycle_state] == "unbound"


def test_device_resident_operands_and_prequantized_rhs(be, checker, port):
    k, m = 4096, 512
    for t in (eb.Q4_K, eb.Q8_0):
        w = synth.encoded_weights(port, t, 8, m, k)
        x = synth.activations_f32(9, k)
        dw, dx, dy = be.alloc(w.nbytes), be.alloc(x.nbytes), be.alloc(4 * m)
        assert be.to_device(dw, w) and be.to_device(dx, x)
        assert be.mul_mat(eb.mul_mat_op(dw, t, k, m, dx, 1, dy)) and be.sync()
        y = np.zeros((m, 1), np.float32)
        assert be.to_host(y, dy)
        want = cpu_mul_mat(checker, t, w, k, m, x)
        assert ob.rel_l2(y, want) <= GEMV_TOL
        # the same activations already quantized by the reference quantizer (vector form)
        xq = checker.quantize(act_type(t), x, k)
        y2 = np.zeros((m, 1), np.float32)
        assert be.mul_mat(eb.mul_mat_op(dw, t, k, m, xq, 1, y2, src1_type=act_type(t))), be.last_error
        assert np.array_equal(y2, y)                                 # same integers, same kernel
        for d in (dw, dx, dy):
            assert be.free(d)


def test_linearity_at_full_size(be, port):
    """Size-independent property on configuration-1 shape: W(2^s x) = 2^s W x exactly
    (power-of-two scaling commutes with Q8_K quantization and every f32 product)."""
    k = m = 4096
    w = synth.encoded_weights(port, eb.Q4_K, 11, m, k)
    x = synth.activations_f32(12, k)
    y1 = gpu_mul_mat(be, eb.Q4_K, w, k, m, x)
    y4 = gpu_mul_mat(be, eb.Q4_K, w, k, m, x * np.float32(4.0))
    assert np.array_equal(y4, y1 * np.float32(4.0))


def test_golden_vectors_through_cabi(be):
    g = np.load(GOLDEN)
    for t in WEIGHT_TYPES:
        k, m, n = (int(v) for v in g[f"shape_{t}"])
        y = gpu_mul_mat(be, t, g[f"w_{t}"], k, m, g[f"x_{t}"], n)
        assert ob.rel_l2(y, g[f"y_scalar_{t}"]) <= GEMV_TOL
        assert np.array_equal(y.view(np.uint32), g[f"y_avx2_{t}"].view(np.uint32))    # the route the kernels follow
    for t in (eb.Q8_K, eb.Q8_0):
        x = g[f"quant_x_{t}"]
        k, n = x.shape
        rb = eb.row_bytes(t, k)
        out = np.zeros((n, rb), np.uint8)
        dst = eb.View()
        dst.data, dst.type = out.ctypes.data, t
        dst.ne[0], dst.ne[1], dst.ne[2], dst.ne[3] = k, n, 1, 1
        dst.nb[0], dst.nb[1], dst.nb[2], dst.nb[3] = 1, rb, rb * n, rb * n
        assert be.quantize(eb.dense_view(x, eb.F32, [n, k]), dst)
        for col in range(n):
            assert np.array_equal(out[col], g[f"quant_y_{t}_{col}"])


# ------------------------------------------------------------------ op_mul_mat_argmax
@pytest.mark.parametrize("t", [eb.Q4_K, eb.Q6_K, eb.Q8_0])
@pytest.mark.parametrize("k,m", [(512, 300), (4096, 5000)])
def test_argmax_parity(be, checker, port, t, k, m):
    w = synth.encoded_weights(port, t, 500 + t, m, k).reshape(m, -1)
    x = synth.activations_f32(501, k)
    y = cpu_mul_mat(checker, t, w, k, m, x)[:, 0]
    top = int(np.argmax(y))
    w[min(m - 1, top + 17)] = w[top]                   # exact tie: the lowest row must win
    best, idx = np.zeros(1, np.float32), np.full(1, -1, np.int32)
    assert be.mul_mat_argmax(eb.mul_mat_op(w, t, k, m, x, 1, best, idx)), be.last_error
    rbest, ridx = np.zeros(1, np.float32), np.zeros(1, np.int32)
    assert checker.mul_mat_argmax(ob.mul_mat_op(w, t, k, m, x, 1, rbest, ridx))
    assert idx[0] == ridx[0] == top
    assert best[0] == pytest.approx(rbest[0], rel=1e-5)


def test_argmax_q4_0_rejected_like_reference(be, port):
    k, m = 512, 8
    w = synth.encoded_weights(port, eb.Q4_0, 1, m, k)
    best, idx = np.zeros(1, np.float32), np.zeros(1, np.int32)
    assert not be.mul_mat_argmax(eb.mul_mat_op(w, eb.Q4_0, k, m, np.ones(k, np.float32), 1, best, idx))
    assert be.last_error == eb.UNSUPPORTED_OP


def test_invalid_requests_are_rejected_not_run(be):
    k, m = 512, 4
    w = np.zeros(m * eb.row_bytes(eb.Q4_K, k), np.uint8)
    x = np.zeros(k, np.float32)
    y = np.full(m, 7.0, np.float32)
    op = eb.mul_mat_op(w, eb.Q4_K, k, m, x, 1, y)
    op.src0.nb[1] += 16
    before = be.diagnostics()
    assert not be.mul_mat(op) and be.last_error == eb.INVALID_REQUEST
    after = be.diagnostics()
    assert after["rejected_dispatch_calls"] == before["rejected_dispatch_calls"] + 1
    assert after["kernel_launches"] == before["kernel_launches"] and np.all(y == 7.0)


def test_diagnostics_count_dispatches(be, port):
    k, m = 2048, 16
    before = be.diagnostics()
    for t in WEIGHT_TYPES:
        gpu_mul_mat(be, t, synth.encoded_weights(port, t, 1, m, k), k, m, synth.activations_f32(2, k))
    d = be.diagnostics()
    assert d["optimized_q4_dispatch_calls"] == before["optimized_q4_dispatch_calls"] + 1
    assert d["optimized_q4_vector_dispatch_calls"] == before["optimized_q4_vector_dispatch_calls"] + 1
    assert d["optimized_q6_dispatch_calls"] == before["optimized_q6_dispatch_calls"] + 1
    assert d["optimized_q8_0_dispatch_calls"] == before["optimized_q8_0_dispatch_calls"] + 1
    assert d["optimized_q4_0_dispatch_calls"] == before["optimized_q4_0_dispatch_calls"] + 1
    assert d["kernel_launches"] >= before["kernel_launches"] + 8     # quantize + gemv per call


# ------------------------------------------------------------------ op_flash_attn_ext
def run_flash(lib_call, q, k, v, hd, heads, kvh, T, cap, maker, **kw):
    dst = np.zeros((heads, hd), np.float32)
    op = maker(q, k, v, dst, hd, heads, kvh, T, cap, scale=float(1 / np.sqrt(hd)), masked_total=cap)
    assert lib_call(op, **kw)
    return dst


@pytest.mark.parametrize("hd,heads,kvh,T,cap", [
    (128, 32, 8, 1, 16), (128, 32, 8, 33, 48), (128, 32, 8, 769, 784), (128, 32, 8, 4224, 4224),
    (64, 12, 12, 104, 104), (128, 64, 8, 2050, 2064), (128, 8, 8, 300, 304), (128, 16, 8, 5000, 5008),
])
def test_flash_split_kv(be, port, checker, hd, heads, kvh, T, cap):
    q, k, v = flash_inputs(600 + T, hd, heads, kvh, T, cap)
    be.set_attention_mode(0)
    before = be.diagnostics()["optimized_flash_dispatch_calls"]
    got = run_flash(be.flash_attn_ext, q, k, v, hd, heads, kvh, T, cap, eb.flash_op)
    assert be.diagnostics()["optimized_flash_dispatch_calls"] == before + 1
    dst = np.zeros((heads, hd), np.float32)
    truth = port.flash_attn_f64(ob.flash_op(q, k, v, dst, hd, heads, kvh, T, cap, scale=float(1 / np.sqrt(hd))), heads, hd)
    err_split = np.abs(got - truth).max()
    assert err_split <= 2e-5                           # f32 split-KV sits on the exact softmax
    if T <= 1024:                                      # sequential CPU reference: keep the big ones out of the test time
        want = run_flash(checker.flash_attn, q, k, v, hd, heads, kvh, T, cap, ob.flash_op)
        err_ref = np.abs(want - truth).max()
        # the reference rounds its accumulator to f16 after every token, so it carries the larger
        # error; the two agree to within that error (1e-3 is the reference's tolerance for small values)
        assert err_split <= err_ref + 1e-7
        assert np.abs(got - want).max() <= max(1e-3, 2 * err_ref)


@pytest.mark.parametrize("hd,heads,kvh,T,cap", [(4, 1, 1, 2, 2), (128, 32, 8, 769, 784), (64, 12, 12, 104, 104),
                                                (80, 6, 3, 200, 208), (256, 4, 2, 130, 144)])
def test_flash_reference_order(be, port, hd, heads, kvh, T, cap):
    """Sequential f16-accumulator kernels: the roundings of the reference's scalar route (mode 1)
    and of its x86 AVX2 route (mode 2), in the same order, with libm-exact expf: bit for bit."""
    q, k, v = flash_inputs(700 + T, hd, heads, kvh, T, cap)
    try:
        be.set_attention_mode(1)
        got1 = run_flash(be.flash_attn_ext, q, k, v, hd, heads, kvh, T, cap, eb.flash_op)
        be.set_attention_mode(2)
        got2 = run_flash(be.flash_attn_ext, q, k, v, hd, heads, kvh, T, cap, eb.flash_op)
    finally:
        be.set_attention_mode(0)
    want1 = run_flash(port.flash_attn, q, k, v, hd, heads, kvh, T, cap, ob.flash_op)
    assert np.array_equal(got1.view(np.uint32), want1.view(np.uint32)), float(np.abs(got1 - want1).max())
    ref = ob.ref()
    if ref is not None:
        want2 = run_flash(ref.flash_attn, q, k, v, hd, heads, kvh, T, cap, ob.flash_op, route="avx2")
        assert np.array_equal(got2.view(np.uint32), want2.view(np.uint32)), float(np.abs(got2 - want2).max())
    assert np.abs(got2 - want1).max() <= 1e-3


def test_flash_fixture_and_token_major_layout(be, port):
    """tests/kernel/test_helpers.hpp:324-343 and the interleaved KV layout of
    tests/kernel/lifecycle_tests.cpp:1041-1048; odd head_dim falls to the reference-order kernel."""
    q = np.array([1, 0, 0, 0], np.float32)
    k = np.array([0x3C00, 0, 0, 0, 0, 0x3C00, 0, 0], np.uint16)
    v = np.array([0x4000, 0, 0, 0, 0, 0x4400, 0, 0], np.uint16)
    dst = np.zeros(4, np.float32)
    assert be.flash_attn_ext(eb.flash_op(q, k, v, dst, 4, 1, 1, 2, 2, scale=1.0))
    e = np.exp(1.0)
    np.testing.assert_allclose(dst, [2 * e / (e + 1), 4 / (e + 1), 0, 0], atol=1e-3)

    hd, heads, T = 64, 4, 50
    g = synth.rng(91)
    q = g.standard_normal((heads, hd), dtype=np.float32)
    kk = g.standard_normal((T, heads, hd), dtype=np.float32).astype(np.float16).view(np.uint16)
    vv = g.standard_normal((T, heads, hd), dtype=np.float32).astype(np.float16).view(np.uint16)
    outs = []
    for call, maker in ((be.flash_attn_ext, eb.flash_op), (port.flash_attn, ob.flash_op)):
        d = np.zeros((heads, hd), np.float32)
        op = maker(q, kk, vv, d, hd, heads, heads, T, T, scale=0.125)
        for s in (op.src1, op.src2):
            s.nb[1], s.nb[2], s.nb[3] = 2 * heads * hd, 2 * hd, 2 * heads * hd * T
        assert call(op)
        outs.append(d)
    assert np.abs(outs[0] - outs[1]).max() <= 1e-3


def test_flash_rejects_like_reference(be):
    hd, heads, kvh, T, cap = 64, 8, 2, 40, 48
    q, k, v = flash_inputs(71, hd, heads, kvh, T, cap)
    dst = np.zeros((heads, hd), np.float32)
    op = eb.flash_op(q, k, v, dst, hd, heads, kvh, T, cap, scale=0.125, masked_total=T - 1)
    assert not be.flash_attn_ext(op) and be.last_error == eb.INVALID_REQUEST
    op = eb.flash_op(q, k, v, dst, hd, heads, kvh, T, cap, scale=0.125)
    op.src1.data = None
    assert not be.flash_attn_ext(op) and be.last_error == eb.INVALID_REQUEST


# ------------------------------------------------------------------ quantize once, multiply many
def test_prepared_rhs_matches_full_dispatch(be, port):
    k, n = 4096, 3
    x = synth.activations_f32(800, k, n)
    for t, m in ((eb.Q4_K, 96), (eb.Q6_K, 40), (eb.Q8_0, 64)):
        w = synth.encoded_weights(port, t, 801, m, k)
        full = gpu_mul_mat(be, t, w, k, m, x, n)
        dw = be.alloc(w.nbytes)
        assert be.to_device(dw, w)
        assert be.prepare_rhs(eb.dense_view(x, eb.F32, [n, k]), t), be.last_error
        before = be.diagnostics()["kernel_launches"]
        y = np.zeros((m, n), np.float32)
        assert be.mul_mat_prepared(eb.mul_mat_op(dw, t, k, m, x, n, y)), be.last_error
        assert np.array_equal(y, full)
        y2 = np.zeros((m, n), np.float32)
        assert be.mul_mat_prepared(eb.mul_mat_op(dw, t, k, m, x, n, y2)) and np.array_equal(y2, full)
        assert be.diagnostics()["kernel_launches"] - before <= 4          # matrix kernels only, no quantizer
        # a full dispatch invalidates the planes; a mismatching shape is rejected
        gpu_mul_mat(be, t, w, k, m, x[:, :1].copy(), 1)
        assert not be.mul_mat_prepared(eb.mul_mat_op(dw, t, k, m, x, n, y2)) and be.last_error == eb.INVALID_REQUEST
        assert be.free(dw)


# ------------------------------------------------------------------ device-side synthetic data
@pytest.mark.parametrize("t,tol", [(eb.Q4_K, 0.09), (eb.Q6_K, 0.03), (eb.Q8_0, 0.01), (eb.Q4_0, 0.13)])
def test_synth_encoders_emit_valid_blocks(be, port, t, tol):
    """Blocks encoded on the device decode (reference decoder) back to the f32 draw of the same seed."""
    k, m = 2048, 6
    fdev, qdev = be.alloc(4 * k * m), be.alloc(m * eb.row_bytes(t, k))
    assert be.synth_fill(fdev, eb.F32, k * m, 42, 0.02, 0) and be.synth_fill(qdev, t, k * m, 42, 0.02, 0) and be.sync()
    f = np.zeros((m, k), np.float32)
    q = np.zeros(m * eb.row_bytes(t, k), np.uint8)
    assert be.to_host(f, fdev) and be.to_host(q, qdev)
    assert abs(float(f.std()) - 0.02) < 0.002 and abs(float(f.mean())) < 0.001
    assert ob.rel_l2(port.dequantize(t, q, k, m), f) < tol
    assert be.free(fdev) and be.free(qdev)


@pytest.mark.parametrize("t", WEIGHT_TYPES)
def test_prepared_group_equals_single_products(be, port, t):
    """Q, K, V (or gate, up) against one prepared column in one launch: the same bits as one
    emelb_mul_mat_prepared per matrix; requests the grouped launch does not take fall back to those calls."""
    k, ms = 4096, (512, 128, 136)
    ws = [synth.encoded_weights(port, t, 700 + i, m, k) for i, m in enumerate(ms)]
    x = synth.activations_f32(710 + t, k, 1)
    bufs = [be.alloc(w.nbytes) for w in ws]
    xd, yd = be.alloc(4 * k), be.alloc(4 * sum(ms) * 2)
    try:
        for d, w in zip(bufs, ws):
            assert be.to_device(d, w)
        assert be.to_device(xd, x)
        offs = np.cumsum([0] + list(ms))
        single = [eb.mul_mat_op(d, t, k, m, xd, 1, yd + 4 * int(o)) for d, m, o in zip(bufs, ms, offs)]
        grouped = [eb.mul_mat_op(d, t, k, m, xd, 1, yd + 4 * int(sum(ms) + o)) for d, m, o in zip(bufs, ms, offs)]
        assert be.prepare_rhs(eb.dense_view(xd, eb.F32, [1, k]), t)
        for op in single:
            assert be.mul_mat_prepared(op), be.last_error
        l0 = be.diagnostics()["kernel_launches"]
        assert be.mul_mat_prepared_group(grouped), be.last_error
        assert be.diagnostics()["kernel_launches"] - l0 == 1
        assert be.mul_mat_prepared_group(grouped[:2]), be.last_error
        out = np.zeros(2 * sum(ms), np.float32)
        assert be.to_host(out, yd)
        assert np.array_equal(out[:sum(ms)].view(np.uint32), out[sum(ms):].view(np.uint32))
        # host outputs: not grouped, still right
        host = [np.zeros(m, np.float32) for m in ms]
        assert be.prepare_rhs(eb.dense_view(xd, eb.F32, [1, k]), t)
        assert be.mul_mat_prepared_group([eb.mul_mat_op(d, t, k, m, xd, 1, h) for d, m, h in zip(bufs, ms, host)])
        assert np.array_equal(np.concatenate(host).view(np.uint32), out[:sum(ms)].view(np.uint32))
        # without prepared planes the request is rejected like emelb_mul_mat_prepared rejects it
        assert be.mul_mat(single[0])
        assert not be.mul_mat_prepared_group(grouped)
    finally:
        for d in bufs + [xd, yd]:
            be.free(d)
