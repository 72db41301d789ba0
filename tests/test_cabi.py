"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
public headers declare, and its pure-host entry points (request guards, row
slicing) agree with the oracle.  No compute call is made here."""
import ctypes as C
import glob
import os
import re

import numpy as np
import pytest

import emel_cpp_b200 as eb
from oracle import bindings as ob
from tests.test_oracle import guard_cases, flash_inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    names = []
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        names += re.findall(r"EMELB_API\s+\w+\s+(\w+)\s*\(", open(h).read())
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    lib = eb.lib()
    names = header_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/*.h but not exported"
    for n in eb.declared_symbols():
        assert n in names, f"{n} bound in python but not declared in include/*.h"


def test_no_cpu_fallback_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(eb.BackendError):
        eb.Backend(0)


def as_eb(op: ob.Op) -> eb.Op:
    out = eb.Op()
    C.memmove(C.byref(out), C.byref(op), C.sizeof(eb.Op))
    return out


def test_struct_layouts_match():
    assert C.sizeof(eb.Op) == C.sizeof(ob.Op) == 4 * 80 + 64 + 8 + 8
    assert C.sizeof(eb.View) == 80


def test_mul_mat_guard_matches_oracle(port):
    lib = eb.lib()
    checker = ob.ref() or port
    cases, _keep = guard_cases()
    for name, op in cases:
        got = lib.emelb_can_run(None, eb.OP_MUL_MAT, C.byref(as_eb(op))) == eb.OK
        assert got == checker.can_run(ob.OP_MUL_MAT, op), name


def test_flash_guard_matches_oracle(port):
    lib = eb.lib()
    checker = ob.ref() or port
    hd, heads, kvh, T, cap = 64, 8, 2, 40, 48
    q, k, v = flash_inputs(71, hd, heads, kvh, T, cap)
    dst = np.zeros((heads, hd), np.float32)
    mk = lambda **kw: ob.flash_op(q, k, v, dst, hd, heads, kvh, T, cap, **kw)
    ops = [mk(scale=0.125), mk(), mk(scale=0.125, masked_total=cap), mk(scale=0.125, masked_total=T - 1), mk(scale=-1.0)]
    bad = mk(scale=0.125)
    bad.src1.ne[2] = 0
    bad.src2.ne[2] = 0
    ops.append(bad)
    bad = mk(scale=0.125)
    bad.src0.ne[1] = 2
    bad.dst.ne[1] = 2
    ops.append(bad)
    bad = mk(scale=0.125)
    bad.src2.data = None
    ops.append(bad)
    for i, op in enumerate(ops):
        got = lib.emelb_can_run(None, eb.OP_FLASH_ATTN_EXT, C.byref(as_eb(op))) == eb.OK
        assert got == checker.can_run(ob.OP_FLASH_ATTN_EXT, op), i


def test_argmax_guard():
    lib = eb.lib()
    k, m = 512, 4
    w = np.zeros(m * eb.row_bytes(eb.Q4_K, k), np.uint8)
    x = np.zeros(k, np.float32)
    best, idx = np.zeros(1, np.float32), np.zeros(1, np.int32)
    op = eb.mul_mat_op(w, eb.Q4_K, k, m, x, 1, best, idx)
    assert lib.emelb_can_run(None, eb.OP_MUL_MAT_ARGMAX, C.byref(op)) == eb.OK
    op.index_out = None
    assert lib.emelb_can_run(None, eb.OP_MUL_MAT_ARGMAX, C.byref(op)) == eb.INVALID_REQUEST
    x2 = np.zeros((k, 2), np.float32)
    op = eb.mul_mat_op(w, eb.Q4_K, k, m, x2, 2, best, idx)
    assert lib.emelb_can_run(None, eb.OP_MUL_MAT_ARGMAX, C.byref(op)) == eb.INVALID_REQUEST
    assert lib.emelb_can_run(None, 99, C.byref(op)) == eb.UNSUPPORTED_OP


def test_prequantized_vector_guard():
    lib = eb.lib()
    k, m = 512, 4
    w = np.zeros(m * eb.row_bytes(eb.Q4_K, k), np.uint8)
    xq = np.zeros(eb.row_bytes(eb.Q8_K, k), np.uint8)
    y = np.zeros(m, np.float32)
    op = eb.mul_mat_op(w, eb.Q4_K, k, m, xq, 1, y, src1_type=eb.Q8_K)
    assert lib.emelb_can_run(None, eb.OP_MUL_MAT, C.byref(op)) == eb.OK
    op = eb.mul_mat_op(w, eb.Q4_K, k, m, xq, 1, y, src1_type=eb.Q8_0)   # wrong family for a K-quant
    assert lib.emelb_can_run(None, eb.OP_MUL_MAT, C.byref(op)) == eb.INVALID_REQUEST


def test_row_slice_matches_reference_arithmetic(port):
    """compute_fixed_row_slice / compute_sliced_mul_mat_event (kernel/matmul)."""
    k, m, n = 512, 37, 3
    w = np.zeros(m * eb.row_bytes(eb.Q8_0, k), np.uint8)
    x = np.zeros((k, n), np.float32)
    y = np.zeros((m, n), np.float32)
    op = eb.mul_mat_op(w, eb.Q8_0, k, m, x, n, y)
    for lanes in (2, 4, 8):
        covered = 0
        for lane in range(lanes):
            s, b, c = eb.row_slice(op, lane, lanes)
            assert (b, c) == port.row_slice(m, lane, lanes)
            assert s.src0.data == op.src0.data + b * op.src0.nb[1]
            assert s.dst.data == op.dst.data + b * 4 * n
            assert s.src0.ne[1] == c and s.dst.ne[1] == c and s.src0.nb[2] == c * op.src0.nb[1]
            if c:
                assert eb.lib().emelb_can_run(None, eb.OP_MUL_MAT, C.byref(s)) == eb.OK
            covered += c
        assert covered == m


def test_cuda_actor_adapter_compiles_against_reference_events():
    """emel::kernel::cuda::sm takes the reference's own event structs (needs the reference checkout)."""
    import subprocess
    import tempfile
    from oracle import bindings as ob
    ref = ob.REFERENCE_DIR
    if not os.path.isdir(os.path.join(ref, "src", "emel", "kernel")):
        pytest.skip("reference checkout not present")
    exe = os.path.join(tempfile.gettempdir(), "emelb_cuda_sm_check")
    subprocess.run(["g++", "-std=c++20", f"-I{ref}/src", f"-I{ref}/include", f"-I{ROOT}/include",
                    os.path.join(ROOT, "tests", "cuda_sm_check.cc"), "-o", exe, eb.LIB_PATH,
                    f"-Wl,-rpath,{os.path.dirname(eb.LIB_PATH)}"], check=True)
    out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    fields = dict(kv.split("=") for kv in out.split())
    assert fields["other"] == "0"
    import torch
    if torch.cuda.is_available():
        assert fields["engaged"] == "1" and fields["accepted"] == "1"
    else:
        assert fields["engaged"] == "0" and fields["accepted"] == "0"


def test_entry_points_refuse_null_contexts_without_a_gpu():
    """No compute without a GPU, but every newer entry point must answer a null context with
    invalid_request instead of touching it."""
    lib = eb.lib()
    op = eb.Op()
    assert lib.emelb_mul_mat_prepared_group(None, C.byref(op), 2) == eb.INVALID_REQUEST
    assert lib.emelb_flash_attn_batch(None, None, None, None, None, 64, 8, 2, 1, 0, 64, 0.125) == eb.INVALID_REQUEST
    from emel_cpp_b200 import gguf
    assert lib.emelb_gguf_upload_all(None, None, 0) == gguf.INVALID_REQUEST
    assert lib.emelb_gguf_upload(None, None, 0, 0, None) == gguf.INVALID_REQUEST
