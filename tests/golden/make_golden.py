"""Generates tests/golden/hot_path_golden.npz from the reference's own kernels.

Run where the reference checkout is present (it builds oracle/_ref from it):
    python tests/golden/make_golden.py
Inputs are seeded; outputs are what the reference's scalar route and AVX2 route
produce for the activation quantizers, the block dequantizers, op_mul_mat and
op_flash_attn_ext.  The file is small on purpose (it travels with the repo so
the CPU oracle stays pinned where the reference checkout does not exist).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import bindings as ob  # noqa: E402
from tests import synth  # noqa: E402


def main():
    ob.build()
    ref, port = ob.ref(), ob.port()
    assert ref is not None, "needs oracle/_ref (the reference checkout)"
    out = {}
    for t in (ob.Q8_K, ob.Q8_0):
        k, n = 1024, 3
        x = synth.activations_f32(100 + t, k, n)
        x[0:256, 0] = 0.0
        x[300, 1], x[400, 1] = 2.5, -2.5
        out[f"quant_x_{t}"] = x
        for col in range(n):
            out[f"quant_y_{t}_{col}"] = ref.quantize(t, x, k, n, col)
    for t in (ob.Q4_K, ob.Q6_K, ob.Q8_0, ob.Q4_0):
        k, m, n = 2048, 24, 2
        w = synth.encoded_weights(port, t, 200 + t, m, k)
        x = synth.activations_f32(300 + t, k, n)
        out[f"w_{t}"], out[f"x_{t}"] = w, x
        out[f"shape_{t}"] = np.array([k, m, n])
        out[f"deq_{t}"] = ref.dequantize(t, w, k, m)
        for route in ("scalar", "avx2"):
            y = np.zeros((m, n), np.float32)
            assert ref.mul_mat(ob.mul_mat_op(w, t, k, m, x, n, y), route=route)
            out[f"y_{route}_{t}"] = y
    hd, heads, kvh, T, cap = 128, 8, 2, 200, 208
    g = synth.rng(400)
    q = g.standard_normal((heads, hd), dtype=np.float32)
    kc = (g.standard_normal((kvh, cap, hd), dtype=np.float32) * 0.5).astype(np.float16).view(np.uint16)
    vc = g.standard_normal((kvh, cap, hd), dtype=np.float32).astype(np.float16).view(np.uint16)
    scale = np.float32(1.0 / np.sqrt(hd))
    out.update(flash_q=q, flash_k=kc, flash_v=vc, flash_scale=scale, flash_shape=np.array([hd, heads, kvh, T, cap]))
    for route in ("scalar", "avx2"):
        dst = np.zeros((heads, hd), np.float32)
        assert ref.flash_attn(ob.flash_op(q, kc, vc, dst, hd, heads, kvh, T, cap, scale=float(scale), masked_total=cap), route=route)
        out[f"flash_{route}"] = dst
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hot_path_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
