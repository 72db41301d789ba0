"""Generates tests/golden/gguf_golden.npz: GGUF images, a list of deterministic
corruptions of them, and what the reference's loader answers for each, taken from
the reference's own probe_requirements / parse_bound_storage compiled in place
(oracle/_ref/libemel_ref.so, built by oracle/Makefile from a reference checkout).

Run from the repository root where the reference checkout is present:
    python tests/golden/make_gguf_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import bindings as ob          # noqa: E402
from emel_cpp_b200 import gguf_image as gi         # noqa: E402


def corruptions(image: bytes, head_bytes: int, stride: int):
    """(kind, position, value): kind 0 = keep the first `position` bytes; kind 1 = set byte `position`
    to `value`.  Truncations at every `stride`-th length (all lengths within the metadata) and four
    byte values at every metadata position."""
    out = [(0, n, 0) for n in range(0, head_bytes + 1)]
    out += [(0, n, 0) for n in range(head_bytes + 1, len(image), stride)] + [(0, len(image) - 1, 0)]
    for pos in range(head_bytes):
        b = image[pos]
        for v in sorted({0, 0xFF, b ^ 1, b ^ 0x80} - {b}):
            out.append((1, pos, v))
    return out


def apply(image: bytes, kind: int, pos: int, value: int) -> bytes:
    if kind == 0:
        return image[:pos]
    m = bytearray(image)
    m[pos] = value
    return bytes(m)


def main():
    ref = ob.ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libemel_ref.so is not built")
    images = {"valid": gi.reference_valid_file(), "rich": gi.rich_file(0)}
    out = {}
    for name, image in images.items():
        err, _kvs, tensors = ref.gguf_parse(image)
        assert err == 0
        head = min(t["file_offset"] for t in tensors)       # the data section starts at the first tensor
        specs = corruptions(image, head, 61)
        rows = np.zeros((len(specs), 9), np.uint64)
        for i, (kind, pos, value) in enumerate(specs):
            e, req = ref.gguf_probe(apply(image, kind, pos, value))
            rows[i] = (kind, pos, value, e, *req)
        out[name + "_image"] = np.frombuffer(image, np.uint8)
        out[name + "_cases"] = rows
        out[name + "_tensors"] = np.array([(t["type"], t["n_dims"], *t["dims"], t["data_offset"], t["file_offset"],
                                            t["data_size"]) for t in tensors], np.uint64)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "gguf_golden.npz"), **out)
    for k, v in out.items():
        print(k, v.shape)


if __name__ == "__main__":
    main()
