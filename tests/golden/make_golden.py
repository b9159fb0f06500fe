"""Generates tests/golden/int8_ref_cases.npz from the REFERENCE's own INT8 tile kernel.

Run in a container that has the reference checkout (its location: the ZENDNN_REFERENCE_ROOT variable):
    python tests/golden/make_golden.py
It builds oracle/_ref/libzendnn_ref.so from the reference sources (oracle/Makefile), runs the
reference kernel (u8 x s8 -> s32, per-tensor source scale and zero-point, per-tensor or
per-channel weight scale, f32 bias, fused activation, bf16 / f32 store) on seeded inputs and
stores inputs and outputs.  The fixtures travel with the repository; the reference does not.
Post-op codes follow the reference's fused_postop_t: 0 none, 1 relu, 2 gelu_tanh, 3 gelu_erf,
4 sigmoid, 5 swish, 6 tanh.  The reference kernel computes its activations with polynomial
approximations, so only the `none` and `relu` cases are bit-comparable; the others are stored
for tolerance checks.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

CASES = [
    # M, K, N, per_channel, bias, fused_op, dst
    (1, 64, 16, True, True, 0, "bf16"),
    (4, 128, 32, True, False, 1, "bf16"),
    (7, 100, 48, False, True, 0, "f32"),
    (16, 256, 64, True, True, 1, "bf16"),
    (33, 260, 80, True, True, 0, "bf16"),
    (128, 512, 128, True, True, 1, "bf16"),
    (19, 1024, 96, True, True, 2, "bf16"),
    (12, 384, 64, True, True, 5, "f32"),
    (24, 512, 64, True, True, 3, "bf16"),
    (10, 256, 48, True, True, 4, "bf16"),
    (15, 320, 80, True, False, 6, "bf16"),
    (9, 192, 32, False, True, 3, "f32"),
    (6, 448, 96, True, True, 4, "f32"),
    (21, 128, 64, True, True, 6, "f32"),
]


def main():
    O.build()
    assert O.ref_lib() is not None, "reference kernel unavailable (needs AVX-512 VNNI+BF16 and a reference checkout)"
    out = {}
    for i, (M, K, N, pc, hb, fo, dd) in enumerate(CASES):
        rng = np.random.default_rng(1000 + i)
        A = rng.integers(0, 256, (M, K), dtype=np.uint8)
        B = rng.integers(-127, 128, (K, N), dtype=np.int8)
        zp = int(rng.integers(0, 256))
        ss = np.float32(rng.uniform(0.005, 0.05))
        ws = rng.uniform(0.001, 0.01, N if pc else 1).astype(np.float32)
        bias = rng.normal(size=N).astype(np.float32) if hb else None
        ref = O.ref_int8_matmul(A, B, zp, ss, ws, bias, fo, dd)
        assert ref is not None
        p = "c%d_" % i
        out[p + "A"], out[p + "B"], out[p + "ws"], out[p + "out"] = A, B, ws, ref
        out[p + "meta"] = np.array([M, K, N, zp, fo, int(dd == "bf16"), int(hb)], dtype=np.int64)
        out[p + "ss"] = np.array([ss], dtype=np.float32)
        if hb:
            out[p + "bias"] = bias
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "int8_ref_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
