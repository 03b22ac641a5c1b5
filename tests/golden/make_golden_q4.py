"""Writes tests/golden/reference_q4_0.npz: the reference's own Q4_0 fixtures and expectations
(tests/matrix_test.cu:347-428): the 96 x 256 dequantisation tensor (seed SEED + 1) with the
halves its host reading gives, and the 80 x 128 product tensor (seed SEED + 9) with its inputs
(seeds SEED + 16, + 17) and double products.  Generated through oracle/_ref (the reference's
sources, compiled unmodified).

    python tests/golden/make_golden_q4.py
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle.binding import SEED, Reference  # noqa: E402

Q4_0 = 2


def main():
    ref = Reference()
    if not ref.available:
        raise SystemExit("no reference tree: cannot generate")
    lib = ref.lib
    lib.ref_build_typed.restype = C.c_ulonglong
    lib.ref_build_typed.argtypes = [C.c_void_p, C.c_uint, C.c_uint, C.c_uint, C.c_ulonglong]
    lib.ref_weight_typed.restype = C.c_float
    lib.ref_weight_typed.argtypes = [C.c_void_p, C.c_uint, C.c_uint]
    lib.ref_product_typed.argtypes = [C.c_void_p, C.c_uint, C.c_uint, C.c_uint, C.c_void_p, C.c_uint, C.c_void_p]

    def build(n, k, seed):
        size = lib.ref_build_typed(None, Q4_0, n, k, seed)
        assert size == n * (k // 32) * 18
        out = np.zeros(size, np.uint8)
        lib.ref_build_typed(out.ctypes.data, Q4_0, n, k, seed)
        return out

    out = {}
    w = build(96, 256, SEED + 1)
    out["dequant_w"] = w
    stride = (256 // 32) * 18
    deq = np.zeros((96, 256), np.float32)
    for r in range(96):
        for j in range(256):
            deq[r, j] = lib.ref_weight_typed(w.ctypes.data + r * stride, Q4_0, j)
    out["dequant_want"] = deq.astype(np.float16).view(np.uint16)
    assert np.array_equal(out["dequant_want"].view(np.float16).astype(np.float32), deq)
    w = build(80, 128, SEED + 9)
    out["product_w"] = w
    for s, m in enumerate((1, 64)):
        x = ref.input(m, 128, SEED + 16 + s)
        want = np.zeros((m, 80), np.float64)
        lib.ref_product_typed(w.ctypes.data, Q4_0, 80, 128, x.ctypes.data, m, want.ctypes.data)
        out["product_x_m%d" % m] = x
        out["product_want_m%d" % m] = want
    np.savez_compressed(os.path.join(HERE, "reference_q4_0.npz"), **out)
    print("written")


if __name__ == "__main__":
    main()
