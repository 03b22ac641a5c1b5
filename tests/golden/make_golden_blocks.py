"""Writes tests/golden/blocks.npz: a few random rows of every packed block type and, for each,
the doubles that the REFERENCE's host reading gives (tests/matrix_kref.h for the K types and the
Q4_1 / Q5 types; for Q8_0 and Q4_0, which that header does not cover, tests/matrix_test.cu's
aotx_test_weight before its rounding to half is the plain product d * q, formed here in double).

Run from the repository root where a reference tree is present:
    python tests/golden/make_golden_blocks.py
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import _blocks  # noqa: E402
from oracle import build  # noqa: E402


def main():
    lib = C.CDLL(build.build_kref(force=True))
    lib.kref_weight.restype = C.c_double
    lib.kref_weight.argtypes = [C.c_void_p, C.c_uint, C.c_uint]
    rng = np.random.default_rng(20240)
    out = {}
    n, k = 3, 512
    for kind in _blocks.PACKED:
        w = _blocks.random_rows(kind, n, k, rng)
        stride = _blocks.row_bytes(kind, k)
        want = np.empty((n, k))
        for r in range(n):
            for j in range(k):
                if kind in (2, 8):
                    block = w[r * stride + (j // 32) * (18 if kind == 2 else 34):]
                    d = float(block[:2].view(np.float16)[0])
                    if kind == 8:
                        q = int(block[2 + j % 32].view(np.int8))
                    else:
                        pair = int(block[2 + j % 16])
                        q = ((pair & 15) if j % 32 < 16 else (pair >> 4)) - 8
                    want[r, j] = d * q
                else:
                    want[r, j] = lib.kref_weight(w.ctypes.data + r * stride, kind, j)
        out["w%d" % kind] = w
        out["want%d" % kind] = want
    np.savez_compressed(os.path.join(HERE, "blocks.npz"), **out)
    print("written", sum(v.nbytes for v in out.values()), "bytes before compression")


if __name__ == "__main__":
    main()
