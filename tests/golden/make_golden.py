"""Generate the golden fixtures of the Q8_0 path from the reference's own host functions.

Run where a reference tree is present (`python tests/golden/make_golden.py`).  It builds
`oracle/_ref/libaotx_ref.so` from the reference's unmodified sources and stores, in
`reference_host.npz` beside this file:

* the reference's fixture tensors and inputs for its dequant, product and turned-operand
  cases (tests/matrix_test.cu:347-468: shapes 96x256, 80x128, 64x64; seeds SEED+0, +8, +16,
  +17, +32, +33), byte for byte as its generator makes them;
* the reference's expected values for them: dequantised rows (aotx_test_weight) and the
  double-precision products (aotx_test_ref), plain and turned;
* its float->half conversion of a set of probe values, and its half->float of all 65536
  bit patterns;
* the first draws of its random generator.

The CPU tests compare the oracle restatement with these on any machine.
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle.binding import SEED, Reference, row_bytes  # noqa: E402


def main():
    ref = Reference()
    if not ref.available:
        raise SystemExit("no reference tree: cannot generate")
    out = {}
    # random generator
    state = C.c_uint64(SEED)
    out["next_draws"] = np.array([ref.lib.ref_next(C.byref(state)) for _ in range(16)], np.uint64)
    state = C.c_uint64(SEED)
    out["unit_draws"] = np.array([ref.lib.ref_unit(C.byref(state)) for _ in range(16)], np.float32)
    # half conversions
    rng = np.random.default_rng(7)
    probes = np.concatenate([
        rng.standard_normal(4096).astype(np.float32),
        (rng.standard_normal(4096) * 1e-5).astype(np.float32),
        (rng.standard_normal(2048) * 1e-7).astype(np.float32),
        (rng.standard_normal(1024) * 3e4).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0**-24, 2.0**-25,
                  2.0**-25 * 1.0000001, 3 * 2.0**-25, 6.1e-5, 6.103515625e-5, np.inf, -np.inf],
                 np.float32)])
    out["f2h_in"] = probes
    out["f2h_bits"] = np.array([ref.lib.ref_float_to_half_bits(float(v)) for v in probes], np.uint16)
    out["h2f_all"] = np.array([ref.lib.ref_half_bits_to_float(b) for b in range(65536)], np.float32)
    # dequant case, tests/matrix_test.cu:347-378
    w = ref.build(96, 256, SEED + 0)
    out["dequant_w"] = w
    deq = np.zeros((96, 256), np.float32)
    base = w.ctypes.data
    for r in range(96):
        for j in range(256):
            deq[r, j] = ref.lib.ref_weight(base + r * row_bytes(256), j)
    out["dequant_want"] = deq.astype(np.float16).view(np.uint16)
    assert np.array_equal(out["dequant_want"].view(np.float16).astype(np.float32), deq)
    # product case, tests/matrix_test.cu:382-428
    w = ref.build(80, 128, SEED + 8)
    out["product_w"] = w
    for s, m in enumerate((1, 64)):
        x = ref.input(m, 128, SEED + 16 + s)
        out["product_x_m%d" % m] = x
        out["product_want_m%d" % m] = ref.product(w, 80, 128, x, m)
    # turned operand, tests/matrix_test.cu:432-468
    w = ref.build(64, 64, SEED + 32)
    x = ref.input(64, 64, SEED + 33)
    out["turn_w"] = w
    out["turn_x"] = x
    out["turn_want"] = ref.product(w, 64, 64, x, 64)
    out["turn_want_swapped"] = ref.product(w, 64, 64, x, 64, swap=True)
    # the reference's own comparison applied to a perturbed result
    got = (out["turn_want"] * (1 + 3e-3)).astype(np.float32)
    bad, worst = ref.diff(got, out["turn_want"])
    out["diff_probe"] = np.array([bad, worst], np.float64)
    bad, worst = ref.spot(w, 64, 64, x, 64, got, 64)
    out["spot_probe"] = np.array([bad, worst], np.float64)
    np.savez_compressed(os.path.join(HERE, "reference_host.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_host.npz"))


if __name__ == "__main__":
    main()
