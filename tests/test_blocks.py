"""The decoder of the other block types (aotx_b200/csrc/q_blocks.cuh) on the CPU, against the
reference's own host readings: tests/matrix_kref.h (double, the eight packed types beyond Q8_0
and Q4_0) and aotx_test_weight of tests/matrix_test.cu (Q8_0, Q4_0, F16, F32), both compiled from
the reference tree into oracle/_ref.  The decoder source is the one the kernels compile, built
for the host by tests/blocks_host.cu.  The acceptance bound of the half values is the
reference's (tests/matrix_kcases.h:160-190): relative error at most 2^-10, or an absolute error
of at most one binary16 subnormal step."""
import ctypes as C
import os

import numpy as np
import pytest

import _blocks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "blocks.npz")


@pytest.fixture(scope="module")
def decoder(tmp_path_factory):
    return _blocks.HostDecoder(tmp_path_factory.mktemp("blocks"))


@pytest.fixture(scope="module")
def kref():
    from oracle import build
    path = build.build_kref()
    if path is None:
        pytest.skip("no reference host reading")
    lib = C.CDLL(path)
    lib.kref_weight.restype = C.c_double
    lib.kref_weight.argtypes = [C.c_void_p, C.c_uint, C.c_uint]
    lib.kref_row_bytes.restype = C.c_ulonglong
    lib.kref_row_bytes.argtypes = [C.c_uint, C.c_uint]
    return lib


def kref_rows(kref, kind, w, n, k):
    stride = _blocks.row_bytes(kind, k)
    out = np.empty((n, k))
    for r in range(n):
        row = w.ctypes.data + r * stride
        for j in range(k):
            out[r, j] = kref.kref_weight(row, kind, j)
    return out


def half_to_double(bits):
    return bits.view(np.float16).astype(np.float64)


@pytest.mark.parametrize("kind", [3, 6, 7, 10, 11, 12, 13, 14])
def test_packed_types_against_the_reference_reading(decoder, kref, kind):
    rng = np.random.default_rng(100 + kind)
    n, k = 6, 512
    w = _blocks.random_rows(kind, n, k, rng)
    assert kref.kref_row_bytes(kind, k) == _blocks.row_bytes(kind, k) == decoder.lib.blocks_row_bytes(kind, k)
    want = kref_rows(kref, kind, w, n, k)
    got = decoder.rows(kind, w, n, k).astype(np.float64)
    # the float value is the correctly rounded value of the real expression
    assert (np.abs(got - want) <= np.abs(want) * 2.0 ** -23 + 1e-45).all()
    halves = half_to_double(decoder.rows(kind, w, n, k, half=True))
    err = np.abs(halves - want)
    assert np.isfinite(halves).all()
    assert ((err <= np.abs(want) * 9.765625e-04) | (err <= 5.9604644775390625e-08)).all()
    assert np.abs(want).max() > 0


def test_every_byte_pattern_of_the_packed_codes(decoder, kref):
    """All 256 values in every code position of one block of each type (fixed scales)."""
    for kind in (3, 6, 7, 10, 11, 12, 13, 14):
        name, weights, size, halves = _blocks.TYPES[kind]
        rows = []
        for value in range(256):
            block = np.full(size, value, dtype=np.uint8)
            for offset in halves:
                block[offset:offset + 2] = np.array([0.0123 if offset in (0, 80, 108, 208) else 0.0071],
                                                    np.float16).view(np.uint8)
            rows.append(block)
        w = np.concatenate(rows)
        k = weights
        n = 256
        want = kref_rows(kref, kind, w, n, k)
        got = decoder.rows(kind, w, n, k).astype(np.float64)
        assert (np.abs(got - want) <= np.abs(want) * 2.0 ** -23 + 1e-45).all(), name


def test_q8_q4_f16_f32_are_bit_exact_with_the_reference_test_reading(decoder, reference):
    if not reference.available or not hasattr(reference.lib, "ref_weight_typed"):
        pytest.skip("no reference library with the typed reading")
    fn = reference.lib.ref_weight_typed
    fn.restype = C.c_float
    fn.argtypes = [C.c_void_p, C.c_uint, C.c_uint]
    rng = np.random.default_rng(7)
    for kind in (8, 2, 1, 0):
        n, k = 5, 256
        w = _blocks.random_rows(kind, n, k, rng, subnormal_share=0.3)
        stride = _blocks.row_bytes(kind, k)
        got = decoder.rows(kind, w, n, k, half=True)
        for r in range(n):
            for j in range(k):
                want = np.float32(fn(w.ctypes.data + r * stride, kind, j))
                if kind == 0:
                    # the reading returns the float itself; the dequantisation rounds it to half
                    want = np.float32(np.float16(want))
                assert got[r, j] == np.float16(want).view(np.uint16), (kind, r, j)


def test_golden_blocks_without_the_reference(decoder):
    """tests/golden/blocks.npz: rows of every packed type and the reference reading's doubles
    for them (tests/golden/make_golden_blocks.py)."""
    data = np.load(GOLDEN)
    for kind in _blocks.PACKED:
        w, want = data["w%d" % kind], data["want%d" % kind]
        n, k = want.shape
        got = decoder.rows(kind, w, n, k).astype(np.float64)
        assert (np.abs(got - want) <= np.abs(want) * 2.0 ** -23 + 1e-45).all(), kind


def test_row_bytes_and_unknown_types(decoder):
    for kind, (_, weights, size, _) in _blocks.TYPES.items():
        assert decoder.lib.blocks_row_bytes(kind, 512) == 512 // weights * size
    assert decoder.lib.blocks_row_bytes(12, 128) == 0      # not a whole super block
    assert decoder.lib.blocks_row_bytes(8, 48) == 0
    assert decoder.lib.blocks_row_bytes(4, 32) == 0        # no such type
    out = np.ones(32, np.float32)
    decoder.lib.blocks_decode_run(99, np.zeros(64, np.uint8).ctypes.data, 0, out.ctypes.data)
    assert (out == 0).all()


def test_reference_q4_0_fixtures(decoder):
    """The reference's own Q4_0 cases (tests/matrix_test.cu:347-428), from
    tests/golden/reference_q4_0.npz: its 96 x 256 tensor dequantises to its expected halves bit
    for bit, and the double product over the decoded 80 x 128 tensor is its expected product."""
    data = np.load(os.path.join(ROOT, "tests", "golden", "reference_q4_0.npz"))
    got = decoder.rows(2, data["dequant_w"], 96, 256, half=True)
    assert np.array_equal(got, data["dequant_want"])
    weights = half_to_double(decoder.rows(2, data["product_w"], 80, 128, half=True))
    for m in (1, 64):
        x = data["product_x_m%d" % m].view(np.float16).astype(np.float64).reshape(m, 128)
        want = data["product_want_m%d" % m]
        assert np.abs(x @ weights.T - want).max() <= 1e-9 * np.abs(want).max()


@pytest.mark.parametrize("kind", [3, 6, 7, 10, 11, 12, 13, 14])
def test_oracle_restatement_against_the_reference_reading(oracle, kref, kind):
    """oracle/blocks_oracle.c, the CPU restatement the GPU tests check against, gives the
    reference reading's doubles (same expressions in double: equal to the last bits)."""
    rng = np.random.default_rng(200 + kind)
    n, k = 4, 512
    w = _blocks.random_rows(kind, n, k, rng, subnormal_share=0.3)
    assert oracle.block_row_bytes(kind, k) == kref.kref_row_bytes(kind, k)
    want = kref_rows(kref, kind, w, n, k)
    got = oracle.block_rows(kind, w, k, 0, n)
    assert (np.abs(got - want) <= np.abs(want) * 4e-16).all()
    assert np.array_equal(oracle.block_rows(kind, w, k, 1, 2), got[1:3])


def test_oracle_restatement_of_the_plain_types(oracle, decoder):
    """Q8_0, Q4_0, F16, F32: value = d q (or the stored number); the host decoder's floats are
    exactly these doubles."""
    rng = np.random.default_rng(17)
    for kind in (8, 2, 1, 0):
        n, k = 3, 256
        w = _blocks.random_rows(kind, n, k, rng)
        want = oracle.block_rows(kind, w, k, 0, n)
        got = decoder.rows(kind, w, n, k).astype(np.float64)
        assert np.array_equal(got, want), kind
    for kind, k in ((12, 128), (8, 48), (4, 32), (99, 32)):
        assert oracle.block_row_bytes(kind, k) == 0


def test_oracle_restatement_against_golden(oracle):
    data = np.load(GOLDEN)
    for kind in _blocks.PACKED:
        w, want = data["w%d" % kind], data["want%d" % kind]
        n, k = want.shape
        got = oracle.block_rows(kind, w, k, 0, n)
        assert (np.abs(got - want) <= np.abs(want) * 4e-16).all(), kind
