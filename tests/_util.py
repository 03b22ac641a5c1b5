"""Shared helpers of the GPU parity tests (test code only)."""
import numpy as np

GUARD = -12345.0  # tests/expert_test.cu:16


def torch_mod():
    import torch
    return torch


def dev(array, device="cuda"):
    torch = torch_mod()
    return torch.from_numpy(np.ascontiguousarray(array)).to(device)


def dev_weights(w, device="cuda"):
    """Weights on the device at a 256-byte aligned address, as the reference places tensors
    (cuda/boot/weights_host.cu:22,172-173)."""
    torch = torch_mod()
    t = torch.empty(w.size + 256, dtype=torch.uint8, device=device)
    off = (-t.data_ptr()) % 256
    view = t[off:off + w.size]
    view.copy_(torch.from_numpy(np.ascontiguousarray(w)))
    return view


def x_fp16(m, k, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.standard_normal((m, k)).astype(np.float16)


def x_bf16_bits(m, k, seed):
    torch = torch_mod()
    rng = np.random.Generator(np.random.PCG64(seed))
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(torch.bfloat16)
    return x, x.view(torch.int16).numpy().view(np.uint16)


def check_product(oracle, w, n, k, x_bits, m, y, bf16=False, full_limit=6e9, spots=512):
    """Compare a device result with the oracle: the whole product where that ends in seconds,
    else sampled entries.  Applies both the reference's own measure (<= 1e-2) and the bound
    max|err| <= 1e-2 * max|y_ref| + 1e-3."""
    y = np.asarray(y, np.float32)
    assert np.isfinite(y).all()
    if float(m) * n * k <= full_limit:
        want = oracle.product(w, n, k, x_bits, m, bf16=bf16)
        bad, worst = oracle.diff(y, want)
        ok, err, bound = oracle.within_bound(y, want)
        assert bad == 0, "reference measure: %d over 1e-2, worst %.3e" % (bad, worst)
        assert ok, "max err %.3e over bound %.3e" % (err, bound)
        return worst
    bad, worst = oracle.spot(w, n, k, x_bits, m, y, count=spots, bf16=bf16)
    assert bad == 0, "spot check: %d of %d over 1e-2, worst %.3e" % (bad, spots, worst)
    return worst


def device_synth_q8_0(n, k, seed):
    """Seeded synthetic Q8_0 rows in the benchmark's distribution, generated on the device."""
    import aotx_b200
    return aotx_b200.synth_q8_0_device(n, k, seed)


def check_columns(oracle, w_host, n, k, x_bits, m, y, bf16=True, columns=192, seed=77):
    """Whole columns of a large product against the oracle: `columns` sampled weight rows, every
    row of x.  Applies the reference's measure |err| / max(|want|, rms(want)) <= 1e-2
    (tests/matrix_test.cu:246-274) and the bound max|err| <= 1e-2 * max|y_ref| + 1e-3.  This is
    the check for products whose weights are rounded to bfloat16 (bfloat16 activations above
    128 rows): the reference's sampled measure (tests/matrix_test.cu:279-312) has a floor for
    small sums that assumes binary16 weights."""
    from oracle.binding import row_bytes
    rng = np.random.Generator(np.random.PCG64(seed))
    picks = np.sort(rng.permutation(n)[:min(columns, n)])
    stride = row_bytes(k)
    piece = np.concatenate([w_host[j * stride:(j + 1) * stride] for j in picks])
    want = oracle.product(piece, len(picks), k, x_bits, m, bf16=bf16)
    got = np.ascontiguousarray(np.asarray(y, np.float32)[:, picks])
    assert np.isfinite(got).all()
    bad, worst = oracle.diff(got, want)
    ok, err, bound = oracle.within_bound(got, want)
    assert bad == 0, "reference measure: %d over 1e-2, worst %.3e" % (bad, worst)
    assert ok, "max err %.3e over bound %.3e" % (err, bound)
    return worst
