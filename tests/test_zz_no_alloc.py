"""The context-free entry point for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is off the table: their memory plan is fixed
before the first token, or they are a plug-in that receives a stream and buffers only.
aotx_q8_matmul_static serves them from a fixed array inside the library.  This test calls it
through the C ABI twice in a row for each shape (the array keeps the first call's leftovers, so
the second call checks that they do no harm) and compares each result with the ordinary entry
point and with the oracle; it covers half and bfloat16 activations, the live batch word, and a
shape that the general kernel serves.  The array's own status word must read zero afterwards."""
import ctypes as C

import numpy as np
import pytest

from _util import check_product, dev, dev_weights, torch_mod, x_bf16_bits, x_fp16

pytestmark = pytest.mark.gpu


def test_static_entry_matches_context_entry_and_oracle_twice(oracle):
    import aotx_b200
    torch = torch_mod()
    lib = aotx_b200.load_library()
    ctx = aotx_b200.Q8Context(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = C.c_uint32(7)
    # (n, k, rows of x, bfloat16 x, live batch or None); 80 x 128 has 136-byte rows: general kernel
    cases = ((4096, 4096, 32, False, None), (1000, 2048, 7, False, None), (4096, 4096, 32, True, 17),
             (28672, 4096, 8, True, None), (2304, 1024, 50, False, None), (80, 128, 5, False, 3))
    for n, k, m, bf16, live in cases:
        w_host = aotx_b200.synth_q8_0(n, k, 60 + m)
        w = dev_weights(w_host)
        m_dev = None if live is None else torch.tensor([live], dtype=torch.int32, device="cuda")
        rows = m if live is None else live
        for call in range(2):
            if bf16:
                x_t, bits = x_bf16_bits(m, k, 70 + call)
                x = x_t.cuda()
            else:
                x_host = x_fp16(m, k, 70 + call)
                x, bits = dev(x_host), x_host.view(np.uint16)
            want = ctx.matmul(w, n, k, x, m_dev=m_dev, y=torch.full((m, n), -1.0, dtype=torch.float32, device="cuda"))
            got = torch.full((m, n), -1.0, dtype=torch.float32, device="cuda")
            code = lib.aotx_q8_matmul_static(stream, w.data_ptr(), aotx_b200.Q8_0, n, k, x.data_ptr(),
                                             aotx_b200.BF16 if bf16 else aotx_b200.F16, m,
                                             m_dev.data_ptr() if m_dev is not None else None, got.data_ptr(),
                                             aotx_b200.F32)
            assert code == 0
            torch.cuda.synchronize()
            a, b = got.cpu().numpy(), want.cpu().numpy()
            # the tolerance of the product tests: 1e-2 * max|y| + 1e-3
            assert np.isfinite(a).all()
            assert np.abs(a - b).max() <= 1e-2 * np.abs(b).max() + 1e-3
            assert (a[rows:] == -1.0).all()
            check_product(oracle, w_host, n, k, np.ascontiguousarray(bits[:rows]), rows, a[:rows], bf16=bf16)
    # beyond the limit of the fixed scratch: refused, nothing written
    x = dev(x_fp16(65, 256, 1))
    w = dev_weights(aotx_b200.synth_q8_0(128, 256, 1))
    y = torch.full((65, 128), 5.0, dtype=torch.float32, device="cuda")
    code = lib.aotx_q8_matmul_static(stream, w.data_ptr(), aotx_b200.Q8_0, 128, 256, x.data_ptr(),
                                     aotx_b200.F16, 65, None, y.data_ptr(), aotx_b200.F32)
    assert code == 5
    torch.cuda.synchronize()
    assert (y == 5.0).all()
    # the fixed array's own status word, not the context's
    assert lib.aotx_q8_static_status(C.byref(status), 1) == 0
    assert status.value == 0
    assert ctx.device_status() == 0
    ctx.close()
