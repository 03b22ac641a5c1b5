"""The context-free entry point for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is off the table: their memory plan is fixed
before the first token, or they are a plug-in that receives a stream and buffers only.
aotx_q8_matmul_static serves them from a fixed array inside the library.  This test calls it
through the C ABI twice in a row (the array keeps the first call's leftovers, so the second
call checks that they do no harm) and compares each result with the ordinary entry point."""
import ctypes as C

import numpy as np
import pytest

from _util import dev, dev_weights, torch_mod, x_fp16

pytestmark = pytest.mark.gpu


def test_static_entry_matches_context_entry_twice():
    import aotx_b200
    torch = torch_mod()
    lib = aotx_b200.load_library()
    ctx = aotx_b200.Q8Context(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for n, k, m in ((4096, 4096, 32), (1000, 2048, 7)):
        w = dev_weights(aotx_b200.synth_q8_0(n, k, 60 + m))
        for call in range(2):
            x = dev(x_fp16(m, k, 70 + call))
            want = ctx.matmul(w, n, k, x)
            got = torch.full((m, n), -1.0, dtype=torch.float32, device="cuda")
            code = lib.aotx_q8_matmul_static(stream, w.data_ptr(), aotx_b200.Q8_0, n, k, x.data_ptr(),
                                             aotx_b200.F16, m, None, got.data_ptr(), aotx_b200.F32)
            assert code == 0
            torch.cuda.synchronize()
            a, b = got.cpu().numpy(), want.cpu().numpy()
            # the tolerance of the product tests: 1e-2 * max|y| + 1e-3
            assert np.isfinite(a).all()
            assert np.abs(a - b).max() <= 1e-2 * np.abs(b).max() + 1e-3
    # beyond the limit of the fixed scratch: refused, nothing written
    x = dev(x_fp16(65, 256, 1))
    w = dev_weights(aotx_b200.synth_q8_0(128, 256, 1))
    y = torch.full((65, 128), 5.0, dtype=torch.float32, device="cuda")
    code = lib.aotx_q8_matmul_static(stream, w.data_ptr(), aotx_b200.Q8_0, 128, 256, x.data_ptr(),
                                     aotx_b200.F16, 65, None, y.data_ptr(), aotx_b200.F32)
    assert code == 5
    torch.cuda.synchronize()
    assert (y == 5.0).all()
    assert ctx.device_status() == 0
    ctx.close()
