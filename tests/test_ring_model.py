"""The ring protocol of the one-block-per-SM decode-regime kernel under random interleavings
(tests/ring_model.py).  Every stage setting the kernel is built with must be clean."""
import pytest

import ring_model

# (raw_stages, depth) of StreamShape<NTOK> in aotx_b200/csrc/q8_stream.cu
STREAM_SETTINGS = [(5, 3), (3, 3), (2, 2)]


@pytest.mark.parametrize("raw_stages,depth", STREAM_SETTINGS)
@pytest.mark.parametrize("bf16", [False, True])
def test_stream_kernel_rings(raw_stages, depth, bf16):
    for seed in range(40):
        assert ring_model.stream_kernel(seed, raw_stages, depth, segments=14, bf16=bf16) == []
