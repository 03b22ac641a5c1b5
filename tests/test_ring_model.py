"""The ring protocols of the two tensor-core kernels under random interleavings
(tests/ring_model.py).  Every stage setting the kernels are built with must be clean; a
setting that is known to be unsafe (two MMA stages under four steps per segment: a converter
half can run two phases ahead of the barrier it polls) must be caught, which shows the model
can see the kind of hazard it looks for."""
import pytest

import ring_model

# (raw_stages, depth) of StreamShape<NTOK> in aotx_b200/csrc/q8_stream.cu
STREAM_SETTINGS = [(5, 3), (3, 3), (2, 2)]
# (raw_stages, mma_stages, x_stages) of Shape<NTOK> in aotx_b200/csrc/q8_umma.cu
WIDE_SETTINGS = [(3, 4, 8), (3, 4, 6), (2, 4, 4), (2, 3, 3)]


@pytest.mark.parametrize("raw_stages,depth", STREAM_SETTINGS)
@pytest.mark.parametrize("bf16", [False, True])
def test_stream_kernel_rings(raw_stages, depth, bf16):
    for seed in range(40):
        assert ring_model.stream_kernel(seed, raw_stages, depth, segments=14, bf16=bf16) == []


@pytest.mark.parametrize("raw_stages,mma_stages,x_stages", WIDE_SETTINGS)
def test_wide_kernel_rings(raw_stages, mma_stages, x_stages):
    for seed in range(40):
        assert ring_model.wide_kernel(seed, raw_stages, mma_stages, x_stages, segments=10) == []


def test_model_catches_a_parity_alias():
    found = False
    for seed in range(40):
        if ring_model.wide_kernel(seed, 2, 2, 2, segments=10):
            found = True
            break
    assert found
