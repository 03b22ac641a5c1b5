"""The reference's spill gate, restated: its build requires that the kernels of this path keep
no stack frame and spill nothing (tools/spill-gate.py:103-112, which reads the resource usage of
aotx_model_gemm / gemv / dequant / product / line).  Here the same numbers come from what
`ptxas -v` reports while the library is built (the reference turns that report on as well,
CMakeLists.txt:66-67); nothing is disassembled."""
import pytest

from aotx_b200 import build as builder

# the kernels a product, a dequantisation or the routed-expert step launches on the shipped paths
HOT = ("q8_stream_kernel", "q8_dequant_kernel", "q8_route_kernel", "q8_group_build_kernel",
       "q8_gather_rows_kernel", "q8_collect_ids_kernel", "q8_swiglu_kernel", "q8_expert_sum_kernel",
       "q8_x_to_f16_kernel",
       "q_dequant_any_kernel")
# any-shape fallbacks (shapes the tensor-core kernels do not take), the prefill kernel, and the
# decode kernel for batches of up to 32 rows: its converter loop spills nothing; what it spills
# is in the once-per-tile path where the owner of a cut tile holds another block's 32 partial
# sums while it reads its own (two blocks of 80 registers share an SM)
SMALL_SPILLS = {"q8_gemv_simt_kernel": 32, "q8_gemv_simt_fused_kernel": 64, "q_gemv_any_kernel": 16,
                "q8_expert_feed_kernel": 64, "q8_expert_down_kernel": 64,
                "q8_wide_kernel": 16, "q8_decode_kernel": 256, "store_eight_any": 64, "store_four_any": 64, "store_eight_peers": 64,
                "mbar_wait": 0, "q8_peer_barrier_kernel": 0}


@pytest.fixture(scope="module")
def usage():
    builder.build()
    found = builder.resource_usage()
    assert found, "no ptxas reports beside the objects"
    return found


def test_hot_kernels_keep_no_stack_and_spill_nothing(usage):
    seen = set()
    for name, use in usage.items():
        for hot in HOT:
            if hot in name:
                seen.add(hot)
                assert use["stack"] == 0 and use["spill_stores"] == 0 and use["spill_loads"] == 0, (name, use)
    assert seen == set(HOT)


def test_every_other_kernel_is_listed_with_its_bound(usage):
    for name, use in usage.items():
        if any(hot in name for hot in HOT):
            continue
        bounds = [limit for other, limit in SMALL_SPILLS.items() if other in name]
        assert bounds, "a kernel the gate does not know: " + name
        assert use["spill_stores"] <= bounds[0], (name, use)


def test_register_budgets(usage):
    """One block of 480 threads per SM: at most 128 registers a thread (65536 / 480 rounded down
    to the allocation unit); the two-blocks-per-SM kernel: 352 threads twice, at most 80."""
    for name, use in usage.items():
        if "q8_stream_kernel" in name or "q8_wide_kernel" in name:
            assert use["registers"] <= 128, (name, use)
        if "q8_decode_kernel" in name:
            assert use["registers"] <= 80, (name, use)
