"""aotx_b200 - B200-native Q8_0 weight-matrix path behind AOTX's kernel-call seam.

The compute lives in `libaotx_q8_b200.so` (hand-written CUDA for sm_100a, C ABI declared in
`include/aotx_q8_b200.h`).  This package is the host-side mirror of the reference's
interface for that path; PyTorch supplies device memory and streams only.
"""
from .library import LibraryMissing, load_library  # noqa: F401
from .q8 import (  # noqa: F401
    BF16, EPILOGUE_ADD, EPILOGUE_STORE, EPILOGUE_SWIGLU, F16, F32, PATH_AUTO, PATH_GENERAL, PATH_TENSOR,
    Q8_0, Q8Context, Q8Error, interleave_rows, pack_q8_0, row_bytes, synth_q8_0, synth_q8_0_device,
    unpack_q8_0,
)
