"""Loader of the product library.  There is no fallback: without the built CUDA library
every operation of this package raises."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libaotx_q8_b200.so")

# every symbol include/aotx_q8_b200.h declares
SYMBOLS = (
    "aotx_q8_init", "aotx_q8_destroy", "aotx_q8_set_path", "aotx_q8_set_overlap", "aotx_q8_last_cuda_error",
    "aotx_q8_device_status", "aotx_q8_dequant", "aotx_q8_matmul", "aotx_q8_moe_route",
    "aotx_q8_moe_workspace_bytes", "aotx_q8_moe_ffn", "aotx_q8_moe_combine", "aotx_q8_matmul_static", "aotx_q8_matmul_peers",
)


class LibraryMissing(RuntimeError):
    pass


_lib = None


def load_library():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            "%s is not built; run `python -m aotx_b200.build` (needs nvcc). "
            "This package has no CPU or PyTorch fallback." % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    vp, u32, i32 = C.c_void_p, C.c_uint32, C.c_int
    lib.aotx_q8_init.argtypes = [C.POINTER(vp), i32]
    lib.aotx_q8_destroy.argtypes = [vp]
    lib.aotx_q8_set_path.argtypes = [vp, i32]
    lib.aotx_q8_set_overlap.argtypes = [vp, i32]
    lib.aotx_q8_last_cuda_error.argtypes = [vp]
    lib.aotx_q8_device_status.argtypes = [vp, C.POINTER(u32), i32]
    lib.aotx_q8_dequant.argtypes = [vp, vp, vp, u32, u32, u32, u32, vp]
    lib.aotx_q8_matmul.argtypes = [vp, vp, vp, u32, u32, u32, vp, i32, u32, vp, vp, i32]
    lib.aotx_q8_moe_route.argtypes = [vp, vp, vp, vp, u32, vp, u32, u32, u32, vp, vp]
    lib.aotx_q8_moe_workspace_bytes.argtypes = [u32, u32, u32, u32]
    lib.aotx_q8_moe_workspace_bytes.restype = C.c_size_t
    lib.aotx_q8_moe_ffn.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, vp, vp, vp, u32, vp,
                                    u32, vp, i32, vp, C.c_size_t]
    lib.aotx_q8_moe_combine.argtypes = [vp, vp, vp, vp, vp, u32, vp, u32, u32, u32, vp, i32]
    lib.aotx_q8_matmul_static.argtypes = [vp, vp, u32, u32, u32, vp, i32, u32, vp, vp, i32]
    lib.aotx_q8_matmul_peers.argtypes = [vp, vp, vp, u32, u32, u32, vp, i32, u32, vp, C.POINTER(vp), u32,
                                         u32, u32, i32]
    for name in SYMBOLS:
        fn = getattr(lib, name)
        if name != "aotx_q8_moe_workspace_bytes":
            fn.restype = i32
    _lib = lib
    return lib
