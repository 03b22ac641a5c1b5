"""Loader of the product library.  There is no fallback: without the built CUDA library
every operation of this package raises."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libaotx_q8_b200.so")
# AOTX_Q8_LIBRARY=trace loads the build of `python -m aotx_b200.build --trace` instead
# (development only: switches, time stamps, kernels the product build does not dispatch); any
# other value is taken as the path of a library with the same interface.
if os.environ.get("AOTX_Q8_LIBRARY") == "trace":
    LIB_PATH = os.path.join(HERE, "libaotx_q8_b200_trace.so")
elif os.environ.get("AOTX_Q8_LIBRARY"):
    LIB_PATH = os.path.abspath(os.environ["AOTX_Q8_LIBRARY"])

# every symbol include/aotx_q8_b200.h declares
SYMBOLS = (
    "aotx_q8_init", "aotx_q8_destroy", "aotx_q8_set_path", "aotx_q8_set_overlap", "aotx_q8_last_cuda_error",
    "aotx_q8_device_status", "aotx_q8_dequant", "aotx_q8_matmul", "aotx_q8_moe_route",
    "aotx_q8_moe_workspace_bytes", "aotx_q8_moe_ffn", "aotx_q8_moe_combine", "aotx_q8_matmul_static", "aotx_q8_static_status",
    "aotx_q8_matmul_peers",
    "aotx_q8_matmul_fused", "aotx_q8_moe_ffn_fused", "aotx_q8_peer_barrier", "aotx_q8_matmul_colsplit",
    "aotx_q8_moe_ep_workspace_bytes", "aotx_q8_moe_ep",
)

# every symbol include/aotx_gguf_b200.h declares
GGUF_SYMBOLS = (
    "aotx_gguf_open", "aotx_gguf_close", "aotx_gguf_file_bytes", "aotx_gguf_header_bytes",
    "aotx_gguf_data_bytes", "aotx_gguf_alignment", "aotx_gguf_tensor_count", "aotx_gguf_tensor",
    "aotx_gguf_find", "aotx_gguf_u32", "aotx_gguf_u64", "aotx_gguf_f32", "aotx_gguf_string",
    "aotx_gguf_array", "aotx_gguf_i32s", "aotx_gguf_f32s", "aotx_gguf_bools", "aotx_gguf_strings",
    "aotx_gguf_read", "aotx_gguf_read_threads", "aotx_gguf_row_bytes", "aotx_gguf_row_range",
    "aotx_gguf_loader_init", "aotx_gguf_loader_destroy", "aotx_gguf_loader_last_cuda_error",
    "aotx_gguf_upload", "aotx_gguf_upload_rows",
)


class TensorInfo(C.Structure):
    """aotx_gguf_tensor_info of include/aotx_gguf_b200.h."""
    _fields_ = [("name", C.c_char * 128), ("dim_count", C.c_uint32), ("type", C.c_uint32),
                ("dims", C.c_uint64 * 4), ("offset", C.c_uint64), ("bytes", C.c_uint64)]


class StringArray(C.Structure):
    """aotx_gguf_string_array of include/aotx_gguf_b200.h."""
    _fields_ = [("count", C.c_uint64), ("bytes", C.c_void_p), ("offsets", C.POINTER(C.c_uint64))]


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
    declare_q8(lib)
    declare_gguf(lib)
    _lib = lib
    return lib


def declare_q8(lib):
    """Argument and result types of every entry point of include/aotx_q8_b200.h."""
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
    lib.aotx_q8_moe_ep_workspace_bytes.restype = C.c_size_t
    lib.aotx_q8_moe_ffn.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, vp, vp, vp, u32, vp,
                                    u32, vp, i32, vp, C.c_size_t]
    lib.aotx_q8_moe_combine.argtypes = [vp, vp, vp, vp, vp, u32, vp, u32, u32, u32, vp, i32]
    lib.aotx_q8_matmul_static.argtypes = [vp, vp, u32, u32, u32, vp, i32, u32, vp, vp, i32]
    lib.aotx_q8_static_status.argtypes = [C.POINTER(C.c_uint32), i32]
    lib.aotx_q8_matmul_peers.argtypes = [vp, vp, vp, u32, u32, u32, vp, i32, u32, vp, C.POINTER(vp), u32,
                                         u32, u32, i32]
    lib.aotx_q8_peer_barrier.argtypes = [vp, vp, C.POINTER(vp), u32, u32, vp]
    lib.aotx_q8_matmul_colsplit.argtypes = [vp, vp, vp, u32, u32, u32, vp, i32, u32, vp, C.POINTER(vp), C.POINTER(vp),
                                            u32, u32, u32, u32, i32, vp]
    lib.aotx_q8_matmul_fused.argtypes = [vp, vp, vp, u32, u32, u32, vp, i32, u32, vp, vp, i32, i32]
    lib.aotx_q8_moe_ffn_fused.argtypes = [vp, vp, vp, vp, u32, u32, u32, u32, vp, vp, vp, u32, vp,
                                          u32, vp, i32, vp, C.c_size_t]
    lib.aotx_q8_moe_ep_workspace_bytes.argtypes = [u32, u32, u32, u32, u32]
    lib.aotx_q8_moe_ep.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, C.POINTER(vp), C.POINTER(vp), vp, u32, u32,
                                   C.POINTER(vp), C.POINTER(vp), u32, u32, vp, vp, i32, vp, C.c_size_t]
    for name in SYMBOLS:
        fn = getattr(lib, name)
        if name not in ("aotx_q8_moe_workspace_bytes", "aotx_q8_moe_ep_workspace_bytes"):
            fn.restype = i32


def declare_gguf(lib):
    """Argument and result types of every entry point of include/aotx_gguf_b200.h."""
    vp, u32, i32 = C.c_void_p, C.c_uint32, C.c_int
    u64, info = C.c_uint64, C.POINTER(TensorInfo)
    lib.aotx_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    lib.aotx_gguf_close.argtypes = [vp]
    lib.aotx_gguf_close.restype = None
    for name in ("aotx_gguf_file_bytes", "aotx_gguf_header_bytes", "aotx_gguf_data_bytes",
                 "aotx_gguf_tensor_count"):
        getattr(lib, name).argtypes = [vp]
        getattr(lib, name).restype = u64
    lib.aotx_gguf_alignment.argtypes = [vp]
    lib.aotx_gguf_alignment.restype = u32
    lib.aotx_gguf_tensor.argtypes = [vp, u64, info]
    lib.aotx_gguf_find.argtypes = [vp, C.c_char_p, info]
    lib.aotx_gguf_u32.argtypes = [vp, C.c_char_p, C.POINTER(u32)]
    lib.aotx_gguf_u64.argtypes = [vp, C.c_char_p, C.POINTER(u64)]
    lib.aotx_gguf_f32.argtypes = [vp, C.c_char_p, C.POINTER(C.c_float)]
    lib.aotx_gguf_string.argtypes = [vp, C.c_char_p, C.POINTER(vp), C.POINTER(C.c_size_t)]
    lib.aotx_gguf_array.argtypes = [vp, C.c_char_p, C.POINTER(u32), C.POINTER(u64)]
    lib.aotx_gguf_i32s.argtypes = [vp, C.c_char_p, C.POINTER(vp), C.POINTER(u64)]
    lib.aotx_gguf_f32s.argtypes = [vp, C.c_char_p, C.POINTER(vp), C.POINTER(u64)]
    lib.aotx_gguf_bools.argtypes = [vp, C.c_char_p, C.POINTER(vp), C.POINTER(u64)]
    lib.aotx_gguf_strings.argtypes = [vp, C.c_char_p, C.POINTER(StringArray)]
    lib.aotx_gguf_read.argtypes = [vp, u64, u64, vp]
    lib.aotx_gguf_read_threads.argtypes = [vp, u64, u64, vp, u32]
    lib.aotx_gguf_row_bytes.argtypes = [u32, u64]
    lib.aotx_gguf_row_bytes.restype = u64
    lib.aotx_gguf_row_range.argtypes = [info, u64, u64, C.POINTER(u64), C.POINTER(u64)]
    lib.aotx_gguf_loader_init.argtypes = [C.POINTER(vp), i32, C.c_size_t]
    lib.aotx_gguf_loader_destroy.argtypes = [vp]
    lib.aotx_gguf_loader_last_cuda_error.argtypes = [vp]
    lib.aotx_gguf_upload.argtypes = [vp, vp, u64, u64, vp, vp]
    lib.aotx_gguf_upload_rows.argtypes = [vp, vp, u64, u64, u64, vp, u64, vp]
