"""Random rows of every block type, and a host build of the product's decoder (test helpers)."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# type id -> (name, weights per block, bytes per block, byte offsets of the binary16 fields)
TYPES = {
    0: ("F32", 1, 4, ()), 1: ("F16", 1, 2, ()),
    2: ("Q4_0", 32, 18, (0,)), 3: ("Q4_1", 32, 20, (0, 2)), 6: ("Q5_0", 32, 22, (0,)), 7: ("Q5_1", 32, 24, (0, 2)),
    8: ("Q8_0", 32, 34, (0,)),
    10: ("Q2_K", 256, 84, (80, 82)), 11: ("Q3_K", 256, 110, (108,)), 12: ("Q4_K", 256, 144, (0, 2)),
    13: ("Q5_K", 256, 176, (0, 2)), 14: ("Q6_K", 256, 210, (208,)),
}
PACKED = [t for t in TYPES if t >= 2]


def row_bytes(kind, k):
    _, weights, size, _ = TYPES[kind]
    assert k % weights == 0
    return k // weights * size


def random_rows(kind, n, k, rng, subnormal_share=0.1):
    """n rows of k weights: random codes, finite binary16 scales (some of them subnormal, like
    the scales of real tensors), as one flat uint8 array."""
    _, weights, size, halves = TYPES[kind]
    if kind == 0:
        return rng.standard_normal(n * k).astype(np.float32).view(np.uint8).copy()
    if kind == 1:
        return (rng.standard_normal(n * k) * 0.05).astype(np.float16).view(np.uint8).copy()
    blocks = n * (k // weights)
    raw = rng.integers(0, 256, (blocks, size), dtype=np.uint8)
    for offset in halves:
        scale = np.abs(rng.standard_normal(blocks)) * 0.02 / 16.0
        tiny = rng.random(blocks) < subnormal_share
        scale = np.where(tiny, scale * 1e-3, scale).astype(np.float16)
        if offset in (2, 82):     # a minimum or offset may be negative in the affine legacy types
            scale = np.where(rng.random(blocks) < 0.5, scale, -scale).astype(np.float16) if kind in (3, 7) else scale
        raw[:, offset:offset + 2] = scale.view(np.uint8).reshape(blocks, 2)
    return raw.reshape(-1)


class HostDecoder:
    """aotx_b200/csrc/q_blocks.cuh compiled for the host (tests/blocks_host.cu)."""

    def __init__(self, build_dir):
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        path = os.path.join(str(build_dir), "libblocks_host.so")
        done = subprocess.run(
            [nvcc, "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fno-strict-aliasing", "-gencode",
             "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "aotx_b200", "csrc"), "-o", path,
             os.path.join(ROOT, "tests", "blocks_host.cu")], capture_output=True, text=True, timeout=900)
        assert done.returncode == 0, done.stderr[-2000:]
        lib = C.CDLL(path)
        lib.blocks_decode_run.argtypes = [C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p]
        lib.blocks_decode_run_half.argtypes = [C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p]
        lib.blocks_row_bytes.argtypes = [C.c_uint32, C.c_uint32]
        lib.blocks_row_bytes.restype = C.c_ulonglong
        self.lib = lib

    def rows(self, kind, w, n, k, half=False):
        """[n][k] float32 (or the binary16 bits the dequantisation writes)."""
        stride = row_bytes(kind, k)
        w = np.ascontiguousarray(w)
        out = np.empty((n, k), dtype=np.uint16 if half else np.float32)
        fn = self.lib.blocks_decode_run_half if half else self.lib.blocks_decode_run
        for r in range(n):
            row = w.ctypes.data + r * stride
            for run in range(k // 32):
                fn(kind, row, run, out[r, run * 32:].ctypes.data)
        return out
