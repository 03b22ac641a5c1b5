"""The GPU tests on a machine without a GPU, against the library's own code.

`pytest --emulated-device -m gpu tests/test_gpu_X.py` runs the GPU tests with `Q8Context` bound
to the library of tests/api_emu.cu - every source of the product library compiled as host code
around stand-ins for the hardware instructions, "device" memory being host memory - instead of
the CUDA build.  Where `--fake-device` (tests/_fake.py) answers from the oracle and so checks
only the tests, this runs the kernels and the host code that ship, a block as host threads, so
a GPU test that passes here has exercised the real argument checks, tensor maps, schedules,
dequantisation arithmetic and stores.  It is slow (a block of 480 threads per unit of work):
meant for the small and medium cases, one file at a time.  Test infrastructure only; the
product package still refuses to run without a device."""
import ctypes as C
import os
import shutil
import subprocess
import tempfile

import numpy as np
import torch as real_torch

import _fake

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_lib = None


def emulated_library():
    global _lib
    if _lib is not None:
        return _lib
    from aotx_b200 import library
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    path = os.path.join(tempfile.mkdtemp(prefix="aotx_emulated_"), "libapi_emu.so")
    done = subprocess.run([nvcc, "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fno-strict-aliasing", "-gencode",
                           "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "aotx_b200", "csrc"),
                           "-I", os.path.join(ROOT, "tests"), "-o", path, os.path.join(ROOT, "tests", "api_emu.cu")],
                          capture_output=True, text=True, timeout=1800)
    if done.returncode != 0:
        raise RuntimeError(done.stderr[-3000:])
    lib = C.CDLL(path)
    library.declare_q8(lib)
    lib.api_emu_status.restype = C.c_uint
    _lib = lib
    return lib


def install():
    import _util
    import aotx_b200
    import aotx_b200.gguf
    from aotx_b200 import q8

    class EmulatedContext(q8.Q8Context):
        """aotx_b200.Q8Context over the emulated library, on CPU tensors."""

        def __init__(self, device=0):
            self.lib = emulated_library()
            self.device = real_torch.device("cpu")
            handle = C.c_void_p()
            self._check(self.lib.aotx_q8_init(C.byref(handle), 0))
            self.handle = handle

        def _stream(self):
            return None

        def moe_workspace(self, tokens, used, hidden, ffn):
            # device allocations are 256-byte aligned; host ones need the slice
            size = self.lib.aotx_q8_moe_workspace_bytes(tokens, used, hidden, ffn)
            raw = real_torch.empty(size + 256, dtype=real_torch.uint8)
            skip = (-raw.data_ptr()) % 256
            return raw[skip:skip + size]

        def device_status(self, clear=True):
            # the emulation's own findings count as a device status too
            return super().device_status(clear) | self.lib.api_emu_status()

    fake = _fake.FakeTorch()
    aotx_b200.Q8Context = EmulatedContext
    q8.Q8Context = EmulatedContext
    aotx_b200.load_library = emulated_library      # tests that call the C ABI directly
    aotx_b200.gguf.GGUFLoader = _fake.FakeLoader
    _util.torch_mod = lambda: fake
    _util.dev = lambda array, device="cpu": real_torch.from_numpy(np.ascontiguousarray(array))
    _util.dev_weights = lambda w, device="cpu": real_torch.from_numpy(np.ascontiguousarray(w))
    real_torch.Tensor.cuda = lambda self, *a, **k: self
