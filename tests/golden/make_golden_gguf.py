"""Writes tests/golden/model_small.gguf (a small synthetic model file: a Q8_0 projection, a
stacked Q8_0 expert tensor, an F32 norm, an F16 table, one tensor of a block type without a
layout) and tests/golden/model_small.json = what the REFERENCE's reader
(disk/modelfile/gguf.c + meta.c, compiled unmodified by oracle/build.py) reports for it: the
sizes, every row of the tensor table with the byte sum of its data as read through the
reference's bounded read, and the result of every metadata getter for every key.

Run from the repository root where a reference tree is present:
    python tests/golden/make_golden_gguf.py
"""
import ctypes as C
import json
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import gguf_writer as gw  # noqa: E402
from oracle import build  # noqa: E402


class Info(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("dim_count", C.c_uint32), ("type", C.c_uint32),
                ("dims", C.c_uint64 * 4), ("offset", C.c_uint64), ("bytes", C.c_uint64)]


def main():
    import aotx_b200
    meta = [
        ("general.architecture", gw.STRING, "qwen3moe"),
        ("general.name", gw.STRING, "golden small"),
        ("general.alignment", gw.U32, 64),
        ("qwen3moe.block_count", gw.U32, 1),
        ("qwen3moe.embedding_length", gw.U64, 128),
        ("qwen3moe.expert_count", gw.I32, 3),
        ("qwen3moe.expert_used_count", gw.U8, 2),
        ("qwen3moe.expert_feed_forward_length", gw.U16, 64),
        ("qwen3moe.rope.freq_base", gw.F32, 1000000.0),
        ("qwen3moe.attention.layer_norm_rms_epsilon", gw.F64, 1e-6),
        ("qwen3moe.offset", gw.I64, -7),
        ("qwen3moe.flag", gw.BOOL, 0),
        ("tokenizer.ggml.tokens", gw.ARRAY, (gw.STRING, ["<s>", "a", "b"])),
        ("tokenizer.ggml.token_type", gw.ARRAY, (gw.I32, [3, 1, 1])),
    ]
    rng = np.random.default_rng(2024)
    tensors = [
        {"name": "blk.0.attn_q.weight", "dims": [128, 96], "type": 8,
         "data": aotx_b200.synth_q8_0(96, 128, 1).tobytes()},
        {"name": "blk.0.ffn_gate_exps.weight", "dims": [128, 64, 3], "type": 8,
         "data": aotx_b200.synth_q8_0(3 * 64, 128, 2).tobytes()},
        {"name": "blk.0.attn_norm.weight", "dims": [128], "type": 0,
         "data": rng.standard_normal(128).astype(np.float32).tobytes()},
        {"name": "token_embd.weight", "dims": [128, 3], "type": 1,
         "data": rng.standard_normal(384).astype(np.float16).tobytes()},
        {"name": "blk.0.other", "dims": [40], "type": 30, "data": bytes(range(40))},
    ]
    blob, _ = gw.build(meta, tensors, alignment=64, declare_alignment=False)
    path = os.path.join(HERE, "model_small.gguf")
    with open(path, "wb") as f:
        f.write(blob)

    lib = C.CDLL(build.build_gguf_ref(force=True))
    vp, u64 = C.c_void_p, C.c_uint64
    lib.aotx_modelfile_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    for name in ("file_bytes", "header_bytes", "data_bytes", "tensor_count"):
        fn = getattr(lib, "aotx_modelfile_" + name)
        fn.argtypes, fn.restype = [vp], u64
    lib.aotx_modelfile_tensor.argtypes = [vp, u64, C.POINTER(Info)]
    lib.aotx_modelfile_read.argtypes = [vp, u64, u64, vp]
    lib.aotx_modelfile_u32.argtypes = [vp, C.c_char_p, C.POINTER(C.c_uint32)]
    lib.aotx_modelfile_u64.argtypes = [vp, C.c_char_p, C.POINTER(u64)]
    lib.aotx_modelfile_f32.argtypes = [vp, C.c_char_p, C.POINTER(C.c_float)]
    lib.aotx_modelfile_string.argtypes = [vp, C.c_char_p, C.POINTER(vp), C.POINTER(C.c_size_t)]
    lib.aotx_modelfile_close.argtypes = [vp]
    handle = vp()
    assert lib.aotx_modelfile_open(path.encode(), C.byref(handle)) == 0
    out = {"sizes": [lib.aotx_modelfile_file_bytes(handle), lib.aotx_modelfile_header_bytes(handle),
                     lib.aotx_modelfile_data_bytes(handle)], "tensors": [], "meta": {}}
    for i in range(lib.aotx_modelfile_tensor_count(handle)):
        info = Info()
        assert lib.aotx_modelfile_tensor(handle, i, C.byref(info)) == 0
        data = np.zeros(info.bytes, np.uint8)
        assert lib.aotx_modelfile_read(handle, info.offset, info.bytes, data.ctypes.data) == 0
        out["tensors"].append([info.name.decode(), info.type, [info.dims[d] for d in range(info.dim_count)],
                               info.offset, info.bytes, int(data.astype(np.uint64).sum())])
    for key, _, _ in meta + [("absent.key", 0, 0)]:
        k = key.encode()
        a, b, c = C.c_uint32(), u64(), C.c_float()
        p, n = vp(), C.c_size_t()
        rc32 = lib.aotx_modelfile_u32(handle, k, C.byref(a))
        rc64 = lib.aotx_modelfile_u64(handle, k, C.byref(b))
        rcf = lib.aotx_modelfile_f32(handle, k, C.byref(c))
        rcs = lib.aotx_modelfile_string(handle, k, C.byref(p), C.byref(n))
        out["meta"][key] = [rc32, a.value, rc64, b.value, rcf, struct.pack("f", c.value).hex(),
                            rcs, C.string_at(p.value, n.value).hex() if rcs == 0 else ""]
    lib.aotx_modelfile_close(handle)
    with open(os.path.join(HERE, "model_small.json"), "w") as f:
        json.dump(out, f, indent=1)
    print(path, len(blob), "bytes")


if __name__ == "__main__":
    main()
