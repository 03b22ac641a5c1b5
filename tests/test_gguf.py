"""The model-file reader (include/aotx_gguf_b200.h, aotx_b200/csrc/gguf_table.cpp) against the
reference's own reader.

`oracle/_ref/libgguf_ref.so` is the reference's disk/modelfile/gguf.c and meta.c compiled
unmodified (oracle/build.py: build_gguf_ref).  Both readers open the same files - well formed
ones, files that are wrong in one named way, and files with random damage in the head - and
must agree on the return code of open and, where the file opens, on every size, every row of
the tensor table bit for bit, every metadata getter and every read.  Without the reference
library (no reference tree and no prebuilt copy) the comparison tests are skipped and the
golden file of tests/golden/ still pins the reader."""
import ctypes as C
import json
import os
import random
import struct

import numpy as np
import pytest

import gguf_writer as gw

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


class RefInfo(C.Structure):
    # aotx_tensor_info, disk/modelfile/modelfile.h:99-106
    _fields_ = [("name", C.c_char * 128), ("dim_count", C.c_uint32), ("type", C.c_uint32),
                ("dims", C.c_uint64 * 4), ("offset", C.c_uint64), ("bytes", C.c_uint64)]


class RefStrings(C.Structure):
    # aotx_string_array, disk/modelfile/modelfile.h:108-114
    _fields_ = [("count", C.c_uint64), ("bytes", C.c_void_p), ("offsets", C.POINTER(C.c_uint64))]


@pytest.fixture(scope="module")
def ref():
    from oracle import build
    path = build.build_gguf_ref()
    if path is None:
        pytest.skip("no reference reader library")
    lib = C.CDLL(path)
    vp, u64 = C.c_void_p, C.c_uint64
    lib.aotx_modelfile_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    lib.aotx_modelfile_close.argtypes = [vp]
    lib.aotx_modelfile_close.restype = None
    for name in ("file_bytes", "header_bytes", "data_bytes", "tensor_count"):
        fn = getattr(lib, "aotx_modelfile_" + name)
        fn.argtypes, fn.restype = [vp], u64
    lib.aotx_modelfile_tensor.argtypes = [vp, u64, C.POINTER(RefInfo)]
    lib.aotx_modelfile_find.argtypes = [vp, C.c_char_p, C.POINTER(RefInfo)]
    lib.aotx_modelfile_u32.argtypes = [vp, C.c_char_p, C.POINTER(C.c_uint32)]
    lib.aotx_modelfile_u64.argtypes = [vp, C.c_char_p, C.POINTER(u64)]
    lib.aotx_modelfile_f32.argtypes = [vp, C.c_char_p, C.POINTER(C.c_float)]
    lib.aotx_modelfile_string.argtypes = [vp, C.c_char_p, C.POINTER(vp), C.POINTER(C.c_size_t)]
    lib.aotx_modelfile_read.argtypes = [vp, u64, u64, vp]
    for name in ("i32s", "f32s", "bools"):
        getattr(lib, "aotx_modelfile_" + name).argtypes = [vp, C.c_char_p, C.POINTER(vp), C.POINTER(u64)]
    lib.aotx_modelfile_strings.argtypes = [vp, C.c_char_p, C.POINTER(RefStrings)]
    return lib


@pytest.fixture(scope="module")
def mine():
    from aotx_b200 import build
    build.build()
    from aotx_b200.library import load_library
    return load_library()


def open_both(ref, mine, path):
    r, m = C.c_void_p(), C.c_void_p()
    rc_ref = ref.aotx_modelfile_open(path.encode(), C.byref(r))
    rc_mine = mine.aotx_gguf_open(path.encode(), C.byref(m))
    return rc_ref, r, rc_mine, m


def close_both(ref, mine, r, m):
    if r.value:
        ref.aotx_modelfile_close(r)
    if m.value:
        mine.aotx_gguf_close(m)


def compare_open_files(ref, mine, r, m, keys):
    from aotx_b200.library import StringArray, TensorInfo
    assert mine.aotx_gguf_file_bytes(m) == ref.aotx_modelfile_file_bytes(r)
    assert mine.aotx_gguf_header_bytes(m) == ref.aotx_modelfile_header_bytes(r)
    assert mine.aotx_gguf_data_bytes(m) == ref.aotx_modelfile_data_bytes(r)
    count = ref.aotx_modelfile_tensor_count(r)
    assert mine.aotx_gguf_tensor_count(m) == count
    for i in range(count):
        a, b = RefInfo(), TensorInfo()
        assert ref.aotx_modelfile_tensor(r, i, C.byref(a)) == 0
        assert mine.aotx_gguf_tensor(m, i, C.byref(b)) == 0
        assert bytes(a) == bytes(b), a.name
        c = TensorInfo()
        assert mine.aotx_gguf_find(m, a.name, C.byref(c)) == 0 and bytes(c) == bytes(a)
    assert mine.aotx_gguf_tensor(m, count, C.byref(TensorInfo())) == 1
    for key in list(keys) + ["no.such.key"]:
        k = key.encode() if isinstance(key, str) else key
        a32, b32 = C.c_uint32(7), C.c_uint32(7)
        assert ref.aotx_modelfile_u32(r, k, C.byref(a32)) == mine.aotx_gguf_u32(m, k, C.byref(b32)), key
        assert a32.value == b32.value
        a64, b64 = C.c_uint64(7), C.c_uint64(7)
        assert ref.aotx_modelfile_u64(r, k, C.byref(a64)) == mine.aotx_gguf_u64(m, k, C.byref(b64)), key
        assert a64.value == b64.value
        af, bf = C.c_float(7), C.c_float(7)
        assert ref.aotx_modelfile_f32(r, k, C.byref(af)) == mine.aotx_gguf_f32(m, k, C.byref(bf)), key
        assert struct.pack("f", af.value) == struct.pack("f", bf.value)
        ap, bp, al, bl = C.c_void_p(), C.c_void_p(), C.c_size_t(), C.c_size_t()
        rc = ref.aotx_modelfile_string(r, k, C.byref(ap), C.byref(al))
        assert rc == mine.aotx_gguf_string(m, k, C.byref(bp), C.byref(bl)), key
        if rc == 0:
            assert C.string_at(ap.value, al.value) == C.string_at(bp.value, bl.value)
        for name, width in (("i32s", 4), ("f32s", 4), ("bools", 1)):
            ap, bp, ac, bc = C.c_void_p(), C.c_void_p(), C.c_uint64(99), C.c_uint64(99)
            rc = getattr(ref, "aotx_modelfile_" + name)(r, k, C.byref(ap), C.byref(ac))
            assert rc == getattr(mine, "aotx_gguf_" + name)(m, k, C.byref(bp), C.byref(bc)), (key, name)
            if rc == 0:
                assert ac.value == bc.value
                assert C.string_at(ap.value, ac.value * width) == C.string_at(bp.value, bc.value * width), (key, name)
        sa, sb = RefStrings(), StringArray()
        rc = ref.aotx_modelfile_strings(r, k, C.byref(sa))
        assert rc == mine.aotx_gguf_strings(m, k, C.byref(sb)), key
        if rc == 0:
            assert sa.count == sb.count
            assert [sa.offsets[i] for i in range(sa.count + 1)] == [sb.offsets[i] for i in range(sb.count + 1)]
            total = sa.offsets[sa.count]
            assert C.string_at(sa.bytes, total) == C.string_at(sb.bytes, total)


def sample_file(rng, alignment=32):
    """A well-formed file with every value type, several block types and real Q8_0 bytes."""
    meta = [
        ("general.architecture", gw.STRING, "llama"),
        ("general.name", gw.STRING, "synthetic é model"),
        ("llama.block_count", gw.U32, 2),
        ("llama.embedding_length", gw.U64, 256),
        ("llama.feed_forward_length", gw.I32, 512),
        ("llama.expert_count", gw.U8, 4),
        ("llama.expert_used_count", gw.I8, 2),
        ("llama.negative", gw.I16, -3),
        ("llama.wide", gw.U64, 1 << 40),
        ("llama.rope.freq_base", gw.F32, 10000.5),
        ("llama.attention.layer_norm_rms_epsilon", gw.F64, 1e-6),
        ("llama.flag", gw.BOOL, 1),
        ("llama.small", gw.U16, 65535),
        ("llama.signed_wide", gw.I64, -(1 << 50)),
        ("tokenizer.ggml.tokens", gw.ARRAY, (gw.STRING, ["a", "", "hello", "世界"])),
        ("tokenizer.ggml.token_type", gw.ARRAY, (gw.I32, [1, 2, 3, -4])),
        ("tokenizer.ggml.scores", gw.ARRAY, (gw.F32, [0.5, -1.25])),
        ("tokenizer.flags", gw.ARRAY, (gw.BOOL, [0, 1, 1])),
        ("tokenizer.bytes", gw.ARRAY, (gw.U8, list(range(9)))),
        ("tokenizer.wide", gw.ARRAY, (gw.U64, [1, 1 << 60])),
        ("empty.array", gw.ARRAY, (gw.F64, [])),
        ("", gw.U32, 5),
    ]
    tensors = []
    shapes = [("blk.0.attn_q.weight", [256, 384], 8), ("blk.0.ffn_gate_exps.weight", [256, 128, 4], 8),
              ("blk.0.attn_norm.weight", [256], 0), ("token_embd.weight", [256, 100], 1),
              ("blk.0.ffn_down.weight", [512, 256], 12), ("blk.1.q4", [64, 3, 2, 2], 2),
              ("blk.1.q6k", [256, 5], 14), ("blk.1.unknown", [100, 3], 30)]
    for name, dims, kind in shapes:
        size = gw.tensor_bytes(kind, dims) if kind in gw.LAYOUT else 0
        tensors.append({"name": name, "dims": dims, "type": kind,
                        "data": rng.integers(0, 256, size, dtype=np.uint8).tobytes()})
    blob, placed = gw.build(meta, tensors, alignment=alignment)
    return blob, placed, [m[0] for m in meta] + ["general.alignment"]


@pytest.mark.parametrize("alignment", [32, 64, 4096, 1])
def test_well_formed_files_read_the_same(ref, mine, tmp_path, alignment):
    rng = np.random.default_rng(alignment)
    blob, placed, keys = sample_file(rng, alignment)
    path = str(tmp_path / "model.gguf")
    open(path, "wb").write(blob)
    rc_ref, r, rc_mine, m = open_both(ref, mine, path)
    try:
        assert rc_ref == 0 and rc_mine == 0
        assert mine.aotx_gguf_alignment(m) == alignment
        compare_open_files(ref, mine, r, m, keys)
        data = mine.aotx_gguf_data_bytes(m)
        for offset, count in [(0, 0), (0, 1), (0, data), (data, 0), (17, 1000), (data - 5, 5)]:
            a, b = np.zeros(count + 1, np.uint8), np.zeros(count + 1, np.uint8)
            assert ref.aotx_modelfile_read(r, offset, count, a.ctypes.data) == 0
            assert mine.aotx_gguf_read(m, offset, count, b.ctypes.data) == 0
            assert np.array_equal(a, b)
        for offset, count in [(data, 1), (0, data + 1), (2 ** 63, 2 ** 63), (data + 1, 0)]:
            scratch = np.zeros(8, np.uint8)
            assert ref.aotx_modelfile_read(r, offset, count, scratch.ctypes.data) \
                == mine.aotx_gguf_read(m, offset, count, scratch.ctypes.data) != 0
    finally:
        close_both(ref, mine, r, m)


def damaged_files():
    """(label, file bytes): each wrong in one named way."""
    rng = np.random.default_rng(5)
    base_meta = [("general.architecture", gw.STRING, "llama"), ("a.count", gw.U32, 3)]
    base_tensors = [{"name": "w", "dims": [64, 4], "type": 8}, {"name": "v", "dims": [32], "type": 0}]
    good, _ = gw.build(base_meta, base_tensors)
    cases = [("good", good), ("empty", b""), ("three bytes", good[:3]), ("magic", b"GGUX" + good[4:]),
             ("version 2", gw.build(base_meta, base_tensors, version=2)[0]),
             ("version 4", gw.build(base_meta, base_tensors, version=4)[0]),
             ("tensor count lies", gw.build(base_meta, base_tensors, tensor_count=3)[0]),
             ("tensor count huge", gw.build(base_meta, base_tensors, tensor_count=1 << 40)[0]),
             ("meta count lies", gw.build(base_meta, base_tensors, meta_count=5)[0]),
             ("meta count huge", gw.build(base_meta, base_tensors, meta_count=1 << 62)[0]),
             ("fewer tensors than written", gw.build(base_meta, base_tensors, tensor_count=1)[0]),
             ("no tensors no meta", gw.build([], [])[0]),
             ("header only", gw.build([], [])[0][:24]),
             ("trailing bytes", gw.build(base_meta, base_tensors, tail=b"xyz")[0])]
    for cut in (8, 16, 24, 30, 60, len(good) - 300, len(good) - 1):
        cases.append(("cut at %d" % cut, good[:cut]))

    def with_meta(label, *pairs):
        cases.append((label, gw.build(list(pairs), base_tensors)[0]))

    with_meta("bool 2", ("flag", gw.BOOL, 2))
    cases.append(("value type 13", good.replace(struct.pack("<I", gw.U32) + struct.pack("<I", 3),
                                               struct.pack("<I", 13) + struct.pack("<I", 3), 1)))
    with_meta("array of arrays", ("k", gw.ARRAY, (gw.ARRAY, [])))
    with_meta("array unknown element", ("k", gw.ARRAY, (13, [])))
    with_meta("bool array 2", ("k", gw.ARRAY, (gw.BOOL, [0, 2])))
    with_meta("key too long", ("k" * 256, gw.U32, 1))
    with_meta("key longest", ("k" * 255, gw.U32, 1))
    with_meta("key with zero", (b"a\x00b", gw.U32, 1))
    with_meta("repeated key", ("k", gw.U32, 1), ("k", gw.U32, 2))
    with_meta("alignment 0", ("general.alignment", gw.U32, 0))
    with_meta("alignment 3", ("general.alignment", gw.U32, 3))
    with_meta("alignment 131072", ("general.alignment", gw.U32, 131072))
    with_meta("alignment as string", ("general.alignment", gw.STRING, "32"))
    with_meta("alignment as float", ("general.alignment", gw.F32, 32.0))
    with_meta("alignment negative", ("general.alignment", gw.I32, -32))
    with_meta("alignment as bool", ("general.alignment", gw.BOOL, 1))
    with_meta("alignment as u64 big", ("general.alignment", gw.U64, 1 << 33))
    with_meta("alignment i8 16", ("general.alignment", gw.I8, 16))
    with_meta("empty array", ("k", gw.ARRAY, (gw.U32, [])))
    lying = gw.text("k") + struct.pack("<I", gw.ARRAY) + struct.pack("<IQ", gw.U64, 1 << 22)
    cases.append(("array longer than file", b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + lying))
    lying = gw.text("k") + struct.pack("<I", gw.ARRAY) + struct.pack("<IQ", gw.STRING, 1 << 22)
    cases.append(("string array longer than file", b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + lying))
    lying = gw.text("k") + struct.pack("<I", gw.ARRAY) + struct.pack("<IQ", gw.U8, (8 << 20) + 1)
    cases.append(("array over the element limit", b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + lying + bytes(64)))
    cases.append(("string longer than file", b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 1 << 50)))

    def with_tensors(label, *tensors, **kw):
        cases.append((label, gw.build(base_meta, list(tensors), **kw)[0]))

    with_tensors("zero dimension", {"name": "w", "dims": [64, 0], "type": 8, "data": b""})
    with_tensors("five dimensions", {"name": "w", "dims": [32, 1, 1, 1, 1], "type": 8, "data": bytes(34)})
    with_tensors("no dimensions", {"name": "w", "dims": [], "type": 0, "data": bytes(4)})
    with_tensors("row not whole blocks", {"name": "w", "dims": [48, 2], "type": 8, "data": bytes(102)})
    with_tensors("k row not 256", {"name": "w", "dims": [128, 2], "type": 12, "data": bytes(144)})
    with_tensors("name too long", {"name": "n" * 128, "dims": [32], "type": 8})
    with_tensors("name longest", {"name": "n" * 127, "dims": [32], "type": 8})
    with_tensors("name empty", {"name": "", "dims": [32], "type": 8})
    with_tensors("name with zero", {"name": b"a\x00b", "dims": [32], "type": 8})
    with_tensors("repeated name", {"name": "w", "dims": [32], "type": 8}, {"name": "w", "dims": [32], "type": 8})
    with_tensors("offset off the alignment", {"name": "w", "dims": [32], "type": 8, "offset": 8})
    with_tensors("offset past the end", {"name": "w", "dims": [32], "type": 8, "offset": 1 << 20, "data": b""})
    with_tensors("tensor longer than data", {"name": "w", "dims": [32, 1000], "type": 8, "data": bytes(34)})
    with_tensors("overlapping tensors", {"name": "a", "dims": [32], "type": 8, "offset": 0},
                 {"name": "b", "dims": [32], "type": 8, "offset": 0})
    with_tensors("unknown type", {"name": "w", "dims": [10], "type": 99, "data": bytes(40)})
    with_tensors("huge dims", {"name": "w", "dims": [1 << 40, 1 << 40], "type": 0, "data": b""})
    with_tensors("huge dims one block", {"name": "w", "dims": [1 << 62, 2], "type": 0, "data": b""})
    with_tensors("weights times bytes overflow", {"name": "w", "dims": [1 << 62], "type": 0, "data": b""})
    with_tensors("aligned 64", {"name": "w", "dims": [32], "type": 8}, alignment=64)
    padded = gw.build(base_meta, [], alignment=4096)[0]
    cases.append(("padding only", padded))
    cases.append(("pad past the end", padded[:-100]))
    return cases


def test_damaged_files_get_the_same_verdict(ref, mine, tmp_path):
    seen = set()
    for label, blob in damaged_files():
        path = str(tmp_path / "case.gguf")
        open(path, "wb").write(blob)
        rc_ref, r, rc_mine, m = open_both(ref, mine, path)
        try:
            assert rc_ref == rc_mine, (label, rc_ref, rc_mine)
            seen.add(rc_ref)
            if rc_ref == 0:
                compare_open_files(ref, mine, r, m, ["general.architecture", "a.count", "k", "flag",
                                                     "general.alignment", "k" * 255])
        finally:
            close_both(ref, mine, r, m)
    assert seen == {0, 2}


def test_unreadable_paths_get_the_same_verdict(ref, mine, tmp_path):
    for path in (str(tmp_path / "absent.gguf"), str(tmp_path)):
        rc_ref, r, rc_mine, m = open_both(ref, mine, path)
        close_both(ref, mine, r, m)
        assert rc_ref == rc_mine == 1


def test_random_damage_in_the_head(ref, mine, tmp_path):
    """Flip, overwrite, insert and delete bytes in the head of a good file; whatever the reference
    reader says about the result, this reader says too."""
    rng = np.random.default_rng(11)
    blob, _, keys = sample_file(rng)
    head = 1400  # the head of the sample is a little longer than this
    rnd = random.Random(3)
    opened = 0
    rounds = 600
    for step in range(rounds):
        data = bytearray(blob)
        for _ in range(rnd.choice([1, 1, 1, 2, 4])):
            at = rnd.randrange(head)
            kind = rnd.randrange(5)
            if kind == 0:
                data[at] ^= 1 << rnd.randrange(8)
            elif kind == 1:
                data[at] = rnd.choice([0, 1, 2, 8, 9, 12, 13, 31, 32, 33, 127, 128, 255])
            elif kind == 2:
                data[at:at] = bytes([rnd.randrange(256)])
            elif kind == 3:
                del data[at]
            else:
                data[at:at + 8] = struct.pack("<Q", rnd.choice([0, 1, 5, 1 << 20, 1 << 32, (1 << 64) - 1]))
        path = str(tmp_path / "fuzz.gguf")
        open(path, "wb").write(bytes(data))
        rc_ref, r, rc_mine, m = open_both(ref, mine, path)
        try:
            assert rc_ref == rc_mine, (step, rc_ref, rc_mine)
            if rc_ref == 0:
                opened += 1
                compare_open_files(ref, mine, r, m, keys)
        finally:
            close_both(ref, mine, r, m)
    assert 0 < opened < rounds


def test_golden_file_without_the_reference(mine):
    """tests/golden/model_small.gguf and what the reference's reader reports for it
    (tests/golden/make_golden_gguf.py wrote both)."""
    from aotx_b200.gguf import GGUFFile
    want = json.load(open(os.path.join(GOLDEN, "model_small.json")))
    with GGUFFile(os.path.join(GOLDEN, "model_small.gguf")) as f:
        assert [f.file_bytes, f.header_bytes, f.data_bytes] == want["sizes"]
        assert len(f) == len(want["tensors"])
        for i, row in enumerate(want["tensors"]):
            t = f.tensor(i)
            assert [t.name, t.type, list(t.dims), t.offset, t.bytes] == row[:5]
            got = f.read(t.offset, t.bytes)
            assert int(got.astype(np.uint64).sum()) == row[5]
        for key, (rc32, v32, rc64, v64, rcf, vf, rcs, vs) in want["meta"].items():
            for fn, rc, value in ((f.u32, rc32, v32), (f.u64, rc64, v64)):
                if rc == 0:
                    assert fn(key) == value
                else:
                    with pytest.raises(KeyError if rc == 1 else TypeError):
                        fn(key)
            if rcf == 0:
                assert struct.pack("f", f.f32(key)) == bytes.fromhex(vf)
            if rcs == 0:
                assert f.string(key) == bytes.fromhex(vs)


def test_row_ranges_are_the_shards_of_a_column_split(mine, tmp_path):
    """Rows of a tensor are contiguous bytes: a rank's rows of a projection and a rank's experts
    of a stacked expert tensor are one range each, equal to what ColumnSplit computes."""
    import aotx_b200
    from aotx_b200.gguf import GGUFFile, row_bytes
    from aotx_b200.sharded import ColumnSplit, shard_rows
    n, k, experts, ffn = 100, 256, 6, 64
    w = aotx_b200.synth_q8_0(n, k, 3)
    stacked = aotx_b200.synth_q8_0(experts * ffn, k, 4)
    blob, _ = gw.build([("general.architecture", gw.STRING, "llama")],
                       [{"name": "output.weight", "dims": [k, n], "type": 8, "data": w.tobytes()},
                        {"name": "blk.0.ffn_gate_exps.weight", "dims": [k, ffn, experts], "type": 8,
                         "data": stacked.tobytes()}])
    path = str(tmp_path / "m.gguf")
    open(path, "wb").write(blob)
    assert row_bytes(8, k) == aotx_b200.row_bytes(k) and row_bytes(8, 48) == 0 and row_bytes(99, 32) == 0
    assert row_bytes(12, 256) == 144 and row_bytes(0, 7) == 28 and row_bytes(1, 7) == 14
    with GGUFFile(path) as f:
        t = f.find("output.weight")
        assert t.rows == n and t.row_weights == k
        for world in (1, 2, 3, 8):
            parts = []
            for rank in range(world):
                first, last = shard_rows(n, world, rank)
                offset, count = f.row_range(t, first, last - first)
                b0, b1 = ColumnSplit.shard_bytes(n, k, world, rank)
                assert (offset - t.offset, offset - t.offset + count) == (b0, b1)
                parts.append(f.read(offset, count))
            assert np.array_equal(np.concatenate(parts), w)
        e = f.find("blk.0.ffn_gate_exps.weight")
        assert e.rows == experts * ffn
        first, last = shard_rows(experts, 4, 1)
        got = f.read_rows(e, first * ffn, (last - first) * ffn)
        stride = aotx_b200.row_bytes(k)
        assert np.array_equal(got, stacked[first * ffn * stride:last * ffn * stride])
        for bad in ((n, 1), (0, n + 1), (2 ** 63, 2 ** 63)):
            with pytest.raises(ValueError):
                f.row_range(t, *bad)
        with pytest.raises(KeyError):
            f.find("absent")
        assert f.string("general.architecture") == b"llama"


def test_array_values_through_the_python_mirror(mine, tmp_path):
    from aotx_b200.gguf import GGUFFile
    blob, _, _ = sample_file(np.random.default_rng(3))
    path = str(tmp_path / "s.gguf")
    open(path, "wb").write(blob)
    with GGUFFile(path) as f:
        assert f.strings("tokenizer.ggml.tokens") == [b"a", b"", b"hello", "世界".encode()]
        assert f.i32s("tokenizer.ggml.token_type").tolist() == [1, 2, 3, -4]
        assert f.f32s("tokenizer.ggml.scores").tolist() == [0.5, -1.25]
        assert f.bools("tokenizer.flags").tolist() == [False, True, True]
        assert f.array("tokenizer.wide") == (gw.U64, 2)
        with pytest.raises(TypeError):
            f.i32s("tokenizer.wide")          # 64-bit elements do not come as int32
        with pytest.raises(TypeError):
            f.strings("llama.block_count")
        with pytest.raises(KeyError):
            f.f32s("absent")


def test_library_exports_every_declared_gguf_symbol(mine):
    import re
    header = open(os.path.join(ROOT, "include", "aotx_gguf_b200.h")).read()
    declared = set(re.findall(r"\b(aotx_gguf_[a-z0-9_]+)\s*\(", header))
    from aotx_b200.library import GGUF_SYMBOLS
    assert declared == set(GGUF_SYMBOLS)
    for name in declared:
        assert hasattr(mine, name), name


def test_upload_needs_a_device(mine):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from aotx_b200.gguf import GGUFError, GGUFLoader
    with pytest.raises(GGUFError) as info:
        GGUFLoader(0, 1 << 20)
    assert info.value.code == 3


def test_threaded_read_equals_plain_read(mine, tmp_path):
    """A range long enough to be cut into slices (4 MiB least) reads the same on 1, 3 and 8
    threads, at offsets and lengths that are not on any boundary."""
    from aotx_b200.gguf import GGUFError, GGUFFile
    rng = np.random.default_rng(8)
    payload = rng.integers(0, 256, 9 * (1 << 22) + 12345, dtype=np.uint8)
    pad = (-payload.size) % 4
    data = np.concatenate([payload, np.zeros(pad, np.uint8)])
    blob, _ = gw.build([], [{"name": "big", "dims": [data.size // 4], "type": 0, "data": data.tobytes()}])
    path = str(tmp_path / "big.gguf")
    open(path, "wb").write(blob)
    with GGUFFile(path) as f:
        t = f.find("big")
        assert t.bytes == data.size
        for offset, count in [(0, data.size), (1, data.size - 1), (4097, 5 * (1 << 22) + 3), (7, 100)]:
            want = data[offset:offset + count]
            for threads in (1, 3, 8):
                assert np.array_equal(f.read(t.offset + offset, count, threads=threads), want)
        with pytest.raises(GGUFError):
            f.read(t.offset + 1, f.data_bytes, threads=8)


def random_structure(rnd):
    """A random well-formed file: any value types, arrays of any element type, 0 to 12 tensors
    of any listed type (and a few ids without a layout), any legal alignment."""
    kinds = [gw.U8, gw.I8, gw.U16, gw.I16, gw.U32, gw.I32, gw.F32, gw.BOOL, gw.STRING, gw.U64, gw.I64, gw.F64]
    ranges = {gw.U8: (0, 255), gw.I8: (-128, 127), gw.U16: (0, 65535), gw.I16: (-32768, 32767),
              gw.U32: (0, 2 ** 32 - 1), gw.I32: (-2 ** 31, 2 ** 31 - 1), gw.U64: (0, 2 ** 64 - 1),
              gw.I64: (-2 ** 63, 2 ** 63 - 1)}

    def value(kind):
        if kind in ranges:
            low, high = ranges[kind]
            return rnd.choice([low, high, 0, 1, rnd.randint(low, high)])
        if kind in (gw.F32, gw.F64):
            return rnd.choice([0.0, -1.5, 1e-30, 3.0e38 if kind == gw.F32 else 1e300, rnd.random()])
        if kind == gw.BOOL:
            return rnd.randint(0, 1)
        return "".join(rnd.choice("abcxyz.é_0") for _ in range(rnd.randint(0, 12)))

    meta, keys = [], set()
    for _ in range(rnd.randint(0, 14)):
        key = ".".join("".join(rnd.choice("abcdefgh") for _ in range(rnd.randint(1, 6)))
                       for _ in range(rnd.randint(1, 3)))
        if key in keys:
            continue
        keys.add(key)
        if rnd.random() < 0.3:
            element = rnd.choice(kinds)
            meta.append((key, gw.ARRAY, (element, [value(element) for _ in range(rnd.randint(0, 6))])))
        else:
            kind = rnd.choice(kinds)
            meta.append((key, kind, value(kind)))
    alignment = rnd.choice([1, 2, 8, 32, 32, 64, 256, 65536])
    tensors, names = [], set()
    for _ in range(rnd.randint(0, 12)):
        name = "t" + "".join(rnd.choice("abc.0123") for _ in range(rnd.randint(1, 20)))
        if name in names:
            continue
        names.add(name)
        kind = rnd.choice(sorted(gw.LAYOUT) + [4, 9, 30])
        block = gw.LAYOUT.get(kind, (1, 0))[0]
        dims = [block * rnd.randint(1, 3)] + [rnd.randint(1, 4) for _ in range(rnd.randint(0, 3))]
        size = gw.tensor_bytes(kind, dims) if kind in gw.LAYOUT else rnd.randint(0, 64)
        tensors.append({"name": name, "dims": dims, "type": kind,
                        "data": bytes(rnd.getrandbits(8) for _ in range(size))})
    blob, _ = gw.build(meta, tensors, alignment=alignment)
    return blob, [m[0] for m in meta] + ["general.alignment"]


def test_random_well_formed_structures(ref, mine, tmp_path):
    rnd = random.Random(2024)
    path = str(tmp_path / "random.gguf")
    for _ in range(150):
        blob, keys = random_structure(rnd)
        open(path, "wb").write(blob)
        rc_ref, r, rc_mine, m = open_both(ref, mine, path)
        try:
            assert rc_ref == 0 and rc_mine == 0
            compare_open_files(ref, mine, r, m, keys)
        finally:
            close_both(ref, mine, r, m)


def test_upload_logic_dry_run(tmp_path):
    """aotx_b200/csrc/gguf_upload.cu built with tests/gguf_dry.h in front (the CUDA runtime calls
    become host calls) and driven like the GPU test drives the real one: byte ranges and row
    ranges through pieces smaller and larger than the range, the strided row copy that
    interleaves two tensors, and the refusals.  Checks the loader's host logic, not a GPU."""
    import shutil
    import subprocess
    import aotx_b200
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    path = str(tmp_path / "libgguf_dry.so")
    csrc = os.path.join(ROOT, "aotx_b200", "csrc")
    subprocess.run([nvcc, "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fno-strict-aliasing", "-diag-suppress", "174",
                    "-gencode", "arch=compute_100a,code=sm_100a", "-include",
                    os.path.join(ROOT, "tests", "gguf_dry.h"), "-o", path,
                    os.path.join(csrc, "gguf_table.cpp"), os.path.join(csrc, "gguf_upload.cu")],
                   check=True, timeout=900)
    lib = C.CDLL(path)
    vp, u64 = C.c_void_p, C.c_uint64
    lib.aotx_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    lib.aotx_gguf_close.argtypes = [vp]
    lib.aotx_gguf_find.argtypes = [vp, C.c_char_p, vp]
    lib.aotx_gguf_loader_init.argtypes = [C.POINTER(vp), C.c_int, C.c_size_t]
    lib.aotx_gguf_loader_destroy.argtypes = [vp]
    lib.aotx_gguf_upload.argtypes = [vp, vp, u64, u64, vp, vp]
    lib.aotx_gguf_upload_rows.argtypes = [vp, vp, u64, u64, u64, vp, u64, vp]
    lib.aotx_gguf_data_bytes.argtypes = [vp]
    lib.aotx_gguf_data_bytes.restype = u64

    k, n, ffn, experts = 512, 300, 40, 3
    stride = aotx_b200.row_bytes(k)
    w = aotx_b200.synth_q8_0(n, k, 51)
    gate = aotx_b200.synth_q8_0(experts * ffn, k, 52)
    up = aotx_b200.synth_q8_0(experts * ffn, k, 53)
    big = np.random.default_rng(54).integers(0, 256, 9 * (1 << 20) + 32, dtype=np.uint8)
    blob, placed = gw.build([], [{"name": "w", "dims": [k, n], "type": 8, "data": w.tobytes()},
                                 {"name": "g", "dims": [k, ffn, experts], "type": 8, "data": gate.tobytes()},
                                 {"name": "u", "dims": [k, ffn, experts], "type": 8, "data": up.tobytes()},
                                 {"name": "big", "dims": [big.size // 4], "type": 0, "data": big.tobytes()}])
    offsets = {name: offset for name, offset, _ in placed}
    file_path = str(tmp_path / "m.gguf")
    open(file_path, "wb").write(blob)
    handle = vp()
    assert lib.aotx_gguf_open(file_path.encode(), C.byref(handle)) == 0
    try:
        for piece in (1000, 4096, 1 << 20, 0):
            loader = vp()
            assert lib.aotx_gguf_loader_init(C.byref(loader), 0, piece) == 0
            try:
                # byte ranges: whole tensor, a shard, an odd range, nothing
                for offset, count in ((offsets["w"], w.size), (offsets["w"] + 7 * stride, 100 * stride),
                                      (offsets["w"] + 3, 12345), (offsets["big"], big.size), (0, 0)):
                    out = np.full(count + 8, 0xAB, np.uint8)
                    assert lib.aotx_gguf_upload(loader, handle, offset, count, out.ctypes.data, None) == 0
                    assert np.array_equal(out[:count], np.frombuffer(blob, np.uint8)[
                        len(blob) - lib.aotx_gguf_data_bytes(handle) + offset:][:count])
                    assert (out[count:] == 0xAB).all()
                # interleaved rows of two tensors (a piece must hold at least one row)
                both = np.full(2 * experts * ffn * stride + 16, 0xCD, np.uint8)
                for which, name in enumerate(("g", "u")):
                    code = lib.aotx_gguf_upload_rows(loader, handle, offsets[name], stride, experts * ffn,
                                                     both.ctypes.data + which * stride, 2 * stride, None)
                    assert code == (1 if 0 < piece < stride else 0)
                if not 0 < piece < stride:
                    assert np.array_equal(both[:-16], aotx_b200.interleave_rows(gate, up, k, groups=experts))
                    assert (both[-16:] == 0xCD).all()
                # refusals: past the end of the tensor bytes, pitch below the row
                data = lib.aotx_gguf_data_bytes(handle)
                scratch = np.zeros(64, np.uint8)
                assert lib.aotx_gguf_upload(loader, handle, data, 1, scratch.ctypes.data, None) == 2
                assert lib.aotx_gguf_upload_rows(loader, handle, 0, stride, 1, scratch.ctypes.data, stride - 1, None) == 1
                assert lib.aotx_gguf_upload_rows(loader, handle, data - stride, stride, 2, scratch.ctypes.data,
                                                 stride, None) == 2
            finally:
                lib.aotx_gguf_loader_destroy(loader)
    finally:
        lib.aotx_gguf_close(handle)
