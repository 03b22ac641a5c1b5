"""A small GGUF (version 3) writer for the tests (test infrastructure).

Layout, from the published format description: magic "GGUF", u32 version, u64 tensor count,
u64 metadata count; metadata pairs (string key, u32 value type, value); tensor infos (string
name, u32 dimension count, u64 dimensions, u32 type, u64 offset from the start of the tensor
bytes); padding to the alignment; tensor bytes.  Strings are a u64 length and the bytes; an
array value is a u32 element type, a u64 count and the elements.  Everything little-endian.

The writer takes raw specifications so that the tests can also build files that are wrong on
purpose (counts that lie, bad types, offsets off the alignment)."""
import struct

U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)

_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B",
           U64: "<Q", I64: "<q", F64: "<d"}

# block type -> (weights per block, bytes per block)
LAYOUT = {0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34),
          10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210)}


def text(value):
    raw = value if isinstance(value, bytes) else value.encode()
    return struct.pack("<Q", len(raw)) + raw


def scalar(kind, value):
    return struct.pack(_SCALAR[kind], value)


def value_bytes(kind, value):
    """Encoded metadata value of type `kind`.  Arrays are (element kind, [elements])."""
    if kind == STRING:
        return text(value)
    if kind == ARRAY:
        element, items = value
        out = struct.pack("<IQ", element, len(items))
        for item in items:
            out += value_bytes(element, item)
        return out
    return scalar(kind, value)


def pair(key, kind, value):
    return text(key) + struct.pack("<I", kind) + value_bytes(kind, value)


def tensor_bytes(block_type, dims):
    weights = 1
    for d in dims:
        weights *= d
    per, size = LAYOUT[block_type]
    return weights // per * size


def tensor_info(name, dims, block_type, offset):
    out = text(name) + struct.pack("<I", len(dims))
    for d in dims:
        out += struct.pack("<Q", d)
    return out + struct.pack("<IQ", block_type, offset)


def build(meta, tensors, alignment=32, version=3, magic=b"GGUF", tensor_count=None, meta_count=None,
          declare_alignment=True, tail=b""):
    """meta: list of (key, kind, value).  tensors: list of dicts with name, dims, type and
    either `data` (bytes) or nothing (zeros of the natural size); optional `offset` overrides the
    placement.  Returns the file bytes and the list of (name, offset, size) as placed."""
    pairs = list(meta)
    if declare_alignment and alignment != 32:
        pairs.append(("general.alignment", U32, alignment))
    placed = []
    cursor = 0
    infos = b""
    blobs = []
    for t in tensors:
        size = len(t["data"]) if "data" in t else tensor_bytes(t["type"], t["dims"]) if t["type"] in LAYOUT else 0
        offset = t.get("offset", cursor)
        infos += tensor_info(t["name"], t["dims"], t["type"], offset)
        data = t.get("data", bytes(size))
        blobs.append((offset, data))
        placed.append((t["name"], offset, size))
        end = offset + size
        cursor = max(cursor, (end + alignment - 1) // alignment * alignment) if alignment else end
    head = magic + struct.pack("<I", version)
    head += struct.pack("<QQ", len(tensors) if tensor_count is None else tensor_count,
                        len(pairs) if meta_count is None else meta_count)
    for key, kind, value in pairs:
        head += pair(key, kind, value)
    head += infos
    pad = (-len(head)) % alignment if alignment else 0
    body = bytearray(max([0] + [o + len(d) for o, d in blobs]))
    for offset, data in blobs:
        body[offset:offset + len(data)] = data
    return head + bytes(pad) + bytes(body) + tail, placed
