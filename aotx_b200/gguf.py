"""Host-side mirror of the model-file entry points (include/aotx_gguf_b200.h): open a GGUF
file, look tensors and metadata up, read or upload a tensor's rows.  ctypes on the product
library; PyTorch only supplies the device buffer and the stream of an upload."""
import ctypes as C

import numpy as np

from .library import TensorInfo, load_library

Q8_0 = 8


class GGUFError(RuntimeError):
    def __init__(self, call, code):
        super().__init__("%s failed with code %d" % (call, code))
        self.code = code


class Tensor:
    """One row of the tensor table."""

    def __init__(self, info):
        self.info = info
        self.name = info.name.decode("utf-8", "replace")
        self.type = int(info.type)
        self.dims = tuple(int(info.dims[d]) for d in range(int(info.dim_count)))
        self.offset = int(info.offset)
        self.bytes = int(info.bytes)

    @property
    def row_weights(self):
        return self.dims[0]

    @property
    def rows(self):
        total = 1
        for d in self.dims[1:]:
            total *= d
        return total

    def __repr__(self):
        return "Tensor(%r, type=%d, dims=%r, offset=%d, bytes=%d)" % (
            self.name, self.type, self.dims, self.offset, self.bytes)


class GGUFFile:
    def __init__(self, path):
        self.lib = load_library()
        handle = C.c_void_p()
        code = self.lib.aotx_gguf_open(str(path).encode(), C.byref(handle))
        if code != 0:
            raise GGUFError("aotx_gguf_open", code)
        self.handle = handle

    def close(self):
        if self.handle is not None:
            self.lib.aotx_gguf_close(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- sizes ----------------------------------------------------------------------------
    @property
    def file_bytes(self):
        return int(self.lib.aotx_gguf_file_bytes(self.handle))

    @property
    def header_bytes(self):
        return int(self.lib.aotx_gguf_header_bytes(self.handle))

    @property
    def data_bytes(self):
        return int(self.lib.aotx_gguf_data_bytes(self.handle))

    @property
    def alignment(self):
        return int(self.lib.aotx_gguf_alignment(self.handle))

    # -- tensor table ---------------------------------------------------------------------
    def __len__(self):
        return int(self.lib.aotx_gguf_tensor_count(self.handle))

    def tensor(self, index):
        info = TensorInfo()
        if self.lib.aotx_gguf_tensor(self.handle, index, C.byref(info)) != 0:
            raise IndexError(index)
        return Tensor(info)

    def find(self, name):
        info = TensorInfo()
        if self.lib.aotx_gguf_find(self.handle, name.encode(), C.byref(info)) != 0:
            raise KeyError(name)
        return Tensor(info)

    def tensors(self):
        return [self.tensor(i) for i in range(len(self))]

    # -- metadata -------------------------------------------------------------------------
    def _get(self, fn, key, holder):
        code = fn(self.handle, key.encode(), C.byref(holder))
        if code == 1:
            raise KeyError(key)
        if code != 0:
            raise TypeError("%s holds another type" % key)
        return holder.value

    def u32(self, key):
        return self._get(self.lib.aotx_gguf_u32, key, C.c_uint32())

    def u64(self, key):
        return self._get(self.lib.aotx_gguf_u64, key, C.c_uint64())

    def f32(self, key):
        return self._get(self.lib.aotx_gguf_f32, key, C.c_float())

    def string(self, key):
        value, length = C.c_void_p(), C.c_size_t()
        code = self.lib.aotx_gguf_string(self.handle, key.encode(), C.byref(value), C.byref(length))
        if code == 1:
            raise KeyError(key)
        if code != 0:
            raise TypeError("%s holds another type" % key)
        return C.string_at(value.value, length.value)

    def array(self, key):
        """(element type, count) of an array value."""
        kind, count = C.c_uint32(), C.c_uint64()
        code = self.lib.aotx_gguf_array(self.handle, key.encode(), C.byref(kind), C.byref(count))
        if code == 1:
            raise KeyError(key)
        if code != 0:
            raise TypeError("%s holds another type" % key)
        return int(kind.value), int(count.value)

    def _numbers(self, fn, key, dtype):
        values, count = C.c_void_p(), C.c_uint64()
        code = fn(self.handle, key.encode(), C.byref(values), C.byref(count))
        if code == 1:
            raise KeyError(key)
        if code != 0:
            raise TypeError("%s holds another type" % key)
        raw = C.string_at(values.value, count.value * np.dtype(dtype).itemsize)
        return np.frombuffer(raw, dtype=dtype).copy()

    def i32s(self, key):
        return self._numbers(self.lib.aotx_gguf_i32s, key, np.int32)

    def f32s(self, key):
        return self._numbers(self.lib.aotx_gguf_f32s, key, np.float32)

    def bools(self, key):
        return self._numbers(self.lib.aotx_gguf_bools, key, np.uint8).astype(bool)

    def strings(self, key):
        """The strings of an array value, as bytes objects."""
        from .library import StringArray
        array = StringArray()
        code = self.lib.aotx_gguf_strings(self.handle, key.encode(), C.byref(array))
        if code == 1:
            raise KeyError(key)
        if code != 0:
            raise TypeError("%s holds another type" % key)
        offsets = [array.offsets[i] for i in range(array.count + 1)]
        run = C.string_at(array.bytes, offsets[-1])
        return [run[offsets[i]:offsets[i + 1]] for i in range(array.count)]

    # -- bytes ----------------------------------------------------------------------------
    def read(self, offset, count, threads=1):
        out = np.empty(count, dtype=np.uint8)
        if threads > 1:
            code = self.lib.aotx_gguf_read_threads(self.handle, offset, count,
                                                   out.ctypes.data_as(C.c_void_p), threads)
        else:
            code = self.lib.aotx_gguf_read(self.handle, offset, count, out.ctypes.data_as(C.c_void_p))
        if code != 0:
            raise GGUFError("aotx_gguf_read", code)
        return out

    def row_range(self, tensor, first_row, rows):
        """(offset, bytes) of rows [first_row, first_row + rows) inside the tensor bytes."""
        offset, count = C.c_uint64(), C.c_uint64()
        if self.lib.aotx_gguf_row_range(C.byref(tensor.info), first_row, rows, C.byref(offset),
                                        C.byref(count)) != 0:
            raise ValueError("rows [%d, %d) are not in %s" % (first_row, first_row + rows, tensor.name))
        return int(offset.value), int(count.value)

    def read_rows(self, tensor, first_row, rows):
        return self.read(*self.row_range(tensor, first_row, rows))


def row_bytes(block_type, row_weights):
    return int(load_library().aotx_gguf_row_bytes(block_type, row_weights))


class GGUFLoader:
    """Two pinned buffers and their events on one device; uploads one byte range at a time."""

    def __init__(self, device=0, piece_bytes=0):
        self.lib = load_library()
        handle = C.c_void_p()
        code = self.lib.aotx_gguf_loader_init(C.byref(handle), device, piece_bytes)
        if code != 0:
            raise GGUFError("aotx_gguf_loader_init", code)
        self.handle = handle
        self.device = device

    def close(self):
        if self.handle is not None:
            self.lib.aotx_gguf_loader_destroy(self.handle)
            self.handle = None

    def upload(self, gguf, offset, count, out=None):
        """Bytes [offset, offset + count) of the tensor bytes as a uint8 device tensor, enqueued
        on the current stream."""
        import torch
        if out is None:
            out = torch.empty(count, dtype=torch.uint8, device=torch.device("cuda", self.device))
        stream = torch.cuda.current_stream(out.device).cuda_stream
        code = self.lib.aotx_gguf_upload(self.handle, gguf.handle, offset, count, out.data_ptr(), stream)
        if code != 0:
            raise GGUFError("aotx_gguf_upload (cuda error %d)"
                            % self.lib.aotx_gguf_loader_last_cuda_error(self.handle), code)
        return out

    def upload_rows(self, gguf, tensor, first_row, rows, out=None):
        """One rank's rows of a tensor: the shard of a column-split projection, or a range of
        experts of a stacked expert tensor."""
        return self.upload(gguf, *gguf.row_range(tensor, first_row, rows), out=out)

    def upload_interleaved(self, gguf, gate, up, first_row=0, rows=None):
        """Rows [first_row, first_row + rows) of two tensors of one shape as one device tensor
        with the rows interleaved (row 2r from `gate`, row 2r + 1 from `up`)."""
        import torch
        if gate.dims != up.dims or gate.type != up.type:
            raise ValueError("gate and up must have one shape and type")
        rows = gate.rows - first_row if rows is None else rows
        stride = row_bytes(gate.type, gate.row_weights)
        out = torch.empty(2 * rows * stride, dtype=torch.uint8, device=torch.device("cuda", self.device))
        stream = torch.cuda.current_stream(out.device).cuda_stream
        for which, tensor in enumerate((gate, up)):
            offset, _ = gguf.row_range(tensor, first_row, rows)
            code = self.lib.aotx_gguf_upload_rows(self.handle, gguf.handle, offset, stride, rows,
                                                  out.data_ptr() + which * stride, 2 * stride, stream)
            if code != 0:
                raise GGUFError("aotx_gguf_upload_rows (cuda error %d)"
                                % self.lib.aotx_gguf_loader_last_cuda_error(self.handle), code)
        return out
