"""A stand-in for the device, for checking the GPU TESTS THEMSELVES on a machine without a GPU.

`pytest --fake-device -m gpu tests/test_gpu_X.py` runs the GPU tests with `Q8Context` replaced
by a class that computes every result on the CPU from the oracle (test infrastructure, never
the product: the product package still refuses to run without a device).  What this checks is
the test code - shapes, argument names, tolerances, guard handling, the error codes a test
expects - so that a test written while no GPU was at hand does not fail on its own mistakes
when it first meets one.  It says nothing about the kernels.
"""
import numpy as np
import torch as real_torch

class FakeCuda:
    @staticmethod
    def synchronize(*args, **kwargs):
        return None

    @staticmethod
    def is_available():
        return True

    @staticmethod
    def current_stream(*args, **kwargs):
        class Stream:
            cuda_stream = 0
        return Stream()


class FakeTorch:
    """torch with the device arguments taken out."""

    cuda = FakeCuda()

    def __getattr__(self, name):
        return getattr(real_torch, name)

    @staticmethod
    def _strip(kwargs):
        kwargs.pop("device", None)
        return kwargs

    def full(self, *args, **kwargs):
        return real_torch.full(*args, **self._strip(kwargs))

    def zeros(self, *args, **kwargs):
        return real_torch.zeros(*args, **self._strip(kwargs))

    def empty(self, *args, **kwargs):
        return real_torch.empty(*args, **self._strip(kwargs))

    def tensor(self, *args, **kwargs):
        return real_torch.tensor(*args, **self._strip(kwargs))


def _bits16(t):
    return t.contiguous().view(real_torch.int16).numpy().view(np.uint16)


class FakeContext:
    """The methods of aotx_b200.Q8Context that the tests use, on CPU tensors."""

    def __init__(self, device=0):
        from oracle.binding import Oracle
        from aotx_b200.q8 import Q8Error
        self.oracle = Oracle()
        self.Q8Error = Q8Error
        self.path = 0

    # -- housekeeping -------------------------------------------------------------------
    def close(self):
        pass

    def device_status(self, clear=True):
        return 0

    def set_path(self, path):
        if path not in (0, 1, 2):
            raise self.Q8Error(1)
        self.path = path

    def set_overlap(self, enabled):
        pass

    def _weights(self, kind, w, n, k):
        from aotx_b200.q8 import row_bytes
        w = w.numpy() if hasattr(w, "numpy") else np.asarray(w)
        if kind == 8:
            stride = row_bytes(k)
            return self.oracle.dequant(w[:n * stride], k, 0, n).view(np.float16).astype(np.float64)
        return self.oracle.block_rows(kind, w, k, 0, n)

    def _check_shape(self, kind, k):
        run = {0: 32, 1: 32, 2: 32, 3: 32, 6: 32, 7: 32, 8: 32, 10: 256, 11: 256, 12: 256, 13: 256, 14: 256}
        if kind not in run:
            raise self.Q8Error(2)
        if k == 0 or k % run[kind] != 0:
            raise self.Q8Error(1)

    def _live(self, m, m_dev):
        return m if m_dev is None else min(m, int(m_dev[0]))

    def _sums(self, kind, w, n, k, x, m):
        weights = self._weights(kind, w, n, k)
        return x[:m].double().numpy() @ weights.T

    # -- entry points -------------------------------------------------------------------
    def dequant(self, w, k, first_row, rows, out=None, type=8):
        self._check_shape(type, k)
        if out is None:
            out = real_torch.empty((rows, k), dtype=real_torch.float16)
        if type == 8:
            from aotx_b200.q8 import row_bytes
            bits = self.oracle.dequant(w.numpy()[:(first_row + rows) * row_bytes(k)], k, first_row, rows)
            values = bits.view(np.float16).reshape(rows, k)
        else:
            values = self.oracle.block_rows(type, w.numpy(), k, first_row, rows).astype(np.float32).astype(np.float16)
        out[:rows] = real_torch.from_numpy(values.copy())
        return out

    def matmul(self, w, n, k, x, m=None, m_dev=None, y=None, y_dtype=None, type=8):
        self._check_shape(type, k)
        if self.path == 2 and (type != 8 or k % 256 != 0):
            raise self.Q8Error(4)   # the forced tensor-core kernel cannot take it
        m = x.shape[0] if m is None else m
        if y is None:
            y = real_torch.empty((m, n), dtype=y_dtype or real_torch.float32)
        live = self._live(m, m_dev)
        if live:
            sums = self._sums(type, w, n, k, x, live).astype(np.float32)
            y[:live] = real_torch.from_numpy(sums).to(y.dtype)
        return y

    def matmul_fused(self, w, n, k, x, epilogue, m=None, m_dev=None, y=None, y_dtype=None, type=8):
        if epilogue == 0:
            return self.matmul(w, n, k, x, m=m, m_dev=m_dev, y=y, y_dtype=y_dtype, type=type)
        if type != 8:
            raise self.Q8Error(2)
        if epilogue not in (1, 2):
            raise self.Q8Error(1)
        m = x.shape[0] if m is None else m
        if y is None:
            if epilogue == 1:
                raise ValueError("EPILOGUE_ADD adds into a y that the caller gives")
            y = real_torch.empty((m, n // 2 if epilogue == 2 else n), dtype=y_dtype or real_torch.float32)
        if (epilogue == 1 and y.dtype != real_torch.float32) or (epilogue == 2 and n % 2):
            raise self.Q8Error(1)
        self._check_shape(type, k)
        live = self._live(m, m_dev)
        if not live:
            return y
        sums = real_torch.from_numpy(self._sums(8, w, n, k, x, live).astype(np.float32))
        if epilogue == 1:
            y[:live] = y[:live] + sums
        else:
            gate, up = sums[:, 0::2], sums[:, 1::2]
            y[:live] = ((gate / (1.0 + real_torch.exp(-gate))) * up).to(y.dtype)
        return y

    def moe_route(self, x, router, used, **kwargs):
        prob, ids = self.oracle.route(_bits16(x), router.numpy(), used)
        return (real_torch.from_numpy(prob.astype(np.float32)),
                real_torch.from_numpy(ids.view(np.int32).copy()))

    def moe_workspace(self, tokens, used, hidden, ffn):
        return real_torch.empty(256, dtype=real_torch.uint8)

    def _moe(self, wg, wu, wd, experts, hidden, ffn, x, prob, ids, tokens, out, out_dtype):
        tokens = x.shape[0] if tokens is None else tokens
        prob = prob.numpy()[:tokens].copy()
        ids = ids.numpy().view(np.uint32)[:tokens].copy()
        # a selection outside the expert table adds nothing: stand in an expert the token did
        # not select, with probability zero
        for t, r in zip(*np.nonzero(ids >= experts)):
            spare = min(set(range(experts)) - set(int(e) for e in ids[t] if e < experts))
            ids[t, r] = spare
            prob[t, spare] = 0.0
        want = self.oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, _bits16(x[:tokens]), prob, ids)
        if out is None:
            out = real_torch.empty((tokens, hidden), dtype=out_dtype or real_torch.float32)
        out[:tokens] = real_torch.from_numpy(np.asarray(want, np.float32)).to(out.dtype)
        return out

    def moe_ffn(self, w_gate, w_up, w_down, experts, hidden, ffn, x, prob, ids, tokens=None,
                tokens_dev=None, out=None, out_dtype=None, workspace=None, type=8):
        return self._moe(w_gate.numpy(), w_up.numpy(), w_down.numpy(), experts, hidden, ffn, x, prob, ids,
                         tokens, out, out_dtype)

    def moe_ffn_fused(self, w_gate_up, w_down, experts, hidden, ffn, x, prob, ids, tokens=None,
                      tokens_dev=None, out=None, out_dtype=None, workspace=None, type=8):
        from aotx_b200.q8 import row_bytes
        if hidden % 256 or ffn % 256:
            raise self.Q8Error(4)
        rows = w_gate_up.numpy().reshape(-1, row_bytes(hidden))
        gate = np.ascontiguousarray(rows[0::2]).reshape(-1)
        up = np.ascontiguousarray(rows[1::2]).reshape(-1)
        return self._moe(gate, up, w_down.numpy(), experts, hidden, ffn, x, prob, ids, tokens, out, out_dtype)


class FakeLoader:
    """aotx_b200.gguf.GGUFLoader with the upload done by a read into a CPU tensor."""

    def __init__(self, device=0, piece_bytes=0):
        self.piece = piece_bytes

    def close(self):
        pass

    def upload(self, gguf, offset, count, out=None):
        data = real_torch.from_numpy(gguf.read(offset, count))
        if out is None:
            return data
        out[:count] = data
        return out

    def upload_rows(self, gguf, tensor, first_row, rows, out=None):
        return self.upload(gguf, *gguf.row_range(tensor, first_row, rows), out=out)

    def upload_interleaved(self, gguf, gate, up, first_row=0, rows=None):
        from aotx_b200.gguf import row_bytes
        rows = gate.rows - first_row if rows is None else rows
        stride = row_bytes(gate.type, gate.row_weights)
        g = gguf.read_rows(gate, first_row, rows).reshape(rows, stride)
        u = gguf.read_rows(up, first_row, rows).reshape(rows, stride)
        out = np.empty((2 * rows, stride), np.uint8)
        out[0::2], out[1::2] = g, u
        return real_torch.from_numpy(out.reshape(-1))


def install():
    """Swap the device classes and helpers for the CPU stand-ins.  Called from conftest at
    configure time, before any test module is imported (they bind the helpers by name)."""
    import _util
    import aotx_b200
    import aotx_b200.gguf
    fake = FakeTorch()
    aotx_b200.Q8Context = FakeContext
    aotx_b200.gguf.GGUFLoader = FakeLoader
    _util.torch_mod = lambda: fake
    _util.dev = lambda array, device="cpu": real_torch.from_numpy(np.ascontiguousarray(array))
    _util.dev_weights = lambda w, device="cpu": real_torch.from_numpy(np.ascontiguousarray(w))
    real_torch.Tensor.cuda = lambda self, *a, **k: self
