"""Host-side mirror of the reference's matrix interface for the Q8_0 path.

Names follow the reference: a weight tensor is `w[n][k]` in 34-byte blocks, activations are
rows of `x[m][k]`, the result is `y[m][n]` (cuda/model/model.cuh:97-116).  Every method
enqueues on the current CUDA stream of PyTorch and returns without synchronising.
"""
import ctypes as C

import numpy as np

from .library import load_library

Q8_0 = 8  # cuda/model/model.cuh:31
F32, F16, BF16 = 0, 1, 2
PATH_AUTO, PATH_GENERAL, PATH_TENSOR = 0, 1, 2
EPILOGUE_STORE, EPILOGUE_ADD, EPILOGUE_SWIGLU = 0, 1, 2

_ERRORS = {1: "bad argument", 2: "block type without a layout, or not served by this entry point", 3: "CUDA call failed",
           4: "shape unsupported by the forced kernel family", 5: "workspace missing or small",
           6: "a device-side wait ran out"}


class Q8Error(RuntimeError):
    def __init__(self, code, detail=""):
        self.code = code
        super().__init__("aotx_q8 error %d (%s)%s" % (code, _ERRORS.get(code, "?"), detail))


def row_bytes(k):
    """Bytes of one row of k weights (cuda/model/matrix.cuh:77-82)."""
    return (k // 32) * 34


def interleave_rows(w_gate, w_up, k, groups=1):
    """Gate and up tensors of the same shape as one tensor with rows interleaved (row 2r = gate
    row r, row 2r + 1 = up row r), the layout EPILOGUE_SWIGLU and `moe_ffn_fused` read.  Rows are
    whole runs of row_bytes(k) bytes, so this is a strided byte copy; `groups` experts stacked in
    each tensor keep their order."""
    stride = row_bytes(k)
    gate = np.ascontiguousarray(w_gate).reshape(-1, stride)
    up = np.ascontiguousarray(w_up).reshape(-1, stride)
    if gate.shape != up.shape or gate.shape[0] % groups != 0:
        raise ValueError("gate and up must hold the same rows")
    out = np.empty((2 * gate.shape[0], stride), dtype=np.uint8)
    out[0::2] = gate
    out[1::2] = up
    return out.reshape(-1)


def pack_q8_0(q, d):
    """q: int8 [n][k], d: float16 [n][k/32] -> uint8 [n * row_bytes(k)] in the file layout."""
    n, k = q.shape
    out = np.empty((n, k // 32, 34), np.uint8)
    out[..., :2] = np.ascontiguousarray(d, np.float16).view(np.uint8).reshape(n, k // 32, 2)
    out[..., 2:] = np.ascontiguousarray(q, np.int8).view(np.uint8).reshape(n, k // 32, 32)
    return out.reshape(-1)


def unpack_q8_0(w, n, k):
    blocks = np.asarray(w, np.uint8).reshape(n, k // 32, 34)
    d = np.ascontiguousarray(blocks[..., :2]).view(np.float16).reshape(n, k // 32)
    q = np.ascontiguousarray(blocks[..., 2:]).view(np.int8).reshape(n, k)
    return q, d


def synth_q8_0(n, k, seed):
    """Synthetic weights in the benchmark's distribution: q uniform in [-127, 127], one scale
    per 32 weights = half(|N(0, 0.02)| / 127) (about 30 % of them half subnormals)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    q = rng.integers(-127, 128, (n, k), dtype=np.int8)
    d = (np.abs(rng.normal(0.0, 0.02, (n, k // 32))) / 127.0).astype(np.float16)
    return pack_q8_0(q, d)


def _torch():
    import torch
    return torch


def synth_q8_0_device(n, k, seed, device="cuda"):
    """The same distribution generated on the device (the large tensors of the sharded
    configurations take seconds there and minutes on the host); a different stream of numbers
    from `synth_q8_0`.  Returns a uint8 device tensor of n * (k / 32) * 34 bytes at a 256-byte
    aligned address."""
    torch = _torch()
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    blocks = k // 32
    t = torch.empty(n * blocks * 34 + 256, dtype=torch.uint8, device=device)
    off = (-t.data_ptr()) % 256
    out = t[off:off + n * blocks * 34].view(n, blocks, 34)
    step = max(1, (1 << 28) // k)
    for r0 in range(0, n, step):
        r1 = min(n, r0 + step)
        q = torch.randint(-127, 128, (r1 - r0, blocks, 32), dtype=torch.int8, device=device, generator=gen)
        d = (torch.randn((r1 - r0, blocks), device=device, generator=gen).abs() * (0.02 / 127.0)).half()
        out[r0:r1, :, 2:] = q.view(torch.uint8)
        out[r0:r1, :, :2] = d.view(torch.uint8).view(r1 - r0, blocks, 2)
    return out.view(-1)


def _dtype_code(dtype):
    torch = _torch()
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[dtype]


class Q8Context:
    """One per device: owns the scratch of the streaming kernel (aotx_q8_init)."""

    def __init__(self, device=0):
        torch = _torch()
        self.lib = load_library()
        if not torch.cuda.is_available():
            raise RuntimeError("aotx_b200 needs a CUDA device; there is no CPU path")
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        torch.cuda.init()
        torch.zeros(1, device=self.device)
        handle = C.c_void_p()
        self._check(self.lib.aotx_q8_init(C.byref(handle), device))
        self.handle = handle

    def close(self):
        if getattr(self, "handle", None) is not None:
            self.lib.aotx_q8_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, code):
        if code != 0:
            detail = ""
            if code == 3 and getattr(self, "handle", None) is not None:
                detail = " cudaError=%d" % self.lib.aotx_q8_last_cuda_error(self.handle)
            raise Q8Error(code, detail)

    def _stream(self):
        return C.c_void_p(_torch().cuda.current_stream(self.device).cuda_stream)

    def set_path(self, path):
        self._check(self.lib.aotx_q8_set_path(self.handle, path))

    def set_overlap(self, enabled):
        self._check(self.lib.aotx_q8_set_overlap(self.handle, int(bool(enabled))))

    def device_status(self, clear=True):
        status = C.c_uint32(0)
        code = self.lib.aotx_q8_device_status(self.handle, C.byref(status), int(clear))
        if code not in (0, 6):
            self._check(code)
        return status.value

    # -- aotx_model_dequant ------------------------------------------------------------
    def dequant(self, w, k, first_row, rows, out=None, type=Q8_0):
        torch = _torch()
        if out is None:
            out = torch.empty((rows, k), dtype=torch.float16, device=self.device)
        self._check(self.lib.aotx_q8_dequant(self.handle, self._stream(), w.data_ptr(), type, k,
                                             first_row, rows, out.data_ptr()))
        return out

    # -- aotx_model_matrix --------------------------------------------------------------
    def matmul(self, w, n, k, x, m=None, m_dev=None, y=None, y_dtype=None, type=Q8_0):
        """y[m][n] = x[m][k] . w[n][k]^T.  `m_dev`: optional uint32 device tensor holding the
        live batch (read on the device); `m` is then the largest batch."""
        torch = _torch()
        if m is None:
            m = x.shape[0]
        if y is None:
            y = torch.empty((m, n), dtype=y_dtype or torch.float32, device=self.device)
        self._check(self.lib.aotx_q8_matmul(
            self.handle, self._stream(), w.data_ptr(), type, n, k, x.data_ptr(),
            _dtype_code(x.dtype), m, m_dev.data_ptr() if m_dev is not None else None,
            y.data_ptr(), _dtype_code(y.dtype)))
        return y

    def matmul_fused(self, w, n, k, x, epilogue, m=None, m_dev=None, y=None, y_dtype=None, type=Q8_0):
        """The product with the next step of the layer in its store.  EPILOGUE_ADD: `y` is the
        float residual stream, the product is added to it.  EPILOGUE_SWIGLU: `w` holds gate and
        up rows interleaved (`interleave_rows`), the result is silu(gate) * up, [m][n // 2]."""
        torch = _torch()
        if m is None:
            m = x.shape[0]
        if y is None:
            if epilogue == EPILOGUE_ADD:
                raise ValueError("EPILOGUE_ADD adds into a y that the caller gives")
            width = n // 2 if epilogue == EPILOGUE_SWIGLU else n
            y = torch.empty((m, width), dtype=y_dtype or torch.float32, device=self.device)
        self._check(self.lib.aotx_q8_matmul_fused(
            self.handle, self._stream(), w.data_ptr(), type, n, k, x.data_ptr(),
            _dtype_code(x.dtype), m, m_dev.data_ptr() if m_dev is not None else None,
            y.data_ptr(), _dtype_code(y.dtype), epilogue))
        return y

    def matmul_peers(self, w, n, k, x, m, y_ptrs, ldy, col0, y_dtype, m_dev=None, type=Q8_0):
        """Column-split product: columns [col0, col0 + n) of y[m][ldy], stored into every buffer
        of `y_ptrs` (device addresses: this GPU's y and the peers', peer-mapped)."""
        array = (C.c_void_p * len(y_ptrs))(*[C.c_void_p(int(p)) for p in y_ptrs])
        self._check(self.lib.aotx_q8_matmul_peers(
            self.handle, self._stream(), w.data_ptr(), type, n, k, x.data_ptr(), _dtype_code(x.dtype), m,
            m_dev.data_ptr() if m_dev is not None else None, array, len(y_ptrs), ldy, col0,
            _dtype_code(y_dtype)))

    def peer_barrier(self, flag_ptrs, rank, step_word):
        """The library's own barrier between the ranks of a column split: `flag_ptrs` are the
        device addresses of every rank's flag array (own and peer-mapped), `step_word` a uint32
        device tensor of this rank (zero at the start)."""
        array = (C.c_void_p * len(flag_ptrs))(*[C.c_void_p(int(p)) for p in flag_ptrs])
        self._check(self.lib.aotx_q8_peer_barrier(self.handle, self._stream(), array, len(flag_ptrs), rank,
                                                  step_word.data_ptr()))

    def matmul_colsplit(self, w, n, k, x, m, y_ptrs, flag_ptrs, rank, ldy, col0, y_dtype, step_word, m_dev=None,
                        type=Q8_0):
        """`matmul_peers` followed by `peer_barrier`: one call per rank and step."""
        ys = (C.c_void_p * len(y_ptrs))(*[C.c_void_p(int(p)) for p in y_ptrs])
        flags = (C.c_void_p * len(flag_ptrs))(*[C.c_void_p(int(p)) for p in flag_ptrs])
        self._check(self.lib.aotx_q8_matmul_colsplit(
            self.handle, self._stream(), w.data_ptr(), type, n, k, x.data_ptr(), _dtype_code(x.dtype), m,
            m_dev.data_ptr() if m_dev is not None else None, ys, flags, len(y_ptrs), rank, ldy, col0,
            _dtype_code(y_dtype), step_word.data_ptr()))

    def matmul_host(self, w, n, k, x_host, y_host, x_dev, y_dev):
        """The same product with the activations and the result in pinned host memory: copy
        in, multiply, copy out, all on the current stream (weights stay resident on the
        device, as the reference keeps them)."""
        x_dev.copy_(x_host, non_blocking=True)
        self.matmul(w, n, k, x_dev, y=y_dev)
        y_host.copy_(y_dev, non_blocking=True)
        return y_host

    # -- routed experts -------------------------------------------------------------------
    def moe_route(self, x, router, used, tokens=None, tokens_dev=None, prob=None, ids=None):
        torch = _torch()
        tokens = x.shape[0] if tokens is None else tokens
        experts, hidden = router.shape
        if prob is None:
            prob = torch.empty((tokens, experts), dtype=torch.float32, device=self.device)
        if ids is None:
            ids = torch.empty((tokens, used), dtype=torch.int32, device=self.device)
        self._check(self.lib.aotx_q8_moe_route(
            self.handle, self._stream(), x.data_ptr(), router.data_ptr(), tokens,
            tokens_dev.data_ptr() if tokens_dev is not None else None, hidden, experts, used,
            prob.data_ptr(), ids.data_ptr()))
        return prob, ids

    def moe_workspace(self, tokens, used, hidden, ffn):
        torch = _torch()
        size = self.lib.aotx_q8_moe_workspace_bytes(tokens, used, hidden, ffn)
        return torch.empty(size, dtype=torch.uint8, device=self.device)

    def moe_ffn(self, w_gate, w_up, w_down, experts, hidden, ffn, x, prob, ids, tokens=None,
                tokens_dev=None, out=None, out_dtype=None, workspace=None, type=Q8_0):
        torch = _torch()
        tokens = x.shape[0] if tokens is None else tokens
        used = ids.shape[1]
        if out is None:
            out = torch.empty((tokens, hidden), dtype=out_dtype or torch.float32, device=self.device)
        if workspace is None:
            workspace = self.moe_workspace(tokens, used, hidden, ffn)
        self._check(self.lib.aotx_q8_moe_ffn(
            self.handle, self._stream(), w_gate.data_ptr(), w_up.data_ptr(), w_down.data_ptr(),
            type, experts, hidden, ffn, x.data_ptr(), prob.data_ptr(), ids.data_ptr(), tokens,
            tokens_dev.data_ptr() if tokens_dev is not None else None, used, out.data_ptr(),
            _dtype_code(out.dtype), workspace.data_ptr(), workspace.numel()))
        return out

    def moe_ffn_fused(self, w_gate_up, w_down, experts, hidden, ffn, x, prob, ids, tokens=None,
                      tokens_dev=None, out=None, out_dtype=None, workspace=None, type=Q8_0):
        """`moe_ffn` with gate and up of every expert interleaved in one tensor
        ([experts][2 * ffn][hidden], see `interleave_rows`)."""
        torch = _torch()
        tokens = x.shape[0] if tokens is None else tokens
        used = ids.shape[1]
        if out is None:
            out = torch.empty((tokens, hidden), dtype=out_dtype or torch.float32, device=self.device)
        if workspace is None:
            workspace = self.moe_workspace(tokens, used, hidden, ffn)
        self._check(self.lib.aotx_q8_moe_ffn_fused(
            self.handle, self._stream(), w_gate_up.data_ptr(), w_down.data_ptr(), type, experts, hidden,
            ffn, x.data_ptr(), prob.data_ptr(), ids.data_ptr(), tokens,
            tokens_dev.data_ptr() if tokens_dev is not None else None, used, out.data_ptr(),
            _dtype_code(out.dtype), workspace.data_ptr(), workspace.numel()))
        return out

    def moe_ep_workspace(self, tokens, used, hidden, ffn, peers):
        torch = _torch()
        size = self.lib.aotx_q8_moe_ep_workspace_bytes(tokens, used, hidden, ffn, peers)
        return torch.empty(size, dtype=torch.uint8, device=self.device)

    def moe_ep(self, w_gate, w_up, w_down, experts_total, hidden, ffn, x_ptrs, ids_ptrs, prob, tokens, used,
               proj_ptrs, flag_ptrs, rank, step_word, out, workspace, type=Q8_0):
        """The expert-parallel routed step of this rank (aotx_q8_moe_ep): `x_ptrs`, `ids_ptrs`,
        `proj_ptrs`, `flag_ptrs` are device addresses of every rank's arrays (own and
        peer-mapped); w_* hold this rank's experts."""
        table = lambda ptrs: (C.c_void_p * len(ptrs))(*[C.c_void_p(int(p)) for p in ptrs])
        self._check(self.lib.aotx_q8_moe_ep(
            self.handle, self._stream(), w_gate.data_ptr(), w_up.data_ptr(), w_down.data_ptr(), type,
            experts_total, hidden, ffn, table(x_ptrs), table(ids_ptrs), prob.data_ptr(), tokens, used,
            table(proj_ptrs), table(flag_ptrs), len(flag_ptrs), rank, step_word.data_ptr(), out.data_ptr(),
            _dtype_code(out.dtype), workspace.data_ptr(), workspace.numel()))
        return out

    def moe_combine(self, proj, prob, ids, tokens=None, tokens_dev=None, out=None, out_dtype=None):
        """aotx_model_expert_add over all ranks: proj is float [tokens][used][hidden]."""
        torch = _torch()
        tokens = proj.shape[0] if tokens is None else tokens
        used, hidden = proj.shape[1], proj.shape[2]
        experts = prob.shape[1]
        if out is None:
            out = torch.empty((tokens, hidden), dtype=out_dtype or torch.float32, device=self.device)
        self._check(self.lib.aotx_q8_moe_combine(
            self.handle, self._stream(), proj.data_ptr(), prob.data_ptr(), ids.data_ptr(), tokens,
            tokens_dev.data_ptr() if tokens_dev is not None else None, hidden, experts, used,
            out.data_ptr(), _dtype_code(out.dtype)))
        return out
