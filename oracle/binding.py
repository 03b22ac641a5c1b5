"""ctypes bindings of the checker libraries.  TEST INFRASTRUCTURE ONLY.

`Oracle` wraps `libq8_oracle.so` (the C restatement in `q8_oracle.c`); `Reference` wraps
`_ref/libaotx_ref.so` (the reference's own sources, compiled unmodified).  Only the test
suite, the smoke check and the CPU-baseline leg of the benchmark import this module.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

SEED = 0x243F6A8885A308D3  # tests/matrix_test.cu:27
SPOT_SEED = SEED ^ 0x5A5A5A5A  # tests/matrix_test.cu:282

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")


def row_bytes(k):
    return (k // 32) * 34


class Oracle:
    def __init__(self):
        path = _build.build_oracle()
        lib = C.CDLL(path)
        self.lib = lib
        lib.q8o_f32_to_f16.restype = C.c_uint16
        lib.q8o_f32_to_f16.argtypes = [C.c_float]
        lib.q8o_f16_to_f32.restype = C.c_float
        lib.q8o_f16_to_f32.argtypes = [C.c_uint16]
        lib.q8o_f32_to_bf16.restype = C.c_uint16
        lib.q8o_f32_to_bf16.argtypes = [C.c_float]
        lib.q8o_bf16_to_f32.restype = C.c_float
        lib.q8o_bf16_to_f32.argtypes = [C.c_uint16]
        lib.q8o_next.restype = C.c_uint64
        lib.q8o_next.argtypes = [C.POINTER(C.c_uint64)]
        lib.q8o_unit.restype = C.c_float
        lib.q8o_unit.argtypes = [C.POINTER(C.c_uint64)]
        lib.q8o_build.argtypes = [_u8p, C.c_uint32, C.c_uint32, C.c_uint64]
        lib.q8o_input.argtypes = [_u16p, C.c_uint32, C.c_uint32, C.c_uint64]
        lib.q8o_weight.restype = C.c_float
        lib.q8o_weight.argtypes = [C.c_void_p, C.c_uint32]
        lib.q8o_dequant.argtypes = [_u8p, C.c_uint32, C.c_uint32, C.c_uint32, _u16p]
        lib.q8o_product.argtypes = [_u8p, C.c_uint32, C.c_uint32, _u16p, C.c_int, C.c_uint32,
                                    _f64p, C.c_int, C.c_int]
        lib.q8o_diff.restype = C.c_uint32
        lib.q8o_diff.argtypes = [_f32p, _f64p, C.c_size_t, C.c_double, C.POINTER(C.c_double)]
        lib.q8o_spot.restype = C.c_uint32
        lib.q8o_spot.argtypes = [_u8p, C.c_uint32, C.c_uint32, _u16p, C.c_int, C.c_uint32, _f32p,
                                 C.c_uint32, C.c_uint64, C.c_double, C.POINTER(C.c_double)]
        lib.q8o_within_bound.restype = C.c_int
        lib.q8o_within_bound.argtypes = [_f32p, _f64p, C.c_size_t, C.POINTER(C.c_double),
                                         C.POINTER(C.c_double)]
        lib.q8o_block_row_bytes.restype = C.c_uint64
        lib.q8o_block_row_bytes.argtypes = [C.c_uint32, C.c_uint32]
        lib.q8o_block_weight.restype = C.c_double
        lib.q8o_block_weight.argtypes = [C.c_uint32, C.c_void_p, C.c_uint32]
        lib.q8o_block_rows.argtypes = [C.c_uint32, _u8p, C.c_uint32, C.c_uint32, C.c_uint32, _f64p]
        lib.q8o_route.argtypes = [_u16p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                  _f64p, _u32p]
        lib.q8o_rank.argtypes = [_f32p, C.c_uint32, C.c_uint32, C.c_uint32, _u32p]
        lib.q8o_expert_matrix.argtypes = [_u8p, C.c_uint32, C.c_uint32, _u16p, _u32p, C.c_uint32,
                                          C.c_uint32, C.c_uint32, _f64p, _f64p]
        lib.q8o_ordered_sum.argtypes = [_f32p, _f32p, _u32p, C.c_uint32, C.c_uint32, C.c_uint32,
                                        C.c_uint32, _f32p]
        lib.q8o_moe_ffn.argtypes = [_u8p, _u8p, _u8p, C.c_uint32, C.c_uint32, C.c_uint32, _u16p,
                                    _f32p, _u32p, C.c_uint32, C.c_uint32, _f32p, C.c_void_p,
                                    C.c_int]
        lib.q8o_max_threads.restype = C.c_int

    # fixtures of the reference's own recipe -------------------------------------------
    def build(self, n, k, seed):
        w = np.zeros(n * row_bytes(k), np.uint8)
        self.lib.q8o_build(w, n, k, seed)
        return w

    def input(self, m, k, seed):
        x = np.zeros(m * k, np.uint16)
        self.lib.q8o_input(x, m, k, seed)
        return x.reshape(m, k)

    # the checks ------------------------------------------------------------------------
    def dequant(self, w, k, first, rows):
        out = np.zeros((rows, k), np.uint16)
        self.lib.q8o_dequant(np.ascontiguousarray(w), k, first, rows, out)
        return out

    def product(self, w, n, k, x, m, bf16=False, swap=False, threads=None):
        y = np.zeros((m, n), np.float64)
        threads = threads or self.max_threads()
        self.lib.q8o_product(np.ascontiguousarray(w), n, k,
                             np.ascontiguousarray(x).reshape(-1), int(bf16), m, y, int(swap),
                             threads)
        return y

    def diff(self, got, want, tol=1e-2):
        worst = C.c_double(0)
        got = np.ascontiguousarray(got, np.float32).reshape(-1)
        want = np.ascontiguousarray(want, np.float64).reshape(-1)
        bad = self.lib.q8o_diff(got, want, got.size, tol, C.byref(worst))
        return bad, worst.value

    def spot(self, w, n, k, x, m, y, count=64, bf16=False, seed=SPOT_SEED, tol=1e-2):
        worst = C.c_double(0)
        bad = self.lib.q8o_spot(np.ascontiguousarray(w), n, k,
                                np.ascontiguousarray(x).reshape(-1), int(bf16), m,
                                np.ascontiguousarray(y, np.float32).reshape(-1), count, seed, tol,
                                C.byref(worst))
        return bad, worst.value

    def block_row_bytes(self, kind, k):
        return int(self.lib.q8o_block_row_bytes(kind, k))

    def block_rows(self, kind, w, k, first, rows):
        """[rows][k] doubles: the value of every weight of rows [first, first + rows) of a tensor
        of block type `kind` (blocks_oracle.c)."""
        out = np.empty((rows, k), np.float64)
        self.lib.q8o_block_rows(kind, np.ascontiguousarray(w, np.uint8).reshape(-1), k, first, rows, out)
        return out

    def within_bound(self, got, want):
        err = C.c_double(0)
        bound = C.c_double(0)
        got = np.ascontiguousarray(got, np.float32).reshape(-1)
        want = np.ascontiguousarray(want, np.float64).reshape(-1)
        ok = self.lib.q8o_within_bound(got, want, got.size, C.byref(err), C.byref(bound))
        return bool(ok), err.value, bound.value

    def route(self, x, router, used):
        tokens, hidden = x.shape
        experts = router.shape[0]
        prob = np.zeros((tokens, experts), np.float64)
        ids = np.full((tokens, used), 0xFFFFFFFF, np.uint32)
        self.lib.q8o_route(np.ascontiguousarray(x).reshape(-1),
                           np.ascontiguousarray(router, np.float32).reshape(-1), tokens, hidden,
                           experts, used, prob, ids)
        return prob, ids

    def rank(self, prob, used):
        tokens, experts = prob.shape
        ids = np.full((tokens, used), 0xFFFFFFFF, np.uint32)
        self.lib.q8o_rank(np.ascontiguousarray(prob, np.float32).reshape(-1), tokens, experts,
                          used, ids)
        return ids

    def expert_matrix(self, w, n, k, x, ids, rank):
        tokens = x.shape[0]
        used = ids.shape[1]
        y = np.zeros((tokens, n), np.float64)
        mag = np.zeros((tokens, n), np.float64)
        self.lib.q8o_expert_matrix(np.ascontiguousarray(w), n, k,
                                   np.ascontiguousarray(x).reshape(-1),
                                   np.ascontiguousarray(ids, np.uint32).reshape(-1), used, rank,
                                   tokens, y, mag)
        return y, mag

    def ordered_sum(self, proj, prob, ids):
        used, tokens, hidden = proj.shape
        experts = prob.shape[1]
        out = np.zeros((tokens, hidden), np.float32)
        self.lib.q8o_ordered_sum(np.ascontiguousarray(proj, np.float32).reshape(-1),
                                 np.ascontiguousarray(prob, np.float32).reshape(-1),
                                 np.ascontiguousarray(ids, np.uint32).reshape(-1), tokens, hidden,
                                 experts, used, out)
        return out

    def moe_ffn(self, w_gate, w_up, w_down, experts, hidden, ffn, x, prob, ids, threads=None,
                want_act=False):
        tokens = x.shape[0]
        used = ids.shape[1]
        out = np.zeros((tokens, hidden), np.float32)
        act = np.zeros((used, tokens, ffn), np.uint16) if want_act else None
        self.lib.q8o_moe_ffn(np.ascontiguousarray(w_gate), np.ascontiguousarray(w_up),
                             np.ascontiguousarray(w_down), experts, hidden, ffn,
                             np.ascontiguousarray(x).reshape(-1),
                             np.ascontiguousarray(prob, np.float32).reshape(-1),
                             np.ascontiguousarray(ids, np.uint32).reshape(-1), tokens, used, out,
                             act.ctypes.data if act is not None else None,
                             threads or self.max_threads())
        return (out, act) if want_act else out

    def max_threads(self):
        return min(self.lib.q8o_max_threads(), os.cpu_count() or 1)


class Reference:
    """The reference's own host functions; None-like (`available` False) when not built."""

    def __init__(self):
        path = _build.build_ref()
        self.available = path is not None and os.path.exists(path)
        if not self.available:
            return
        lib = C.CDLL(path)
        self.lib = lib
        lib.ref_next.restype = C.c_uint64
        lib.ref_next.argtypes = [C.POINTER(C.c_uint64)]
        lib.ref_unit.restype = C.c_float
        lib.ref_unit.argtypes = [C.POINTER(C.c_uint64)]
        lib.ref_weight.restype = C.c_float
        lib.ref_weight.argtypes = [C.c_void_p, C.c_uint32]
        lib.ref_float_to_half_bits.restype = C.c_uint16
        lib.ref_float_to_half_bits.argtypes = [C.c_float]
        lib.ref_half_bits_to_float.restype = C.c_float
        lib.ref_half_bits_to_float.argtypes = [C.c_uint16]
        lib.ref_build.restype = C.c_uint64
        lib.ref_build.argtypes = [_u8p, C.c_uint32, C.c_uint32, C.c_uint64]
        lib.ref_input.argtypes = [_u16p, C.c_uint32, C.c_uint32, C.c_uint64]
        lib.ref_product.argtypes = [_u8p, C.c_uint32, C.c_uint32, _u16p, C.c_uint32, _f64p,
                                    C.c_int]
        lib.ref_diff.restype = C.c_uint32
        lib.ref_diff.argtypes = [_f32p, _f64p, C.c_size_t, C.c_double, C.POINTER(C.c_double)]
        lib.ref_spot.restype = C.c_uint32
        lib.ref_spot.argtypes = [_u8p, C.c_uint32, C.c_uint32, _u16p, C.c_uint32, _f32p,
                                 C.c_uint32, C.POINTER(C.c_double)]
        lib.ref_same.restype = C.c_uint32
        lib.ref_same.argtypes = [_u8p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _u16p]
        for name in ("ref_gpu_gemv", "ref_gpu_gemm"):
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32,
                           C.c_void_p, C.c_void_p]
        lib.ref_gpu_dequant.restype = C.c_int
        lib.ref_gpu_dequant.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                        C.c_void_p, C.c_void_p]

    def build(self, n, k, seed):
        w = np.zeros(n * row_bytes(k), np.uint8)
        self.lib.ref_build(w, n, k, seed)
        return w

    def input(self, m, k, seed):
        x = np.zeros(m * k, np.uint16)
        self.lib.ref_input(x, m, k, seed)
        return x.reshape(m, k)

    def product(self, w, n, k, x, m, swap=False):
        y = np.zeros((m, n), np.float64)
        self.lib.ref_product(np.ascontiguousarray(w), n, k,
                             np.ascontiguousarray(x).reshape(-1), m, y, int(swap))
        return y

    def diff(self, got, want, tol=1e-2):
        worst = C.c_double(0)
        got = np.ascontiguousarray(got, np.float32).reshape(-1)
        want = np.ascontiguousarray(want, np.float64).reshape(-1)
        bad = self.lib.ref_diff(got, want, got.size, tol, C.byref(worst))
        return bad, worst.value

    def spot(self, w, n, k, x, m, y, count=64):
        worst = C.c_double(0)
        bad = self.lib.ref_spot(np.ascontiguousarray(w), n, k,
                                np.ascontiguousarray(x).reshape(-1), m,
                                np.ascontiguousarray(y, np.float32).reshape(-1), count,
                                C.byref(worst))
        return bad, worst.value

    def same(self, w, n, k, first, rows, got):
        return self.lib.ref_same(np.ascontiguousarray(w), n, k, first, rows,
                                 np.ascontiguousarray(got, np.uint16).reshape(-1))


class ReferenceExperts:
    """The reference's routed-expert kernels run on a CUDA device (`_ref/libaotx_ref.so`:
    cuda/model/experts.cu, expert_matrix.cu, norm.cu compiled unmodified; launchers in
    ref_wrap.cu).  Device memory comes from torch.  The checker of the routed-expert oracle and
    the second baseline of the benchmark's routed-expert workload; never on the product path."""

    def __init__(self):
        import torch
        self.torch = torch
        self.ref = Reference()
        if not self.ref.available:
            raise RuntimeError("the reference library is not built")
        lib = self.ref.lib
        self.lib = lib
        P, U = C.c_void_p, C.c_uint32
        lib.ref_gpu_moe_install.restype = C.c_int
        lib.ref_gpu_moe_install.argtypes = [U, U, U, U, U, P, P, P, P, P, P, P, P, P]
        lib.ref_gpu_moe_route.restype = C.c_int
        lib.ref_gpu_moe_route.argtypes = [U, P]
        lib.ref_gpu_moe_matrix.restype = C.c_int
        lib.ref_gpu_moe_matrix.argtypes = [U, P, U, U, P, P, U, P]
        lib.ref_gpu_moe_add.restype = C.c_int
        lib.ref_gpu_moe_add.argtypes = [U, U, P]
        lib.ref_gpu_moe_ffn.restype = C.c_int
        lib.ref_gpu_moe_ffn.argtypes = [P, P, P, U, U, U, P, P, P, P, P, U, P]

    def _dev(self, array):
        return self.torch.from_numpy(np.ascontiguousarray(array)).cuda()

    def _check(self, code, what):
        if code != 0:
            raise RuntimeError("%s: CUDA error %d" % (what, code))

    def install(self, hidden, ffn, experts, used, tokens, router=None, x=None, prob=None, ids=None,
                gate=None, up=None, act=None, proj=None, total=None):
        ptr = lambda t: t.data_ptr() if t is not None else None
        self._check(self.lib.ref_gpu_moe_install(hidden, ffn, experts, used, tokens, ptr(router), ptr(x),
                                                 ptr(prob), ptr(ids), ptr(gate), ptr(up), ptr(act),
                                                 ptr(proj), ptr(total)), "install")

    def route(self, x, router, used, grid=None):
        torch = self.torch
        tokens, hidden = x.shape
        experts = router.shape[0]
        xd, rd = self._dev(x.view(np.uint16).view(np.int16)), self._dev(router)
        prob = torch.zeros(tokens, experts, dtype=torch.float32, device="cuda")
        ids = torch.full((tokens, used), -1, dtype=torch.int32, device="cuda")
        self.install(hidden, 0, experts, used, tokens, router=rd, x=xd, prob=prob, ids=ids)
        self._check(self.lib.ref_gpu_moe_route(grid or tokens, None), "route")
        torch.cuda.synchronize()
        return prob.cpu().numpy(), ids.cpu().numpy().view(np.uint32)

    def ordered_sum(self, proj, prob, ids):
        """proj [used][tokens][hidden]; one add launch per rank as tests/expert_test.cu:164-187."""
        torch = self.torch
        used, tokens, hidden = proj.shape
        experts = prob.shape[1]
        pd = self._dev(prob)
        idd = self._dev(ids.view(np.int32))
        buf = torch.zeros(tokens, hidden, dtype=torch.float32, device="cuda")
        total = torch.zeros(tokens, hidden, dtype=torch.float32, device="cuda")
        self.install(hidden, 0, experts, used, tokens, prob=pd, ids=idd, proj=buf, total=total)
        for rank in range(used):
            buf.copy_(self._dev(proj[rank]))
            self._check(self.lib.ref_gpu_moe_add(rank, 7, None), "add")
        torch.cuda.synchronize()
        return total.cpu().numpy()

    def expert_matrix(self, w, n, k, x, ids, rank, experts):
        torch = self.torch
        tokens = x.shape[0]
        used = ids.shape[1]
        wd = self._dev(w)
        xd = self._dev(x.view(np.uint16).view(np.int16))
        idd = self._dev(ids.view(np.int32))
        y = torch.zeros(tokens, n, dtype=torch.float32, device="cuda")
        self.install(0, 0, experts, used, tokens, ids=idd)
        self._check(self.lib.ref_gpu_moe_matrix(rank, wd.data_ptr(), n, k, xd.data_ptr(), y.data_ptr(),
                                                tokens + 2 if tokens == 1 else 7, None), "matrix")
        torch.cuda.synchronize()
        return y.cpu().numpy()

    def ffn_buffers(self, wg, wu, wd, experts, hidden, ffn, x, router, used):
        """Device tensors of a whole routed step, installed; returns a dict of them."""
        torch = self.torch
        tokens = x.shape[0]
        f32 = dict(dtype=torch.float32, device="cuda")
        b = {"wg": self._dev(wg), "wu": self._dev(wu), "wd": self._dev(wd),
             "x": self._dev(x.view(np.uint16).view(np.int16)), "router": self._dev(router),
             "prob": torch.zeros(tokens, experts, **f32),
             "ids": torch.zeros(tokens, used, dtype=torch.int32, device="cuda"),
             "gate": torch.zeros(tokens, ffn, **f32), "up": torch.zeros(tokens, ffn, **f32),
             "act": torch.zeros(tokens, ffn, dtype=torch.float16, device="cuda"),
             "proj": torch.zeros(tokens, hidden, **f32), "sum": torch.zeros(tokens, hidden, **f32)}
        self.install(hidden, ffn, experts, used, tokens, router=b["router"], x=b["x"], prob=b["prob"],
                     ids=b["ids"], gate=b["gate"], up=b["up"], act=b["act"], proj=b["proj"], total=b["sum"])
        b["shape"] = (tokens, experts, used, hidden, ffn)
        return b

    def launch_step(self, b, stream=None):
        """Route and the per-rank loop of cuda/model/experts_host.cu:96-111 on installed buffers."""
        tokens, experts, used, hidden, ffn = b["shape"]
        self._check(self.lib.ref_gpu_moe_route(tokens, stream), "route")
        self._check(self.lib.ref_gpu_moe_ffn(b["wg"].data_ptr(), b["wu"].data_ptr(), b["wd"].data_ptr(),
                                             hidden, ffn, used, b["x"].data_ptr(), b["gate"].data_ptr(),
                                             b["up"].data_ptr(), b["act"].data_ptr(), b["proj"].data_ptr(),
                                             tokens, stream), "expert loop")

    def ffn(self, wg, wu, wd, experts, hidden, ffn, x, router, used):
        b = self.ffn_buffers(wg, wu, wd, experts, hidden, ffn, x, router, used)
        self.launch_step(b)
        self.torch.cuda.synchronize()
        return {"prob": b["prob"].cpu().numpy(), "ids": b["ids"].cpu().numpy().view(np.uint32),
                "sum": b["sum"].cpu().numpy(), "act": b["act"].cpu().numpy().view(np.uint16)}
