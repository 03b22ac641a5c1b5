"""Where the time of a launch of the decode kernel goes: per launch, the earliest and latest time
(microseconds from the first block's start) at which its blocks started, saw the launches before
them finished, got their first x segment, finished converting, had their sums, passed the two
cluster barriers and ended.  Needs a CUDA device and the trace build:

    python -m aotx_b200.build --trace
    AOTX_Q8_LIBRARY=trace Q8_TRACE=1 python -m aotx_b200.timeline [n k rows [bf16|f16]]...

Without arguments: the four projections of the benchmark's decode layer at 32 rows.  Each shape
runs as a captured graph of eight launches over rotating weight copies, replayed a few times;
the stamps are those of the last replay."""
import ctypes as C
import sys

import numpy as np

NAMES = ["start", "x landed", "waited", "converted", "barrier A", "sums", "barrier B", "end"]
BLOCKS = 320


def timeline(ctx, lib, n, k, rows, x_dtype, copies=8):
    import torch
    import aotx_b200
    ws = [aotx_b200.synth_q8_0_device(n, k, 1 + c) for c in range(copies)]
    x = torch.randn(rows, k, device="cuda").to(x_dtype)
    y = torch.empty(rows, n, device="cuda", dtype=torch.bfloat16)
    ctx.matmul(ws[0], n, k, x, y=y)
    torch.cuda.synchronize()
    buf = np.zeros(256 * BLOCKS * 8, np.uint64)
    before = lib.q8_trace_read(buf.ctypes.data_as(C.c_void_p))
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for w in ws:
                ctx.matmul(w, n, k, x, y=y)
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    print("%d x %d, %d rows of %s: %.2f us per launch" % (n, k, rows, str(x_dtype)[6:],
                                                       e0.elapsed_time(e1) * 1e3 / copies))
    lib.q8_trace_read(buf.ctypes.data_as(C.c_void_p))
    stamps = buf.reshape(256, BLOCKS, 8).astype(np.int64)
    origin = None
    for i in range(copies):
        one = stamps[(before + i) % 256]        # the slots are fixed at capture; a replay rewrites them
        live = one[:, 0] > 0
        if origin is None:
            origin = one[live, 0].min()
        parts = []
        for column, name in enumerate(NAMES):
            values = one[live, column]
            values = values[values > 0]
            if len(values):
                parts.append("%s %.1f..%.1f" % (name, (values.min() - origin) / 1e3, (values.max() - origin) / 1e3))
        print("  launch %d, %d blocks: %s" % (i, int(live.sum()), "; ".join(parts)))


def main():
    import torch
    import aotx_b200
    ctx = aotx_b200.Q8Context(0)
    lib = aotx_b200.load_library()
    if not hasattr(lib, "q8_trace_read"):
        raise SystemExit("this is not the trace build: python -m aotx_b200.build --trace, AOTX_Q8_LIBRARY=trace")
    args = sys.argv[1:]
    shapes = []
    while len(args) >= 3:
        kind = torch.float16 if (len(args) > 3 and args[3] == "f16") else torch.bfloat16
        shapes.append((int(args[0]), int(args[1]), int(args[2]), kind))
        args = args[4:] if len(args) > 3 and args[3] in ("f16", "bf16") else args[3:]
    if not shapes:
        shapes = [(6144, 4096, 32, torch.bfloat16), (4096, 4096, 32, torch.bfloat16),
                  (28672, 4096, 32, torch.bfloat16), (4096, 14336, 32, torch.bfloat16)]
    for n, k, rows, kind in shapes:
        timeline(ctx, lib, n, k, rows, kind, copies=4 if n * k > 5e7 else 8)


if __name__ == "__main__":
    main()
