#!/usr/bin/env python
"""Benchmark of the Q8_0 weight-matrix path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Without --workload the line covers every configuration of the benchmark:

* one GPU: the headline is the decode layer step (`decode_m32_llama3_8b_layer`: the four Q8_0
  projections of a Llama-3-8B-shaped layer at a batch of 32 rows - fused QKV 4096->6144, O
  4096->4096, fused gate+up 4096->28672, down 14336->4096 - bf16 activations, float sums, bf16
  results), and `configs` holds short measurements of the single-row product, the prefill layer at
  2048 rows, the routed experts and the LM head, each with its roofline fraction;
* N > 1 GPUs (one rank per GPU, launched by torchrun): the headline is what shards - the LM head
  8192 -> 151936 split by output columns over the ranks, every rank storing its slice of y into
  all ranks' buffers from the kernel's own stores (strong scaling: the total work is fixed) - and
  `sharded` holds that product at 8 and 64 rows and the expert-parallel routed experts, each with
  the one-GPU time measured in the same run and the speed-up over it.

All tensors are seeded synthetic (uniform int8, one half scale per 32 weights).  The metric is
algorithmic bytes moved per second - every weight byte once plus the activations in and the
results out - or FLOP/s for the prefill layer.  Weight copies rotate between steps so that no
step finds its weights in L2.  Prints one JSON line (rank 0).  `value` is timed with inputs
resident in device memory; `e2e` runs the same steps through the library call with activations
and results in pinned host memory, copies inside the timed region.  `--impl reference` times the
reference's own host implementation of the product on this machine's cores over a bounded sample.
"""
import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (rows of x, [(projection, k, n)], x dtype, y dtype)
    "decode_m32_llama3_8b_layer": (32, [("qkv", 4096, 6144), ("o", 4096, 4096),
                                        ("gate_up", 4096, 28672), ("down", 14336, 4096)],
                                   "bfloat16", "bfloat16"),
    "gemv_m1_4096": (1, [("w", 4096, 4096)], "float16", "float16"),
    # the LM head of configuration 4 on one GPU (the N > 1 headline splits it over the ranks)
    "lm_head_m8": (8, [("lm_head", 8192, 151936)], "bfloat16", "bfloat16"),
    "decode_m32_gate_up": (32, [("gate_up", 4096, 28672)], "bfloat16", "bfloat16"),
    "prefill_m2048_gate_up": (2048, [("gate_up", 4096, 28672)], "bfloat16", "bfloat16"),
    "prefill_m2048_llama3_8b_layer": (2048, [("qkv", 4096, 6144), ("o", 4096, 4096),
                                             ("gate_up", 4096, 28672), ("down", 14336, 4096)],
                                      "bfloat16", "bfloat16"),
}
# The same layer with the steps that follow the products folded into their stores: O and down add
# into the float residual stream, gate+up (rows interleaved) leaves as the half activations.
FUSED = {"decode_m32_llama3_8b_layer_fused": "decode_m32_llama3_8b_layer",
         "prefill_m2048_llama3_8b_layer_fused": "prefill_m2048_llama3_8b_layer"}
for _name, _base in FUSED.items():
    WORKLOADS[_name] = WORKLOADS[_base]
EPILOGUE_OF = {"o": 1, "down": 1, "gate_up": 2}  # AOTX_Q8_EPILOGUE_ADD / _SWIGLU

# DRAM bytes (read + write) per algorithmic byte of the dominant kernel: one ncu capture of the
# gate+up projection at 32 rows, scaled to the average launch by bytes (source named in the line).
TRAFFIC_RATIO = {"decode_m32_llama3_8b_layer": 1.2168, "decode_m32_gate_up": 1.2168}
TRAFFIC_SOURCE = "profiles/q8_decode_kernel_gate_up_m32.md (28672 x 4096, 32 rows, one launch)"
TENSOR_BOUND = {"prefill_m2048_llama3_8b_layer", "prefill_m2048_gate_up", "prefill_m2048_llama3_8b_layer_fused"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
        return peaks.get("hbm_gbs", 6650.0), peaks.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def mark_library(line):
    """A line measured on anything but the product library says so (AOTX_Q8_LIBRARY names a
    development build, with the switches set in the environment): not a product number."""
    if os.environ.get("AOTX_Q8_LIBRARY"):
        line["config"]["library"] = os.environ["AOTX_Q8_LIBRARY"]
        line["config"]["switches"] = {k: v for k, v in os.environ.items() if k.startswith("Q8_")}
    return line


def algorithmic_bytes(m, projections, x_bytes, y_bytes, fused=False):
    total = 0
    for name, k, n in projections:
        total += n * (k // 32) * 34 + m * k * x_bytes
        mode = EPILOGUE_OF.get(name, 0) if fused else 0
        if mode == 1:
            total += 2 * m * n * 4          # the float residual stream, read and written
        elif mode == 2:
            total += m * (n // 2) * 2       # half activations, one per gate/up pair
        else:
            total += m * n * y_bytes
    return total


def flops(m, projections):
    return sum(2 * m * n * k for _, k, n in projections)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        while not self.stop_flag.is_set():
            try:
                mhz = self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM)
                util = self.nvml.nvmlDeviceGetUtilizationRates(self.handle).gpu
                mask = self.nvml.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                self.samples.append((mhz, util))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                    "samples": 0}
        return {"sm_mhz": statistics.median(s[0] for s in self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def device_index(local_rank):
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        try:
            return int(visible.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def make_inputs(torch, m, projections, x_dtype, copies, seed):
    import aotx_b200
    rng = np.random.Generator(np.random.PCG64(seed))
    tensors = []
    for index, (name, k, n) in enumerate(projections):
        weights = []
        for c in range(copies):
            host = aotx_b200.synth_q8_0(n, k, seed * 1000 + index * 10 + c)
            dev = torch.empty(host.size, dtype=torch.uint8, device="cuda")
            dev.copy_(torch.from_numpy(host))
            weights.append(dev)
        x_host = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(x_dtype)
        tensors.append({"name": name, "k": k, "n": n, "w": weights, "x_host": x_host.pin_memory()})
    return tensors


def run_ours(args, rank, world, local_rank):
    import torch
    import aotx_b200

    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    m, projections, x_name, y_name = WORKLOADS[args.workload]
    x_dtype, y_dtype = getattr(torch, x_name), getattr(torch, y_name)
    ctx = aotx_b200.Q8Context(local_rank)
    weight_bytes = sum(n * (k // 32) * 34 for _, k, n in projections)
    copies = max(2, int(np.ceil(3 * 126e6 / weight_bytes)) + 1)
    copies = min(copies, 24)
    tensors = make_inputs(torch, m, projections, x_dtype, copies, seed=1 + rank)
    fused = args.workload in FUSED
    for t in tensors:
        t["x"] = t["x_host"].cuda()
        t["mode"] = EPILOGUE_OF.get(t["name"], 0) if fused else 0
        if t["mode"] == 1:
            shape, kind = (m, t["n"]), torch.float32
        elif t["mode"] == 2:
            shape, kind = (m, t["n"] // 2), torch.float16
        else:
            shape, kind = (m, t["n"]), y_dtype
        t["y"] = torch.zeros(shape, dtype=kind, device="cuda")
        t["y_host"] = torch.empty(shape, dtype=kind).pin_memory()

    def product(i, c):
        t = tensors[i]
        if t["mode"]:
            ctx.matmul_fused(t["w"][c], t["n"], t["k"], t["x"], t["mode"], y=t["y"])
        else:
            ctx.matmul(t["w"][c], t["n"], t["k"], t["x"], y=t["y"])

    def step(c):
        for i in range(len(tensors)):
            product(i, c)

    def step_e2e(c):
        for i, t in enumerate(tensors):
            t["x"].copy_(t["x_host"], non_blocking=True)
            product(i, c)
            t["y_host"].copy_(t["y"], non_blocking=True)

    # Captured graphs: the step is launch-bound on the host otherwise.  A graph holds `group`
    # consecutive steps over rotating weight copies (the reference's decode graph holds a whole
    # forward pass): inside a graph a product overlaps the tail of the one before it, as it does
    # in a model; between two graph launches it cannot.
    step(0)
    torch.cuda.synchronize()
    group = steps_per_graph(args.steps)
    distinct = copies // math.gcd(copies, group)
    graphs = []
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for j in range(distinct):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(group):
                    step((j * group + i) % copies)
            graphs.append(g)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        graphs[i % distinct].replay()
    barrier()

    sampler = ClockSampler(device_index(local_rank))
    sampler.start()
    first = torch.cuda.Event(enable_timing=True)
    last = torch.cuda.Event(enable_timing=True)
    first.record()
    for i in range(args.steps // group):
        graphs[i % distinct].replay()
    last.record()
    barrier()
    total_ms = first.elapsed_time(last)
    # A short timed region gives the sampler nothing to see: keep the same load running,
    # untimed, until it has a few samples under load.
    extended = False
    if len(sampler.samples) < 8:
        extended = True
        deadline = time.time() + 1.0
        i = 0
        while time.time() < deadline:
            for _ in range(50):
                graphs[i % distinct].replay()
                i += 1
            torch.cuda.synchronize()
    sampler.stop_flag.set()
    sampler.join()
    status = ctx.device_status()

    # End to end: activations start in pinned host memory and results end there, every step,
    # copies inside the timed region.  The step is captured like the resident one (the
    # reference runs its passes as graphs too): the uploads run on a copy stream ahead of the
    # products, each result goes back on a second copy stream while the next product runs.
    e2e_mode = "graph, copies overlapped on two copy streams"
    e2e_graphs = []
    try:
        main_stream = torch.cuda.Stream()
        up_stream = torch.cuda.Stream()
        down_stream = torch.cuda.Stream()
        with torch.cuda.stream(main_stream):
            for c in range(copies):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=main_stream):
                    up_stream.wait_stream(main_stream)
                    ready = []
                    with torch.cuda.stream(up_stream):
                        for t in tensors:
                            t["x"].copy_(t["x_host"], non_blocking=True)
                            event = torch.cuda.Event()
                            event.record(up_stream)
                            ready.append(event)
                    down_stream.wait_stream(main_stream)
                    for i, (t, event) in enumerate(zip(tensors, ready)):
                        main_stream.wait_event(event)
                        product(i, c)
                        done = torch.cuda.Event()
                        done.record(main_stream)
                        with torch.cuda.stream(down_stream):
                            down_stream.wait_event(done)
                            t["y_host"].copy_(t["y"], non_blocking=True)
                    main_stream.wait_stream(up_stream)
                    main_stream.wait_stream(down_stream)
                e2e_graphs.append(g)
        torch.cuda.synchronize()
    except Exception as error:
        e2e_graphs = []
        e2e_mode = "eager calls (graph capture failed: %s)" % str(error)[:80]

    def run_e2e(c):
        if e2e_graphs:
            e2e_graphs[c].replay()
        else:
            step_e2e(c)

    for i in range(3):
        run_e2e(i % copies)
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        run_e2e(i % copies)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    # the results that came back are the device results
    check = all(bool(torch.equal(t["y_host"], t["y"].cpu())) for t in tensors)

    if world > 1:
        import torch.distributed as dist
        both = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(both, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = both.tolist()

    x_bytes = y_bytes = 2
    step_bytes = algorithmic_bytes(m, projections, x_bytes, y_bytes, fused=fused)
    step_flops = flops(m, projections)
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    launches = len(projections)
    kernel_ms = total_ms / args.steps / launches
    tensor_bound = args.workload in TENSOR_BOUND
    if tensor_bound:
        achieved = step_flops / launches / (kernel_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
                    "frac": achieved / tensor_peak, "traffic": None}
        value = world * step_flops * args.steps / (total_ms * 1e-3) / 1e12
        e2e_value = world * step_flops * args.steps / (e2e_ms * 1e-3) / 1e12
        metric, unit = "q8_prefill_gemm_tflops", "TFLOP/s"
    else:
        achieved = step_bytes / launches / (kernel_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                    "frac": achieved / hbm_peak, "traffic": None}
        value = world * step_bytes * args.steps / (total_ms * 1e-3) / 1e9
        e2e_value = world * step_bytes * args.steps / (e2e_ms * 1e-3) / 1e9
        metric, unit = "q8_decode_gemm_hbm_gbs", "GB/s"
    ratio = TRAFFIC_RATIO.get(args.workload)
    roofline["traffic"] = ratio * step_bytes / launches if ratio else None
    roofline["traffic_source"] = TRAFFIC_SOURCE if ratio else None
    roofline["peak_source"] = peak_kind
    # the nominal figures, for context only (HBM3e 7.7 TB/s; dense bf16 2250 TFLOP/s)
    roofline["frac_of_nominal"] = achieved / (2250.0 if tensor_bound else 7700.0)
    roofline["kernel"] = "q8_wide_kernel" if tensor_bound else "q8_decode_kernel"
    roofline["launches_timed"] = launches * args.steps
    roofline["avg_launch_us"] = kernel_ms * 1e3
    roofline["bytes_per_launch"] = step_bytes / launches
    roofline["tokens_per_s"] = world * m * args.steps / (total_ms * 1e-3)

    h2d = sum(t["x_host"].numel() * t["x_host"].element_size() for t in tensors)
    d2h = sum(t["y_host"].numel() * t["y_host"].element_size() for t in tensors)
    clocks = sampler.summary()
    clocks["probe"] = "extended" if extended else "timed_region"

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16/bf16 operands, f32 sums",
        "data": "synthetic",
        "config": {"workload": args.workload, "rows": m, "x": x_name, "y": y_name,
                   "projections": {name: [k, n] for name, k, n in projections},
                   "weight_copies_rotated": copies, "l2": "weight copies rotate; total > 3x L2",
                   "parallelism": "replicas" if world > 1 else "single", "cuda_graph": True,
                   "steps_per_graph": group},
        "roofline": roofline,
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / args.steps, "mode": e2e_mode, "host_result_matches_device": check},
        "gpu_launches": launches * args.steps,
        "clocks": clocks,
        "device_status": status,
    }
    if world == 1 and args.composite:
        # the other configurations of the benchmark, measured briefly in the same run
        line["configs"] = measure_configs(torch, ctx, tensors, copies)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.workload, budget_s=12.0)
        try:
            line["reference_gpu"] = reference_gpu_baseline(args.workload)
        except Exception as error:  # the second baseline must never break the benchmark line
            line["reference_gpu"] = {"unavailable": str(error)[:120]}
    if rank == 0:
        print(json.dumps(mark_library(line)))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


SHARDED = {
    # BASELINE config 4: LM head 8192 -> 151936, rows of w split over the ranks, all-gather of y
    "lm_head_colsplit": {"n": 151936, "k": 8192},
    # BASELINE config 3: Qwen3-30B-A3B-shaped routed experts, expert parallel over the ranks
    "moe_qwen3_30b_a3b": {"tokens": 512, "experts": 128, "used": 8, "hidden": 2048, "ffn": 768},
}


def setup_lm_head(torch, ctx, world, rank, m, fused, copies=2):
    """BASELINE config 4, LM head: rows of w split over the ranks.  Returns (step, bytes, launches,
    config, result) where result() is the y[m][n] of the last step on this rank."""
    import aotx_b200
    from aotx_b200.sharded import column_split_on_gpu, shard_rows
    spec = SHARDED["lm_head_colsplit"]
    n, k = spec["n"], spec["k"]
    first, last = shard_rows(n, world, rank)
    shards = [aotx_b200.synth_q8_0_device(last - first, k, 7000 + 10 * rank + c) for c in range(copies)]
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(m, k, device="cuda", generator=gen).to(torch.bfloat16)
    state = {}
    if fused and world > 1:
        from aotx_b200.sharded import ColumnSplitFused
        objects = [ColumnSplitFused(ctx, w, n, k, world, rank, m, torch.bfloat16) for w in shards]

        # One barrier per step is enough here even inside a graph: the step rotates over
        # `copies` >= 2 of these objects, so another barrier of the same ranks lies between
        # two uses of one object's buffer.
        def step(c):
            state["y"] = objects[c].matmul(x, m, opening_barrier=False if copies >= 2 else None)
    else:
        splits = [column_split_on_gpu(ctx, w, n, k, world, rank, y_dtype=torch.bfloat16) for w in shards]
        out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

        def step(c):
            state["y"] = splits[c].matmul(x, m, out=out)

    step_bytes = n * (k // 32) * 34 + m * k * 2 + m * n * 2
    config = {"workload": "lm_head_colsplit", "rows": m, "n": n, "k": k, "x": "bfloat16", "y": "bfloat16",
              "parallelism": "single" if world == 1 else
              ("column split x%d, slices stored into peers by the kernel" if fused
               else "column split x%d + all-gather") % world}
    # launches per step: the product and, where the slices go to the peers, the barrier
    return step, step_bytes, 2 if (fused and world > 1) else 1, config, (lambda: state.get("y")), x


def setup_moe(torch, ctx, world, rank, moe_fused=False, copies=2):
    """BASELINE config 3: Qwen3-30B-A3B-shaped routed experts, expert parallel over the ranks."""
    import aotx_b200
    from aotx_b200.sharded import shard_rows
    spec = SHARDED["moe_qwen3_30b_a3b"]
    tokens, experts, used = spec["tokens"], spec["experts"], spec["used"]
    hidden, ffn = spec["hidden"], spec["ffn"]
    e0, e1 = shard_rows(experts, world, rank)
    t0, t1 = shard_rows(tokens, world, rank)
    local = e1 - e0
    sets = []
    for c in range(copies):
        sets.append(tuple(aotx_b200.synth_q8_0_device(local * r, kk, 8000 + 100 * c + 10 * rank + i)
                          for i, (r, kk) in enumerate(((ffn, hidden), (ffn, hidden), (hidden, ffn)))))
    gen = torch.Generator(device="cuda").manual_seed(11)
    x_all = torch.randn(tokens, hidden, device="cuda", generator=gen).half()
    router = (torch.randn(experts, hidden, device="cuda", generator=gen) / hidden ** 0.5).float()
    prob_all, ids_all = ctx.moe_route(x_all, router, used)
    x_loc, prob, ids = x_all[t0:t1].contiguous(), prob_all[t0:t1].contiguous(), ids_all[t0:t1].contiguous()
    if world == 1:
        ws = ctx.moe_workspace(tokens, used, hidden, ffn)
        out = torch.empty((tokens, hidden), dtype=torch.float32, device="cuda")
        if moe_fused:
            # gate and up of every expert as one tensor with the rows interleaved
            both = [torch.from_numpy(aotx_b200.interleave_rows(g.cpu().numpy(), u.cpu().numpy(), hidden,
                                                               groups=experts)).cuda()
                    for g, u, _ in sets]

            def step(c):
                ctx.moe_ffn_fused(both[c], sets[c][2], experts, hidden, ffn, x_loc, prob, ids, out=out,
                                  workspace=ws)
        else:
            def step(c):
                ctx.moe_ffn(*sets[c], experts, hidden, ffn, x_loc, prob, ids, out=out, workspace=ws)
    else:
        # the exchange folded into the library's kernels (aotx_q8_moe_ep): rows and projections
        # are read straight from the GPU that holds them, two barriers of the library's own
        from aotx_b200.sharded import ExpertParallelFused
        eps = [ExpertParallelFused(ctx, *sets[c], experts, used, hidden, ffn, world, rank, t1 - t0)
               for c in range(copies)]

        def step(c):
            eps[c].ffn(x_loc, prob, ids)

    hit = int((torch.bincount(ids_all.reshape(-1).long(), minlength=experts) > 0).sum())
    slice_bytes = 2 * ffn * (hidden // 32) * 34 + hidden * (ffn // 32) * 34
    step_bytes = hit * slice_bytes + tokens * hidden * 2 + tokens * hidden * 4
    # one GPU: table, gather, gate, up, gated unit, down, sum (interleaved: one product and no
    # gated-unit kernel less); expert parallel adds two barriers and the collection of the ids
    launches = (5 if moe_fused else 7) if world == 1 else 10
    config = {"workload": "moe_qwen3_30b_a3b", "interleaved_gate_up": bool(moe_fused and world == 1),
              "tokens": tokens, "experts": experts, "used": used,
              "hidden": hidden, "ffn": ffn, "experts_hit": hit, "x": "float16", "y": "float32",
              "router": "selections made once outside the timed region",
              "parallelism": ("expert parallel x%d, rows and projections read from the peers by the "
                              "library's kernels" % world) if world > 1 else "single"}
    return step, step_bytes, launches, config


def steps_per_graph(steps, most=4):
    """How many consecutive steps one captured graph holds: as many as divide `steps` exactly
    (so that exactly `steps` steps are timed), up to `most`."""
    for group in range(most, 1, -1):
        if steps % group == 0:
            return group
    return 1


def time_steps(torch, step, copies, steps, warmup, world, capture=True, group=1):
    """Warm up, then time `steps` steps that rotate over `copies` weight copies: CUDA events
    between two barriers, the maximum over the ranks.  The steps are captured into CUDA graphs
    where that works, `group` consecutive steps to a graph (the reference's decode graph holds a
    whole forward pass; inside one graph consecutive launches overlap as they do in a model,
    between two graph launches they do not); `steps` must be a multiple of `group`.  Returns
    (total ms, captured, run) - `run(i)` runs the i-th group of steps."""
    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    assert steps % group == 0
    step(0)
    barrier()
    graphs = None
    distinct = copies // math.gcd(copies, group)   # graphs after which the rotation repeats
    if capture:
        try:
            graphs = []
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for j in range(distinct):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        for i in range(group):
                            step((j * group + i) % copies)
                    graphs.append(g)
            torch.cuda.synchronize()
        except Exception:
            graphs = None

    def eager(j):
        for i in range(group):
            step((j * group + i) % copies)

    run = (lambda j: graphs[j % distinct].replay()) if graphs else eager
    for i in range(max(warmup, 3)):
        run(i)
    barrier()
    e0_, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0_.record()
    for i in range(steps // group):
        run(i)
    e1_.record()
    barrier()
    total_ms = e0_.elapsed_time(e1_)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t[0])
    return total_ms, bool(graphs), run


def leave_together(torch, world):
    """Graphs that hold captured collectives must go before the process group does; tearing the
    group down first left every rank waiting at exit."""
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def run_sharded(args, rank, world, local_rank):
    """Strong-scaling workloads: the total work is fixed, the ranks split it."""
    import torch
    import aotx_b200

    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = aotx_b200.Q8Context(local_rank)
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    copies = 2
    if args.workload == "lm_head_colsplit":
        step, step_bytes, launches, config, _, _ = setup_lm_head(torch, ctx, world, rank, args.rows, args.fused, copies)
        capture = True
    else:
        step, step_bytes, launches, config = setup_moe(torch, ctx, world, rank, args.moe_fused, copies)
        capture = world == 1
    sampler = ClockSampler(device_index(local_rank))
    sampler.start()
    total_ms, captured, run = time_steps(torch, step, copies, args.steps, args.warmup, world, capture)
    sampler.stop_flag.set()
    sampler.join()
    status = ctx.device_status()
    value = step_bytes * args.steps / (total_ms * 1e-3) / 1e9
    config["cuda_graph"] = captured
    config["l2"] = "two weight copies rotate; each larger than L2 at N=1"
    line = {
        "metric": "q8_decode_gemm_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16/bf16 operands, f32 sums", "data": "synthetic", "config": config,
        "roofline": {"bound": "hbm", "achieved": value / world, "peak": hbm_peak, "unit": "GB/s",
                     "frac": value / world / hbm_peak, "traffic": None, "peak_source": peak_kind,
                     "note": "per GPU, whole step including the exchange"},
        "gpu_launches": launches * args.steps, "clocks": sampler.summary(), "device_status": status,
    }
    if rank == 0:
        print(json.dumps(mark_library(line)), flush=True)
    run = None
    leave_together(torch, world)


def summary(workload, ms, step_bytes=None, step_flops=None, **more):
    """One entry of `configs` / `sharded`: time per step and the fraction of the binding roofline."""
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    entry = {"workload": workload, "ms_per_step": ms}
    if step_flops is not None:
        achieved = step_flops / (ms * 1e-3) / 1e12
        entry.update({"achieved": achieved, "unit": "TFLOP/s", "bound": "tensor", "peak": tensor_peak,
                      "frac": achieved / tensor_peak})
    else:
        achieved = step_bytes / (ms * 1e-3) / 1e9
        entry.update({"achieved": achieved, "unit": "GB/s", "bound": "hbm", "peak": hbm_peak,
                      "frac": achieved / hbm_peak})
    entry["peak_source"] = peak_kind
    entry.update(more)
    return entry


# shapes of the brief measurements (module level so that a dry run can shrink them)
GEMV_SHAPE = {"n": 4096, "k": 4096, "copies": 24}
PREFILL_ROWS = 2048


def measure_configs(torch, ctx, layer, copies, steps=40):
    """Configurations 0, 2, 3 and the LM head of configuration 4 on this GPU: a few dozen steps
    each after three warm-up steps, weight copies rotating (larger than L2 in total)."""
    import aotx_b200
    out = []
    # configuration 0: one row of x against 4096 x 4096, half in and out
    n, k, many = GEMV_SHAPE["n"], GEMV_SHAPE["k"], GEMV_SHAPE["copies"]
    ws = [aotx_b200.synth_q8_0_device(n, k, 300 + c) for c in range(many)]
    x = torch.randn(1, k, device="cuda").half()
    y = torch.empty(1, n, dtype=torch.float16, device="cuda")
    # one captured graph holds a launch per weight copy (as the reference's decode graph holds
    # a layer's products): a graph of a single 13 us kernel would time the graph launches

    def gemv(c):
        for w in ws:
            ctx.matmul(w, n, k, x, y=y)

    ms, _, _ = time_steps(torch, gemv, 1, 8, 3, 1)
    out.append(summary("gemv_m1_4096", ms / (many * 8), step_bytes=n * (k // 32) * 34 + k * 2 + n * 2, rows=1,
                       us_per_launch=ms / (many * 8) * 1e3, launches_per_graph=many))
    del ws
    # configuration 2: the same layer at 2048 rows, bfloat16 in and out
    m = PREFILL_ROWS
    xs = [torch.randn(m, t["k"], device="cuda").to(torch.bfloat16) for t in layer]
    ys = [torch.empty(m, t["n"], dtype=torch.bfloat16, device="cuda") for t in layer]

    def prefill(c):
        for t, xx, yy in zip(layer, xs, ys):
            ctx.matmul(t["w"][c], t["n"], t["k"], xx, y=yy)

    ms, _, _ = time_steps(torch, prefill, copies, steps, 3, 1, group=steps_per_graph(steps))
    projections = [(t["name"], t["k"], t["n"]) for t in layer]
    out.append(summary("prefill_m2048_llama3_8b_layer", ms / steps, step_flops=flops(m, projections), rows=m,
                       tokens_per_s=m * steps / (ms * 1e-3)))
    del xs, ys
    # configuration 3: routed experts, 512 tokens, 128 experts, 8 used
    # in both forms: gate and up as the model file holds them (two tensors), and interleaved
    # at load into one (aotx_gguf_upload_rows) with the gated unit in the product's store
    step, step_bytes, launches, config = setup_moe(torch, ctx, 1, 0)
    ms, _, run = time_steps(torch, step, 2, steps, 3, 1, group=steps_per_graph(steps))
    run = step = None
    torch.cuda.empty_cache()
    step, _, launches_one, _ = setup_moe(torch, ctx, 1, 0, moe_fused=True)
    ms_one, _, run = time_steps(torch, step, 2, steps, 3, 1, group=steps_per_graph(steps))
    best = min(ms, ms_one)
    out.append(summary("moe_qwen3_30b_a3b", best / steps, step_bytes=step_bytes,
                       launches_per_step=launches_one if ms_one <= ms else launches,
                       experts_hit=config["experts_hit"], interleaved_gate_up=bool(ms_one <= ms),
                       us_separate_tensors=ms / steps * 1e3, us_interleaved=ms_one / steps * 1e3))
    run = step = None
    # configuration 4: the LM head on one GPU, 8 rows
    step, step_bytes, launches, config, _, _ = setup_lm_head(torch, ctx, 1, 0, 8, False)
    ms, _, run = time_steps(torch, step, 2, steps, 3, 1, group=steps_per_graph(steps))
    out.append(summary("lm_head_8192_to_151936_m8", ms / steps, step_bytes=step_bytes, rows=8))
    run = step = None
    torch.cuda.empty_cache()
    return out


def run_scaling(args, rank, world, local_rank):
    """N > 1: what shards.  The headline is the LM head column split at 8 rows (strong scaling,
    the gather in the kernel's own stores); `sharded` adds 64 rows and the expert-parallel routed
    experts, each with the one-GPU time of the same run."""
    import torch
    import torch.distributed as dist
    import aotx_b200

    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = aotx_b200.Q8Context(local_rank)
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    copies = 2
    short = max(10, min(args.steps, 100))
    sharded = {}

    # one-GPU figures first (every rank runs them on its own GPU; rank 0's are reported)
    single = {}
    for rows in (8, 64):
        step, step_bytes, _, _, _, _ = setup_lm_head(torch, ctx, 1, 0, rows, False, copies)
        ms, _, run = time_steps(torch, step, copies, short, 3, 1, group=steps_per_graph(short))
        single["lm_head_m%d" % rows] = ms / short
        run = step = None
        torch.cuda.empty_cache()
    step, moe_bytes, _, _ = setup_moe(torch, ctx, 1, 0, False, copies)
    ms, _, run = time_steps(torch, step, copies, short, 3, 1, group=steps_per_graph(short))
    single["moe"] = ms / short
    run = step = None
    torch.cuda.empty_cache()
    dist.barrier()

    # the headline: LM head, 8 rows, fused column split
    step, step_bytes, launches, config, result, x_dev = setup_lm_head(torch, ctx, world, rank, 8, True, copies)
    sampler = ClockSampler(device_index(local_rank))
    sampler.start()
    group = steps_per_graph(args.steps)
    total_ms, captured, run = time_steps(torch, step, copies, args.steps, args.warmup, world, group=group)
    sampler.stop_flag.set()
    sampler.join()
    value = step_bytes * args.steps / (total_ms * 1e-3) / 1e9
    # end to end: x from pinned host memory every step, the gathered y back to the host
    x_host = x_dev.cpu().pin_memory()
    y_host = torch.empty((8, config["n"]), dtype=torch.bfloat16).pin_memory()

    def step_e2e(c):
        x_dev.copy_(x_host, non_blocking=True)
        step(c)
        y_host.copy_(result(), non_blocking=True)

    e2e_ms, e2e_captured, run_e2e = time_steps(torch, step_e2e, copies, args.steps, 3, world, group=group)
    e2e_value = step_bytes * args.steps / (e2e_ms * 1e-3) / 1e9
    sharded["lm_head_m8"] = summary("lm_head_colsplit", total_ms / args.steps, step_bytes=step_bytes, rows=8,
                                    one_gpu_ms=single["lm_head_m8"],
                                    speedup_over_one_gpu=single["lm_head_m8"] / (total_ms / args.steps),
                                    frac_per_gpu=value / world / hbm_peak)
    run = run_e2e = None

    step64, bytes64, _, _, _, _ = setup_lm_head(torch, ctx, world, rank, 64, True, copies)
    ms64, _, run = time_steps(torch, step64, copies, short, 3, world, group=steps_per_graph(short))
    sharded["lm_head_m64"] = summary("lm_head_colsplit", ms64 / short, step_bytes=bytes64, rows=64,
                                     one_gpu_ms=single["lm_head_m64"],
                                     speedup_over_one_gpu=single["lm_head_m64"] / (ms64 / short),
                                     frac_per_gpu=bytes64 * short / (ms64 * 1e-3) / 1e9 / world / hbm_peak)
    run = step64 = None
    torch.cuda.empty_cache()

    step_moe, moe_bytes, _, moe_config = setup_moe(torch, ctx, world, rank, False, copies)
    ms_moe, moe_captured, run = time_steps(torch, step_moe, copies, short, 3, world, group=steps_per_graph(short))
    sharded["moe_expert_parallel"] = summary("moe_qwen3_30b_a3b", ms_moe / short, step_bytes=moe_bytes,
                                             one_gpu_ms=single["moe"],
                                             speedup_over_one_gpu=single["moe"] / (ms_moe / short),
                                             frac_per_gpu=moe_bytes * short / (ms_moe * 1e-3) / 1e9 / world / hbm_peak)
    run = step_moe = None
    status = ctx.device_status()
    config["cuda_graph"] = captured
    config["steps_per_graph"] = group
    config["l2"] = "two weight copies rotate; the whole tensor is ten times L2"
    sharded["moe_expert_parallel"]["cuda_graph"] = moe_captured
    line = {
        "metric": "q8_decode_gemm_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16/bf16 operands, f32 sums", "data": "synthetic", "config": config,
        "roofline": {"bound": "hbm", "achieved": value / world, "peak": hbm_peak, "unit": "GB/s",
                     "frac": value / world / hbm_peak, "traffic": None, "peak_source": peak_kind,
                     "kernel": "q8_decode_kernel", "note": "per GPU, whole step including the exchange"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": y_host.numel() * 2, "ms_per_step": e2e_ms / args.steps,
                "mode": ("captured graphs" if e2e_captured else "eager calls")
                + ", x up from pinned host memory and the gathered y down to it on every rank, every step"},
        "sharded": sharded,
        "gpu_launches": launches * args.steps, "clocks": sampler.summary(), "device_status": status,
    }
    if rank == 0:
        print(json.dumps(mark_library(line)), flush=True)
    leave_together(torch, world)


def cpu_sample(workload, fraction):
    """A bounded sample of the workload for the host cores: the first `fraction` of the rows
    of every projection, at the full batch and depth, fp16 activations (the reference's host
    code reads halves only)."""
    import aotx_b200
    m, projections, _, _ = WORKLOADS[workload]
    rng = np.random.Generator(np.random.PCG64(99))
    parts = []
    for index, (name, k, n) in enumerate(projections):
        rows = max(8, int(n * fraction) // 8 * 8)
        w = aotx_b200.synth_q8_0(rows, k, 900 + index)
        x = rng.standard_normal((m, k)).astype(np.float16).view(np.uint16)
        parts.append((name, k, rows, w, x))
    return m, parts


def time_cpu(workload, fraction, want_reference=True):
    """One pass of the sample on all host cores.  Uses the reference's own compiled host
    product when that library is present, else the oracle's restatement of it."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle.binding import Oracle, Reference
    cores = os.cpu_count() or 1
    m, parts = cpu_sample(workload, fraction)
    ref = Reference() if want_reference else None
    kind = "reference" if (ref is not None and ref.available) else "port"
    oracle = Oracle()
    begin = time.perf_counter()
    for name, k, rows, w, x in parts:
        if kind == "reference":
            # the reference's product is one thread; split the rows over the cores
            per = max(1, (rows + cores - 1) // cores)
            slices = [(r0, min(rows, r0 + per)) for r0 in range(0, rows, per)]
            stride = (k // 32) * 34

            def one(span):
                r0, r1 = span
                return ref.product(w[r0 * stride:r1 * stride], r1 - r0, k, x, m)

            with ThreadPoolExecutor(cores) as pool:
                list(pool.map(one, slices))
        else:
            oracle.product(w, rows, k, x, m, threads=cores)
    seconds = time.perf_counter() - begin
    sample_bytes = sum(rows * (k // 32) * 34 + m * k * 2 + m * rows * 4 for _, k, rows, _, _ in parts)
    sample_flops = sum(2 * m * rows * k for _, k, rows, _, _ in parts)
    return kind, cores, seconds, sample_bytes, sample_flops


def reference_gpu_baseline(workload):
    """Second baseline: the reference's own CUDA kernels (cuda/model/gemm.cu / gemv.cu), compiled
    unmodified for sm_100a into the checker library, on the same step (half x, float y, as the
    reference has them).  Like the CPU baseline this is a reported number, never the product."""
    import torch
    from oracle.binding import Reference
    import aotx_b200
    ref = Reference()
    if not ref.available:
        return None
    m, projections, _, _ = WORKLOADS[workload]
    tensors = []
    for index, (name, k, n) in enumerate(projections):
        w = torch.from_numpy(aotx_b200.synth_q8_0(n, k, 4000 + index)).cuda()
        x = torch.randn(m, k, device="cuda").half()
        y = torch.empty(m, n, device="cuda", dtype=torch.float32)
        tensors.append((w, n, k, x, y))
    # the reference's regime switch: tensor-core kernel from 17 rows (cuda/model/forward.cuh:43-55)
    fn = ref.lib.ref_gpu_gemm if m >= 17 else ref.lib.ref_gpu_gemv
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        for w, n, k, x, y in tensors:
            fn(w.data_ptr(), n, k, x.data_ptr(), m, y.data_ptr(), stream)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 10
    e0.record()
    for _ in range(reps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    step_bytes = algorithmic_bytes(m, projections, 2, 4)
    return {"kernel": "aotx_model_gemm" if m >= 17 else "aotx_model_gemv", "ms_per_step": ms,
            "value": step_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
            "tflops": flops(m, projections) / (ms * 1e-3) / 1e12,
            "note": "reference kernels recompiled for sm_100a, weights warm in L2 where they fit"}


def cpu_baseline(workload, budget_s):
    kind, cores, seconds, sample_bytes, sample_flops = time_cpu(workload, 1.0 / 64.0)
    # grow the sample toward the budget, once
    fraction = min(1.0, (1.0 / 64.0) * max(1.0, budget_s / max(seconds, 1e-3) / 2.0))
    kind, cores, seconds, sample_bytes, sample_flops = time_cpu(workload, fraction)
    tensor_bound = workload in TENSOR_BOUND
    value = sample_flops / seconds / 1e12 if tensor_bound else sample_bytes / seconds / 1e9
    return {"value": value, "unit": "TFLOP/s" if tensor_bound else "GB/s", "cores": cores, "kind": kind,
            "sample": "first %.4f of the rows of each projection, full batch and depth, fp16 x, "
                      "double sums; %.2f s" % (fraction, seconds),
            "gflops": sample_flops / seconds / 1e9}


def run_reference(args, rank, world):
    """The reference's own CPU implementation of the product (its host check code), all host
    threads, on a bounded sample of the same workload per step."""
    if rank != 0:
        return
    tensor_bound = args.workload in TENSOR_BOUND
    # size one step to about a second
    kind, cores, seconds, sample_bytes, sample_flops = time_cpu(args.workload, 1.0 / 128.0)
    fraction = min(1.0, (1.0 / 128.0) * max(1.0, 1.0 / max(seconds, 1e-3)))
    warmups = min(max(args.warmup, 1), 3)  # a pass is about a second of all cores
    for _ in range(warmups):
        time_cpu(args.workload, fraction)
    total = 0.0
    for _ in range(args.steps):
        kind, cores, seconds, sample_bytes, sample_flops = time_cpu(args.workload, fraction)
        total += seconds
    value = (sample_flops * args.steps / total / 1e12) if tensor_bound \
        else (sample_bytes * args.steps / total / 1e9)
    unit = "TFLOP/s" if tensor_bound else "GB/s"
    m, projections, x_name, y_name = WORKLOADS[args.workload]
    sample = ("first %.4f of the rows of each projection, full batch and depth, per step" % fraction)
    line = {
        "impl": "reference",
        "metric": "q8_prefill_gemm_tflops" if tensor_bound else "q8_decode_gemm_hbm_gbs",
        "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": warmups,
        "ms_per_step": total / args.steps * 1e3, "higher_is_better": True,
        # the same names as this arm's own line at this N (the LM head is split over the ranks there)
        "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "f64 sums over f16", "data": "synthetic",
        "config": ({"workload": "lm_head_colsplit", "rows": m, "n": projections[0][2], "k": projections[0][1],
                    "x": "float16", "y": "float64", "parallelism": "host cores of rank 0"} if world > 1 else
                   {"workload": args.workload, "rows": m, "x": "float16", "y": "float64",
                    "projections": {name: [k, n] for name, k, n in projections}}),
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=2000)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--workload", default=None, choices=sorted(WORKLOADS) + sorted(SHARDED),
                        help="one workload alone; by default the line covers every configuration")
    parser.add_argument("--rows", type=int, default=8, help="rows of x for lm_head_colsplit")
    parser.add_argument("--fused", action="store_true",
                        help="lm_head_colsplit: store the slices into the peers instead of an all-gather")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-configs", action="store_true",
                        help="one GPU, default workload: leave out the `configs` measurements")
    parser.add_argument("--moe-fused", action="store_true",
                        help="moe_qwen3_30b_a3b on one GPU: interleaved gate+up tensor, gated unit in the store")
    args = parser.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    args.composite = args.workload is None and not args.no_configs
    if args.workload is None:
        if world > 1 and args.impl != "reference":
            run_scaling(args, rank, world, local_rank)
            return
        # the reference arm follows the headline: the LM head where the ranks split it
        args.workload = "lm_head_m8" if world > 1 else "decode_m32_llama3_8b_layer"
    if args.impl == "reference":
        if args.steps > 20:
            args.steps = 20
        run_reference(args, rank, world)
        return
    if args.workload in SHARDED:
        run_sharded(args, rank, world, local_rank)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
