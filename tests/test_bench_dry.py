"""A dry run of bench.py's device path on the CPU: the context is the oracle-backed stand-in of
tests/_fake.py, streams / events / graphs are inert stand-ins, the workload is shrunk.  It
checks the benchmark's own code - the loop structure, the JSON line and its keys - not any
number in it."""
import importlib
import io
import json
import sys
import types

import numpy as np
import pytest
import torch as real_torch

import _fake


class Event:
    def __init__(self, enable_timing=False):
        pass

    def record(self, stream=None):
        pass

    def elapsed_time(self, other):
        return 1.0

    def synchronize(self):
        pass


class Stream:
    cuda_stream = 0

    def wait_stream(self, other):
        pass

    def wait_event(self, event):
        pass


class Graph:
    def replay(self):
        pass


class Scope:
    def __init__(self, *args, **kwargs):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class DryCuda:
    Event, Stream, CUDAGraph, graph, stream = Event, Stream, Graph, Scope, Scope

    @staticmethod
    def set_device(device):
        pass

    @staticmethod
    def synchronize(*args):
        pass

    @staticmethod
    def current_stream(*args):
        return Stream()

    @staticmethod
    def is_available():
        return True

    @staticmethod
    def empty_cache():
        pass


class DryTorch(_fake.FakeTorch):
    cuda = DryCuda()

    def Generator(self, *args, **kwargs):
        return real_torch.Generator()

    def randn(self, *args, **kwargs):
        kwargs.pop("device", None)
        kwargs.pop("generator", None)
        return real_torch.randn(*args, **kwargs)


def _host_synth(n, k, seed, device="cuda"):
    """The device-side generator of the harness, on the host for the dry run."""
    import aotx_b200
    return real_torch.from_numpy(aotx_b200.synth_q8_0(n, k, seed))


@pytest.mark.parametrize("workload,extra", [("decode_m32_llama3_8b_layer", []),
                                            ("decode_m32_llama3_8b_layer_fused", []),
                                            ("prefill_m2048_llama3_8b_layer", [])])
def test_default_benchmark_path_runs_to_its_json_line(monkeypatch, capsys, workload, extra):
    import aotx_b200
    bench = importlib.import_module("bench")
    small = [("qkv", 256, 96), ("o", 256, 64), ("gate_up", 256, 128), ("down", 512, 64)]
    rows = 8 if "decode" in workload else 40
    monkeypatch.setitem(bench.WORKLOADS, workload, (rows, small, "bfloat16", "bfloat16"))
    fake = DryTorch()
    monkeypatch.setitem(sys.modules, "torch", fake)
    monkeypatch.setattr(aotx_b200, "Q8Context", _fake.FakeContext)
    monkeypatch.setattr(real_torch.Tensor, "cuda", lambda self, *a, **k: self)
    monkeypatch.setattr(real_torch.Tensor, "pin_memory", lambda self, *a, **k: self)
    monkeypatch.setattr(bench, "reference_gpu_baseline", lambda name: {"unavailable": "dry run"})
    monkeypatch.setattr(bench, "cpu_baseline", lambda name, budget_s: {"value": 0.0, "kind": "dry run"})
    monkeypatch.setattr(aotx_b200, "synth_q8_0_device", _host_synth)
    monkeypatch.setattr(sys, "argv", ["bench.py", "--steps", "3", "--warmup", "1", "--workload", workload] + extra)
    bench.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "roofline", "e2e", "gpu_launches", "clocks",
                "cpu_baseline"):
        assert key in line, key
    for key in ("bound", "achieved", "peak", "unit", "frac", "traffic"):
        assert key in line["roofline"], key
    for key in ("value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"):
        assert key in line["e2e"], key
    assert line["config"]["workload"] == workload and line["steps"] == 3 and line["n_gpus"] == 1
    assert line["gpu_launches"] == 4 * 3
    assert line["e2e"]["host_result_matches_device"] is True


@pytest.mark.parametrize("workload,extra", [("lm_head_colsplit", ["--rows", "4"]),
                                            ("moe_qwen3_30b_a3b", []),
                                            ("moe_qwen3_30b_a3b", ["--moe-fused"])])
def test_sharded_workloads_run_on_one_rank(monkeypatch, capsys, workload, extra):
    import aotx_b200
    bench = importlib.import_module("bench")
    monkeypatch.setitem(bench.SHARDED, "lm_head_colsplit", {"n": 200, "k": 256})
    monkeypatch.setitem(bench.SHARDED, "moe_qwen3_30b_a3b",
                        {"tokens": 12, "experts": 4, "used": 2, "hidden": 256, "ffn": 256})
    fake = DryTorch()
    monkeypatch.setitem(sys.modules, "torch", fake)
    monkeypatch.setattr(aotx_b200, "Q8Context", _fake.FakeContext)
    monkeypatch.setattr(real_torch.Tensor, "cuda", lambda self, *a, **k: self)
    monkeypatch.setattr(aotx_b200, "synth_q8_0_device", _host_synth)
    monkeypatch.setattr(sys, "argv", ["bench.py", "--steps", "2", "--warmup", "1", "--workload", workload] + extra)
    bench.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["config"]["workload"] == workload and line["scaling"] == "strong" and line["n_gpus"] == 1
    assert line["value"] > 0 and "roofline" in line and "clocks" in line
    if workload.startswith("moe"):
        assert line["config"]["interleaved_gate_up"] == bool(extra)


def test_default_line_covers_every_configuration(monkeypatch, capsys):
    """No --workload on one GPU: the decode layer as the headline and a `configs` entry for the
    single-row product, the prefill layer, the routed experts and the LM head."""
    import aotx_b200
    bench = importlib.import_module("bench")
    small = [("qkv", 256, 96), ("o", 256, 64), ("gate_up", 256, 128), ("down", 512, 64)]
    monkeypatch.setitem(bench.WORKLOADS, "decode_m32_llama3_8b_layer", (8, small, "bfloat16", "bfloat16"))
    monkeypatch.setitem(bench.SHARDED, "lm_head_colsplit", {"n": 200, "k": 256})
    monkeypatch.setitem(bench.SHARDED, "moe_qwen3_30b_a3b",
                        {"tokens": 12, "experts": 4, "used": 2, "hidden": 256, "ffn": 256})
    monkeypatch.setattr(bench, "GEMV_SHAPE", {"n": 64, "k": 256, "copies": 2})
    monkeypatch.setattr(bench, "PREFILL_ROWS", 40)
    monkeypatch.setitem(sys.modules, "torch", DryTorch())
    monkeypatch.setattr(aotx_b200, "Q8Context", _fake.FakeContext)
    monkeypatch.setattr(real_torch.Tensor, "cuda", lambda self, *a, **k: self)
    monkeypatch.setattr(real_torch.Tensor, "pin_memory", lambda self, *a, **k: self)
    monkeypatch.setattr(bench, "reference_gpu_baseline", lambda name: {"unavailable": "dry run"})
    monkeypatch.setattr(bench, "cpu_baseline", lambda name, budget_s: {"value": 0.0, "kind": "dry run"})
    monkeypatch.setattr(aotx_b200, "synth_q8_0_device", _host_synth)
    monkeypatch.setattr(sys, "argv", ["bench.py", "--steps", "3", "--warmup", "1"])
    bench.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["config"]["workload"] == "decode_m32_llama3_8b_layer" and line["n_gpus"] == 1
    names = [entry["workload"] for entry in line["configs"]]
    assert names == ["gemv_m1_4096", "prefill_m2048_llama3_8b_layer", "moe_qwen3_30b_a3b",
                     "lm_head_8192_to_151936_m8"]
    for entry in line["configs"]:
        for key in ("ms_per_step", "achieved", "unit", "bound", "frac", "peak"):
            assert key in entry, key


def test_smoke_entry_runs_on_the_stand_in(monkeypatch, capsys):
    """__graft_entry__.smoke(): the same dry run (its checks are real: the stand-in's results
    come from the oracle, so they pass; a mistake in the smoke's own code would not)."""
    import aotx_b200
    entry = importlib.import_module("__graft_entry__")
    monkeypatch.setitem(sys.modules, "torch", DryTorch())
    monkeypatch.setattr(aotx_b200, "Q8Context", _fake.FakeContext)
    monkeypatch.setattr(real_torch.Tensor, "cuda", lambda self, *a, **k: self)
    entry.smoke()
    assert "smoke ok" in capsys.readouterr().out
