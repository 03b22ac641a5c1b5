"""Build recipe of the product library `libaotx_q8_b200.so` (hand-written CUDA for sm_100a).

The library is built in-tree with nvcc; nothing is compiled at import time.  `build()`
rebuilds only the objects whose sources changed.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libaotx_q8_b200.so")
SOURCES = ["q8_api.cu", "q8_simt.cu", "q8_dispatch.cu", "q8_stream.cu", "q8_decode.cu", "q8_wide.cu", "q8_static.cu", "q8_moe.cu", "q8_peers.cu",
           "q_generic.cu", "gguf_table.cpp", "gguf_upload.cu"]
HEADERS = ["q8_common.cuh", "q8_ptx.cuh", "q8_store.cuh", "q8_simt_gemv.cuh", "q8_launch.h", "q8_tile.cuh", "q_blocks.cuh", os.path.join("..", "..", "include", "aotx_q8_b200.h"),
           os.path.join("..", "..", "include", "aotx_gguf_b200.h")]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    stamp = os.path.getmtime(target)
    return any(os.path.getmtime(d) > stamp for d in deps)


def _compile(src):
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    deps = [os.path.join(CSRC, src)] + [os.path.join(CSRC, h) for h in HEADERS]
    log = obj + ".ptxas.log"   # what ptxas -v said for this object: registers, spills, shared memory
    if not _stale(obj, deps) and os.path.exists(log):
        return obj, ""
    cmd = ["nvcc", *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s" % (src, done.stderr))
    with open(log, "w") as f:
        f.write(done.stderr)
    return obj, done.stderr


def resource_usage():
    """{kernel name (mangled): {"registers": r, "spill_stores": s, "spill_loads": l, "stack": b}}
    from the ptxas reports kept beside the objects (build() first)."""
    import re
    usage = {}
    for src in SOURCES:
        log = os.path.join(OBJ, os.path.splitext(src)[0] + ".o.ptxas.log")
        if not os.path.exists(log):
            continue
        name = None
        for line in open(log):
            found = re.search(r"Compiling entry function '([^']+)'", line)
            if found:
                name = found.group(1)
                usage[name] = {}
                continue
            if name is None:
                continue
            found = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
            if found:
                usage[name].update(stack=int(found.group(1)), spill_stores=int(found.group(2)),
                                   spill_loads=int(found.group(3)))
            found = re.search(r"Used (\d+) registers", line)
            if found:
                usage[name]["registers"] = int(found.group(1))
    return usage


TRACE_LIB = os.path.join(HERE, "libaotx_q8_b200_trace.so")


def build_trace():
    """The library with -DQ8_TRACE: the decode kernel writes time stamps (block start, first x
    segment landed, conversion done, accumulator ready, the two cluster barriers, end) that
    aotx_b200/timeline.py reads back.  Never the product build; loaded instead of it when
    AOTX_Q8_LIBRARY=trace (aotx_b200/library.py)."""
    out = os.path.join(OBJ, "trace")
    os.makedirs(out, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f not in ("-Xptxas", "-v")] + ["-DQ8_TRACE"]

    def one(src):
        obj = os.path.join(out, os.path.splitext(src)[0] + ".o")
        done = subprocess.run(["nvcc", *flags, "-c", os.path.join(CSRC, src), "-o", obj], capture_output=True,
                              text=True)
        if done.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (src, done.stderr))
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(one, SOURCES))
    subprocess.run(["nvcc", "-shared", "-o", TRACE_LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                   check=True)
    return TRACE_LIB


def build(verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(_compile, SOURCES))
    objs = [r[0] for r in results]
    log = "".join(r[1] for r in results)
    if log:
        with open(os.path.join(OBJ, "ptxas.log"), "w") as f:
            f.write(log)
    if _stale(LIB, objs):
        subprocess.run(["nvcc", "-shared", "-o", LIB, *objs, "-gencode",
                        "arch=compute_100a,code=sm_100a"], check=True)
    if verbose and log:
        print(log)
    return LIB


if __name__ == "__main__":
    if "--trace" in sys.argv:
        print(build_trace())
    else:
        print(build(verbose="-v" in sys.argv))
