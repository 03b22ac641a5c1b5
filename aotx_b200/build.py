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
SOURCES = ["q8_api.cu", "q8_simt.cu", "q8_umma.cu", "q8_stream.cu", "q8_wide.cu", "q8_duo.cu", "q8_static.cu", "q8_moe.cu",
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
    if not _stale(obj, deps):
        return obj, ""
    cmd = ["nvcc", *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s" % (src, done.stderr))
    return obj, done.stderr


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
    print(build(verbose="-v" in sys.argv))
