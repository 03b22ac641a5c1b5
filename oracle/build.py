"""Build recipes for the checker libraries.  TEST INFRASTRUCTURE ONLY.

`build_oracle()` compiles the C restatements beside this file (`q8_oracle.c`, `blocks_oracle.c`)
into `libq8_oracle.so`.
`build_ref()` compiles the reference's own sources, from where they lie in a reference tree,
into `_ref/libaotx_ref.so`, `build_gguf_ref()` the reference's model-file reader into
`_ref/libgguf_ref.so`; both need that tree and are skipped (return None) without it.
Nothing here is imported by the product package.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libq8_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libaotx_ref.so")
REF_MODULE = os.path.join(REF_DIR, "gemv_q8.cubin")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    stamp = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= stamp for s in sources)


def build_oracle(force=False):
    sources = [os.path.join(HERE, "q8_oracle.c"), os.path.join(HERE, "blocks_oracle.c")]
    if not force and _newer(ORACLE_SO, sources):
        return ORACLE_SO
    cmd = ["gcc", "-O3", "-march=native", "-fopenmp", "-fPIC", "-shared", "-std=c11",
           "-ffp-contract=off", "-o", ORACLE_SO, *sources, "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def reference_root():
    """The reference tree: AOTX_REFERENCE_ROOT, else a directory `reference` beside this
    repository.  None when neither holds the reference's matrix test."""
    beside = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    root = os.environ.get("AOTX_REFERENCE_ROOT", beside)
    probe = os.path.join(root, "tests", "matrix_test.cu")
    return root if os.path.exists(probe) else None


def build_ref(force=False):
    """Compile the reference's matrix and routed-expert kernels and host checks, unmodified, for
    sm_100a, and assemble its single-row PTX module (ptx/gemv_q8.ptx) into `_ref/gemv_q8.cubin`."""
    root = reference_root()
    if root is None or shutil.which("nvcc") is None:
        return REF_SO if os.path.exists(REF_SO) else None
    wrap = os.path.join(HERE, "ref_wrap.cu")
    stubs = os.path.join(HERE, "ref_stubs.c")
    if not force and _newer(REF_SO, [wrap, stubs]) and os.path.exists(REF_MODULE):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    stub_obj = os.path.join(REF_DIR, "ref_stubs.o")
    subprocess.run(["gcc", "-O2", "-fPIC", "-c", stubs, "-o", stub_obj], check=True)
    model = os.path.join(root, "cuda", "model")
    cmd = ["nvcc", "-std=c++17", *ARCH, "-rdc=true", "-O2", "-Xcompiler", "-fPIC", "-shared",
           "-diag-suppress", "20044",
           "-I" + os.path.join(root, "cuda"), "-I" + root, "-I" + os.path.join(root, "tests"),
           '-DAOTX_PTX_DIR="%s"' % os.path.join(root, "ptx"),
           "-o", REF_SO, wrap,
           os.path.join(model, "gemv.cu"), os.path.join(model, "gemm.cu"),
           os.path.join(model, "dequant.cu"), os.path.join(model, "experts.cu"),
           os.path.join(model, "expert_matrix.cu"), os.path.join(model, "norm.cu"), stub_obj]
    subprocess.run(cmd, check=True)
    subprocess.run(["ptxas", "-arch=sm_100a", "-o", REF_MODULE, os.path.join(root, "ptx", "gemv_q8.ptx")],
                   check=True)
    return REF_SO


GGUF_REF_SO = os.path.join(REF_DIR, "libgguf_ref.so")


def build_gguf_ref(force=False):
    """Compile the reference's model-file reader (disk/modelfile/gguf.c and meta.c, plain C, no
    dependency outside its own headers), unmodified, from where it lies in the reference tree.
    It is the checker of the product's own reader (aotx_b200/csrc/gguf_table.cpp)."""
    root = reference_root()
    if root is None or shutil.which("gcc") is None:
        return GGUF_REF_SO if os.path.exists(GGUF_REF_SO) else None
    sources = [os.path.join(root, "disk", "modelfile", name) for name in ("gguf.c", "meta.c")]
    if not force and os.path.exists(GGUF_REF_SO):
        return GGUF_REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-I" + root, "-o", GGUF_REF_SO, *sources], check=True)
    return GGUF_REF_SO


KREF_SO = os.path.join(REF_DIR, "libkref_ref.so")


def build_kref(force=False):
    """The reference's host reading of the packed block types (tests/matrix_kref.h), compiled
    from the reference tree through the two-line wrapper kref_wrap.c."""
    root = reference_root()
    if root is None or shutil.which("gcc") is None:
        return KREF_SO if os.path.exists(KREF_SO) else None
    wrap = os.path.join(HERE, "kref_wrap.c")
    if not force and _newer(KREF_SO, [wrap]):
        return KREF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-I" + os.path.join(root, "tests"), "-o", KREF_SO, wrap,
                    "-lm"], check=True)
    return KREF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
    print(build_gguf_ref(force="--force" in sys.argv))
    print(build_kref(force="--force" in sys.argv))
