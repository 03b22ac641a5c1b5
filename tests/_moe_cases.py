"""Routed-expert fixtures shared by the golden-vector script and the tests (test code only).

The small cases restate the fixtures of the reference's tests/expert_test.cu; the large one has
the shape of the benchmark's routed-expert configuration with seeded synthetic values."""
import numpy as np

ROUTE_CASES = [(1, 7, 1, 0), (64, 7, 3, 0), (64, 7, 7, 0), (64, 64, 8, 0), (5, 256, 256, 0), (64, 3, 1, 1)]
SLICE_CASE = dict(experts=5, used=3, n=19, k=512)          # tests/expert_test.cu:274-290
FFN_CASES = {"small": (64, 16, 4, 256, 256, 11), "full": (512, 128, 8, 2048, 768, 900)}
FULL_SAMPLE_TOKENS = 32


def route_fixture(tokens, experts, precision, hidden=32):
    """Router rows and inputs of tests/expert_test.cu:66-89."""
    router = np.zeros((experts, hidden), np.float32)
    for e in range(experts):
        pos = np.float32(e) / np.float32(max(experts - 1, 1))
        for d in range(hidden):
            router[e, d] = (np.float32(1.0002) if e == 2 else np.float32(1.0)) if precision \
                else np.float32((d % 5) - 2) * np.float32(0.0012345)
        if not precision:
            router[e, 0] = np.float32(3.0) * pos
            router[e, 1] = np.float32(-3.0) * pos * pos
    router[1] = router[0]
    x = np.zeros((tokens, hidden), np.float16)
    for t in range(tokens):
        for d in range(hidden):
            x[t, d] = 1.0 if precision else (((t * 7 + d * 3) % 13) - 6) / 16.0
        if not precision:
            x[t, 0] = np.float32(2.0) * np.float32(t) / np.float32(tokens) + np.float32(0.007)
            x[t, 1] = 1.0
    return router, x


def add_fixture(tokens, used, hidden=32):
    """proj[r][t][d] of tests/expert_test.cu:172-173."""
    proj = np.zeros((used, tokens, hidden), np.float32)
    for r in range(used):
        for t in range(tokens):
            for d in range(hidden):
                proj[r, t, d] = np.float32(((t * 11 + d * 7 + r * 3) % 41) - 20) * np.float32(r + 1) \
                    * np.float32(0.03125)
    return proj


def slice_fixture(tokens):
    """Q8_0 weights, inputs and selections of tests/expert_test.cu:203-238, 286-290."""
    experts, used, n, k = (SLICE_CASE[name] for name in ("experts", "used", "n", "k"))
    rows, blocks = experts * n, k // 32
    w = np.zeros((rows, blocks, 34), np.uint8)
    j = np.arange(34, dtype=np.uint64)
    for r in range(rows):
        for b in range(blocks):
            w[r, b] = ((r * 37 + b * 73 + j * 19 + r * j * 3) & 0xFF).astype(np.uint8)
            scale = np.float16(np.float32(1 + (r + b * 3) % 7) / np.float32(128.0))
            w[r, b, :2] = np.frombuffer(scale.tobytes(), np.uint8)
    t = np.arange(tokens, dtype=np.int64)[:, None]
    d = np.arange(k, dtype=np.int64)[None, :]
    x = ((((t * 11 + d * 7 + t * d) % 29) - 14).astype(np.float32) / np.float32(32.0)).astype(np.float16)
    ids = np.array([[(tt * 3 + r * 2 + 1) % experts for r in range(used)] for tt in range(tokens)], np.uint32)
    return w.reshape(-1), x, ids


def ffn_fixture(name):
    """Seeded synthetic tensors of a routed feed-forward step: (tokens, experts, used, hidden, ffn)
    and gate / up / down weights, half inputs, float router."""
    import aotx_b200
    tokens, experts, used, hidden, ffn, seed = FFN_CASES[name]
    wg = aotx_b200.synth_q8_0(experts * ffn, hidden, seed)
    wu = aotx_b200.synth_q8_0(experts * ffn, hidden, seed + 1)
    wd = aotx_b200.synth_q8_0(experts * hidden, ffn, seed + 2)
    rng = np.random.Generator(np.random.PCG64(seed + 3))
    x = rng.standard_normal((tokens, hidden)).astype(np.float16)
    router = rng.standard_normal((experts, hidden)).astype(np.float32) / np.float32(np.sqrt(hidden))
    return (tokens, experts, used, hidden, ffn), wg, wu, wd, x, router


def full_sample_tokens(tokens):
    rng = np.random.Generator(np.random.PCG64(4242))
    return np.sort(rng.permutation(tokens)[:FULL_SAMPLE_TOKENS])
