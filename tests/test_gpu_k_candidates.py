"""The kernels and switches that only a development build reaches (`python -m aotx_b200.build
--experiment`, loaded with AOTX_Q8_LIBRARY=experiment), each in a process of its own because the
switches are read from the environment when the library first launches:

    duo      Q8_DUO=1            the decode-regime kernel as two blocks per SM (q8_duo.cu)
    bfw      Q8_EXPERIMENT=32    bfloat16 activations with bfloat16 weights in tensor memory
    wide     Q8_WIDE_TILE=2      the 256-row prefill kernel with the weights in tensor memory
    keep_x   Q8_EXPERIMENT=64    x tile kept across the row tiles of the grouped down product

For every variant: the same call six times must give the same bits, and the result must agree
with the oracle within the product tolerance.  These are the checks a candidate has to pass on
the GPU before the product build may dispatch it.  The module is skipped unless
AOTX_Q8_CANDIDATES is set and the development build exists, so the ordinary GPU run leaves it
out."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXPERIMENT = os.path.join(ROOT, "aotx_b200", "libaotx_q8_b200_experiment.so")

CHILD = r'''
import json, os, sys
sys.path.insert(0, %r); sys.path.insert(0, os.path.join(%r, "tests"))
import numpy as np, torch
import aotx_b200
from oracle.binding import Oracle
oracle = Oracle()
ctx = aotx_b200.Q8Context(0)
kind = os.environ["CANDIDATE_KIND"]
out = []
if kind == "product":
    for n, k, m, bf in json.loads(os.environ["CANDIDATE_SHAPES"]):
        w = aotx_b200.synth_q8_0(n, k, 8)
        x = torch.randn(m, k, device="cuda").to(torch.bfloat16 if bf else torch.float16)
        wd = torch.from_numpy(w).cuda()
        ys = [ctx.matmul(wd, n, k, x, y=torch.empty(m, n, device="cuda", dtype=torch.float32)) for _ in range(6)]
        torch.cuda.synchronize()
        same = all(bool((y == ys[0]).all()) for y in ys[1:])
        bits = x.view(torch.int16).cpu().numpy().view(np.uint16)
        bad, worst = oracle.spot(w, n, k, bits, m, ys[0].cpu().numpy(), count=256, bf16=bool(bf))
        out.append({"shape": [n, k, m, bf], "same": same, "bad": int(bad), "worst": float(worst),
                    "status": ctx.device_status()})
else:
    tokens, experts, used, hidden, ffn = 200, 7, 2, 512, 768
    wg = aotx_b200.synth_q8_0(experts * ffn, hidden, 1)
    wu = aotx_b200.synth_q8_0(experts * ffn, hidden, 2)
    wd = aotx_b200.synth_q8_0(experts * hidden, ffn, 3)
    x = torch.randn(tokens, hidden, device="cuda").half()
    router = (torch.randn(experts, hidden, device="cuda") / hidden ** 0.5).float()
    prob, ids = ctx.moe_route(x, router, used)
    dev = [torch.from_numpy(t).cuda() for t in (wg, wu, wd)]
    ys = [ctx.moe_ffn(*dev, experts, hidden, ffn, x, prob, ids).clone() for _ in range(6)]
    torch.cuda.synchronize()
    same = all(bool((y == ys[0]).all()) for y in ys[1:])
    want = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x.cpu().numpy().view(np.uint16), prob.cpu().numpy(),
                          ids.cpu().numpy().view(np.uint32))
    ok, err, bound = oracle.within_bound(ys[0].cpu().numpy(), want.astype(np.float64))
    out.append({"shape": "routed experts", "same": same, "bad": 0 if ok else 1, "worst": float(err),
                "status": ctx.device_status()})
print("RESULT " + json.dumps(out))
''' % (ROOT, ROOT)

DECODE = [[4096, 4096, 1, 0], [6144, 4096, 32, 0], [4736, 2048, 20, 0], [28672, 4096, 32, 0]]
DECODE_BF = [[4096, 4096, 32, 1], [4736, 2048, 20, 1], [28672, 4096, 32, 1]]
PREFILL = [[4096, 4096, 2048, 0], [4736, 4096, 300, 0], [4096, 4096, 2048, 1], [28672, 4096, 2048, 1]]

VARIANTS = {
    "duo": ({"Q8_DUO": "1"}, "product", DECODE + DECODE_BF),
    "bfw": ({"Q8_EXPERIMENT": "32"}, "product", DECODE_BF),
    "wide": ({"Q8_WIDE_TILE": "2"}, "product", PREFILL),
    "keep_x": ({"Q8_EXPERIMENT": "64"}, "experts", []),
    "duo_experts": ({"Q8_DUO": "1", "Q8_GROUP_TOKENS": "32"}, "experts", []),
}


@pytest.fixture(scope="module", autouse=True)
def wanted():
    if not os.environ.get("AOTX_Q8_CANDIDATES"):
        pytest.skip("candidates are checked on request (AOTX_Q8_CANDIDATES=1)")
    if not os.path.exists(EXPERIMENT):
        pytest.skip("no development build: python -m aotx_b200.build --experiment")


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_candidate_repeats_and_agrees_with_the_oracle(name):
    switches, kind, shapes = VARIANTS[name]
    env = dict(os.environ, AOTX_Q8_LIBRARY="experiment", CANDIDATE_KIND=kind, CANDIDATE_SHAPES=json.dumps(shapes),
               **switches)
    done = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.startswith("RESULT ")]
    assert lines, done.stdout[-2000:]
    for result in json.loads(lines[-1][7:]):
        assert result["status"] == 0, result
        assert result["same"], result
        assert result["bad"] == 0, result
