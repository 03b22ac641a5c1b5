"""Write tests/golden/reference_moe.npz: what the reference's own routed-expert kernels
(cuda/model/experts.cu, expert_matrix.cu, norm.cu:92-105, compiled unmodified into
oracle/_ref/libaotx_ref.so) produce on a GPU for the fixtures of tests/_moe_cases.py.

Needs a CUDA device and the compiled reference library.  Usage (from the repository root):
    python tests/golden/make_golden_moe.py [--out PATH]
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import _moe_cases as cases  # noqa: E402
from oracle.binding import ReferenceExperts  # noqa: E402


def main():
    out = os.path.join(HERE, "reference_moe.npz")
    if "--out" in sys.argv:
        out = sys.argv[sys.argv.index("--out") + 1]
    ref = ReferenceExperts()
    data = {}
    for tokens, experts, used, precision in cases.ROUTE_CASES:
        router, x = cases.route_fixture(tokens, experts, precision)
        prob, ids = ref.route(x, router, used, grid=tokens + 2 if tokens == 1 else 7)
        tag = "route_%d_%d_%d_%d" % (tokens, experts, used, precision)
        data[tag + "_prob"], data[tag + "_ids"] = prob, ids
        proj = cases.add_fixture(tokens, used)
        data[tag + "_sum"] = ref.ordered_sum(proj, prob, ids)
    for tokens in (1, 64):
        w, x, ids = cases.slice_fixture(tokens)
        c = cases.SLICE_CASE
        data["slice_%d" % tokens] = np.stack([ref.expert_matrix(w, c["n"], c["k"], x, ids, rank, c["experts"])
                                              for rank in range(c["used"])])
    for name in cases.FFN_CASES:
        (tokens, experts, used, hidden, ffn), wg, wu, wd, x, router = cases.ffn_fixture(name)
        prob, ids = ref.route(x, router, used)
        result = ref.ffn(wg, wu, wd, experts, hidden, ffn, x, router, used)
        assert np.array_equal(result["ids"], ids)
        data["ffn_%s_prob" % name], data["ffn_%s_ids" % name] = prob, ids
        if name == "full":
            keep = cases.full_sample_tokens(tokens)
            data["ffn_full_tokens"] = keep
            data["ffn_full_sum"] = result["sum"][keep]
        else:
            data["ffn_small_sum"] = result["sum"]
            data["ffn_small_last_act"] = result["act"]
    np.savez_compressed(out, **data)
    print(out, sum(v.nbytes for v in data.values()), "bytes in", len(data), "arrays")


if __name__ == "__main__":
    main()
