"""Upload of tensor rows from a GGUF file (aotx_gguf_upload) and a product on what arrived.

The file is written by the tests' own writer; a loader with small pieces moves a rank's rows
of a Q8_0 projection and a range of experts of a stacked tensor to the device through its two
pinned buffers; the device bytes must equal the file bytes, and the product on the uploaded
shard must match the oracle on the same rows."""
import numpy as np
import pytest

import gguf_writer as gw
from _util import check_product, dev, torch_mod, x_fp16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    import aotx_b200
    n, k, experts, ffn = 1000, 1024, 6, 128
    w = aotx_b200.synth_q8_0(n, k, 21)
    stacked = aotx_b200.synth_q8_0(experts * ffn, k, 22)
    big = aotx_b200.synth_q8_0(4096, 4096, 23)
    blob, _ = gw.build([("general.architecture", gw.STRING, "llama")],
                       [{"name": "output.weight", "dims": [k, n], "type": 8, "data": w.tobytes()},
                        {"name": "blk.0.ffn_gate_exps.weight", "dims": [k, ffn, experts], "type": 8,
                         "data": stacked.tobytes()},
                        {"name": "blk.0.ffn_down.weight", "dims": [4096, 4096], "type": 8, "data": big.tobytes()}],
                       alignment=256)
    path = str(tmp_path_factory.mktemp("gguf") / "model.gguf")
    with open(path, "wb") as f:
        f.write(blob)
    return path, (n, k, w), (experts, ffn, stacked), big


@pytest.mark.parametrize("piece", [256 * 1024, 1 << 20, 0])
def test_uploaded_rows_equal_file_rows(model, piece):
    from aotx_b200.gguf import GGUFFile, GGUFLoader
    from aotx_b200.sharded import shard_rows
    import aotx_b200
    torch = torch_mod()
    path, (n, k, w), (experts, ffn, stacked), big = model
    stride = aotx_b200.row_bytes(k)
    loader = GGUFLoader(0, piece)
    try:
        with GGUFFile(path) as f:
            t = f.find("output.weight")
            for world, rank in ((1, 0), (3, 1), (8, 7)):
                first, last = shard_rows(n, world, rank)
                got = loader.upload_rows(f, t, first, last - first)
                torch.cuda.synchronize()
                assert np.array_equal(got.cpu().numpy(), w[first * stride:last * stride])
            e = f.find("blk.0.ffn_gate_exps.weight")
            got = loader.upload_rows(f, e, 2 * ffn, 3 * ffn)
            torch.cuda.synchronize()
            assert np.array_equal(got.cpu().numpy(), stacked[2 * ffn * stride:5 * ffn * stride])
            # long enough for the threaded read of a piece (several slices of 4 MiB)
            d = f.find("blk.0.ffn_down.weight")
            got = loader.upload_rows(f, d, 0, 4096)
            torch.cuda.synchronize()
            assert np.array_equal(got.cpu().numpy(), big)
    finally:
        loader.close()


def test_product_on_an_uploaded_shard(model, oracle):
    """The rows a rank uploads are what its column-split product reads: y[:, first:last]."""
    import aotx_b200
    from aotx_b200.gguf import GGUFFile, GGUFLoader
    from aotx_b200.sharded import shard_rows
    torch = torch_mod()
    path, (n, k, w), _, _ = model
    stride = aotx_b200.row_bytes(k)
    ctx = aotx_b200.Q8Context(0)
    loader = GGUFLoader(0, 512 * 1024)
    try:
        with GGUFFile(path) as f:
            t = f.find("output.weight")
            assert (t.type, t.row_weights, t.rows) == (aotx_b200.Q8_0, k, n)
            first, last = shard_rows(n, 2, 1)
            shard = loader.upload_rows(f, t, first, last - first)
        m = 9
        x = x_fp16(m, k, 5)
        y = ctx.matmul(shard, last - first, k, dev(x))
        torch.cuda.synchronize()
        check_product(oracle, w[first * stride:last * stride], last - first, k, x.view(np.uint16), m,
                      y.cpu().numpy())
        assert ctx.device_status() == 0
    finally:
        loader.close()
        ctx.close()


def test_interleaved_upload_of_gate_and_up(tmp_path):
    """Two tensors uploaded row by row into one with the rows interleaved: the layout the gated
    store reads, equal to what interleave_rows builds on the host."""
    import aotx_b200
    from aotx_b200.gguf import GGUFFile, GGUFLoader
    torch = torch_mod()
    k, ffn, experts = 512, 96, 3
    gate = aotx_b200.synth_q8_0(experts * ffn, k, 31)
    up = aotx_b200.synth_q8_0(experts * ffn, k, 32)
    blob, _ = gw.build([], [{"name": "g", "dims": [k, ffn, experts], "type": 8, "data": gate.tobytes()},
                            {"name": "u", "dims": [k, ffn, experts], "type": 8, "data": up.tobytes()}])
    path = str(tmp_path / "gu.gguf")
    with open(path, "wb") as f:
        f.write(blob)
    loader = GGUFLoader(0, 20000)  # a piece of 36 rows and a bit
    try:
        with GGUFFile(path) as f:
            got = loader.upload_interleaved(f, f.find("g"), f.find("u"))
            part = loader.upload_interleaved(f, f.find("g"), f.find("u"), first_row=ffn, rows=ffn)
        torch.cuda.synchronize()
        want = aotx_b200.interleave_rows(gate, up, k, groups=experts)
        assert np.array_equal(got.cpu().numpy(), want)
        stride = aotx_b200.row_bytes(k)
        assert np.array_equal(part.cpu().numpy(), want[2 * ffn * stride:4 * ffn * stride])
    finally:
        loader.close()
