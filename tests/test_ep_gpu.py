"""Expert parallelism on real GPUs. On one device: the exchange kernels against the numpy
restatement of the message layout, and the whole layer with world size 1 (same code path, the
collective degenerates to a copy). With two devices: tests/ep_gpu_check.py under torchrun over NCCL."""
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import moe_math as om
from promoe_b200 import _lib
from promoe_b200.ep import Geometry
from tests.helpers import TinyModel, dev, dev_bf16

pytestmark = pytest.mark.gpu


def test_pack_and_unpack_kernels_follow_the_message_layout(lib):
    """One rank's messages for three owners, and the row list an owner derives from three messages."""
    from tests.test_ep_cpu import OracleBackend
    model = TinyModel(seed=4, L=1, E=10, H=128, I=64, k=3)
    geo = Geometry(model.E, 3, max_tokens_per_rank=7, top_k=model.k, hidden=model.H, n_pred=2)
    rng = np.random.default_rng(1)
    x = om.bf16_round(rng.standard_normal((7, model.H)).astype(np.float32))
    ids, _ = model.canonical_routing(0, x)
    scores = rng.standard_normal((2, model.E)).astype(np.float32)
    ob = OracleBackend(model, geo, rank=1, cache_rate=0.5)
    b = {}
    ob.permute(torch.from_numpy(ids.astype(np.int32)), b)
    want_send, want_pos = ob.pack(torch.from_numpy(x).to(torch.bfloat16), b, scores, 2)
    send = torch.zeros((geo.rows, geo.hidden), dtype=torch.bfloat16, device="cuda")
    pos_reply = torch.full((ids.size,), -7, dtype=torch.int32, device="cuda")
    bounds = dev(np.array(geo.bounds, np.int32))
    keep = [dev(b[n].astype(np.int32)) for n in ("counts", "offsets", "row_token", "pos")]
    xd, scores_d = dev_bf16(x), dev(scores)          # held in variables: the kernel reads them after the call returns
    _lib.call("pm_k_ep_pack", xd.data_ptr(), geo.hidden, keep[0].data_ptr(), keep[1].data_ptr(),
              keep[2].data_ptr(), keep[3].data_ptr(), ids.size, bounds.data_ptr(), 3, geo.max_block, geo.cap,
              scores_d.data_ptr(), 2, model.E, send.data_ptr(), pos_reply.data_ptr(), None)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(pos_reply.cpu().numpy(), want_pos.numpy())
    got, want = send.cpu().view(torch.int16).numpy(), want_send.view(torch.int16).numpy()
    for g in range(3):
        n = int(b["offsets"][geo.bounds[g + 1]] - b["offsets"][geo.bounds[g]])
        hdr_words = 2 * (geo.max_block + 2 * geo.num_expert)
        np.testing.assert_array_equal(got[g * geo.seg_rows, :hdr_words], want[g * geo.seg_rows, :hdr_words])
        np.testing.assert_array_equal(got[g * geo.seg_rows + 1: g * geo.seg_rows + 1 + n],
                                      want[g * geo.seg_rows + 1: g * geo.seg_rows + 1 + n])
    # the owner side: three sources' messages for rank 1 (here: three copies of differently routed batches)
    recv = torch.zeros((geo.rows, geo.hidden), dtype=torch.bfloat16)
    for s in range(3):
        xs = om.bf16_round(rng.standard_normal((7, model.H)).astype(np.float32))
        ids_s, _ = model.canonical_routing(0, xs)
        bs = {}
        ob.permute(torch.from_numpy(ids_s.astype(np.int32)), bs)
        msg, _ = ob.pack(torch.from_numpy(xs).to(torch.bfloat16), bs, rng.standard_normal((2, model.E)).astype(np.float32), 2)
        recv[s * geo.seg_rows: (s + 1) * geo.seg_rows] = msg[1 * geo.seg_rows: 2 * geo.seg_rows]   # the part addressed to rank 1
    want_re, want_sums = ob.unpack(recv, 2)
    row_expert = torch.full((geo.rows,), 99, dtype=torch.int32, device="cuda")
    sums = torch.zeros((2, geo.num_expert), dtype=torch.float32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    recv_d = recv.cuda()
    _lib.call("pm_k_ep_unpack", recv_d.data_ptr(), geo.hidden, 3, ob.n_local, geo.max_block, geo.cap, 2, geo.num_expert,
              row_expert.data_ptr(), sums.data_ptr(), err.data_ptr(), None)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(row_expert.cpu().numpy(), want_re.numpy())
    np.testing.assert_array_equal(sums.cpu().numpy(), want_sums)
    assert int(err.item()) == 0
    # a header whose counts exceed the capacity voids its segment and raises the flag
    bad = recv.clone()
    bad.view(torch.int16).numpy().view(np.int32)[0, 0] = 1000
    bad_d = bad.cuda()
    _lib.call("pm_k_ep_unpack", bad_d.data_ptr(), geo.hidden, 3, ob.n_local, geo.max_block, geo.cap, 2, geo.num_expert,
              row_expert.data_ptr(), sums.data_ptr(), err.data_ptr(), None)
    torch.cuda.synchronize()
    assert int(err.item()) == 1 and (row_expert.cpu().numpy()[: geo.seg_rows] == -1).all()


@pytest.mark.parametrize("with_pred,pool", [(False, False), (True, False), (True, True)])
def test_layer_with_world_size_one(lib, with_pred, pool):
    """The whole expert-parallel layer on one rank: pack, (copy), unpack, padded routed rows with the
    device-planned launch, shared expert on the side stream, combine; outputs and cache log against
    the oracles. With the pooled miss fetch on, the demand copies travel through the shared-memory
    arena, the staging buffer, the (degenerate) exchange and the scatter kernel instead."""
    import os
    from tests.ep_common import build_rank, oracle_replay
    model, preds, ep, be, cache = build_rank(0, 1, with_pred, pool_tag=f"t{os.getpid()}" if pool else None)
    rng = np.random.default_rng(9)
    xs = []
    for step in range(5):
        x = om.bf16_round(rng.standard_normal((6, model.H)).astype(np.float32))
        xs.append(x)
        for l in range(model.L):
            y = ep.forward(l, dev_bf16(x))
            torch.cuda.synchronize()
            ref, _, _ = model.oracle_forward(l, x)
            got = y.float().cpu().numpy()
            np.testing.assert_allclose(got, ref, rtol=2e-2, atol=2e-2 * np.abs(ref).max() * 0.25)
            assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 5e-3
    oc = oracle_replay(model, preds, [xs], 0, 1)
    assert cache.events() == oc.events
    assert int(be.unpack_err.item()) == 0
    if with_pred:
        assert cache.stats()["prefetch_miss"] > 0
    if pool:
        assert be.pool["exchanges"] > 0 and int(cache.get("pool_bytes_pulled")) > 0
        st = cache.stats()
        # every miss moved one whole record, whichever route its bytes took
        assert st["h2d_bytes"] == (st["precise_miss"] + st["prefetch_miss"]) * int(cache.get("record_bytes"))
    cache.close()


def test_two_rank_nccl_exchange(lib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = Path(__file__).with_name("ep_gpu_check.py")
    for extra in ([], ["--pool"]):
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                            "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), *extra],
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
        assert r.stdout.count(" OK") == 2
