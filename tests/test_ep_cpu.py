"""Expert parallelism, host logic: two gloo ranks on the CPU run ExpertParallelMoE with a test
backend that does the arithmetic with the numpy oracle. Checked: every rank's output equals the
single-process oracle on its tokens, and every rank's cache log equals a single cache over its
block of experts fed with the ids that arrived (ascending, unique)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_math as om
from oracle import srs_policy as sp
from promoe_b200.ep import ExpertParallelMoE, expert_bounds, split_counts
from tests.helpers import TinyModel


class OracleBackend:
    """Stand-in for CudaBackend: same methods, numpy arithmetic, a python cache per rank."""

    def __init__(self, model, rank, world, cache_rate):
        self.model, self.layers = model, [{"shared": model.shared} for _ in range(model.L)]
        b = expert_bounds(model.E, world)
        self.e0, self.n_local = b[rank], b[rank + 1] - b[rank]
        self.cache = sp.SequentialCache(model.L, self.n_local, model.k, cache_rate=cache_rate, num_predict=0)
        self.reported = []

    def route(self, layer, x):
        ids, w = self.model.canonical_routing(layer, x.float().numpy())
        return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(w.astype(np.float32)), None

    def permute(self, ids, num_expert):
        c, o, rt, pos = om.permute(ids.numpy(), num_expert)
        return torch.from_numpy(c), torch.from_numpy(o), torch.from_numpy(rt), torch.from_numpy(pos)

    def gather_rows(self, src, index):
        return src[index.long()].contiguous()

    def expert_rows(self, layer, x_rows, row_expert):
        ids = sorted(set(row_expert.tolist()))
        self.reported.append((layer, ids))
        self.cache.report_layer(layer, ids)
        out = np.zeros((x_rows.shape[0], x_rows.shape[1]), np.float32)
        xr = x_rows.float().numpy()
        for e in ids:
            sel = (row_expert == e).numpy()
            out[sel] = om.swiglu_mlp(xr[sel], *self.model.experts[layer][self.e0 + e], round_h_bf16=True)
        return torch.from_numpy(out)

    def shared_rows(self, layer, x, yexp, first_row):
        s = self.model.shared[layer]
        yexp[first_row:] = torch.from_numpy(om.swiglu_mlp(x.float().numpy(), *s, round_h_bf16=True).astype(np.float32))

    def combine(self, yexp, pos, w, T, H, n_routed_rows, n_shared, shared_scale):
        y = (yexp[pos.long().view(T, -1)] * w[:, :, None]).sum(1)
        if n_shared:
            y = y + yexp[n_routed_rows:]
        return y


def worker(rank, world, port, seed, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    model = TinyModel(seed=seed, L=2, E=8, H=64, I=32, k=2, shared_I=64)
    be = OracleBackend(model, rank, world, cache_rate=0.5)
    ep = ExpertParallelMoE(model.E, be)
    rng = np.random.default_rng(100 + rank)
    errs = []
    for step in range(4):
        x = om.bf16_round(rng.standard_normal((3 + rank, model.H)).astype(np.float32))
        for l in range(model.L):
            y = ep.forward(l, torch.from_numpy(x))
            ref, _, _ = model.oracle_forward(l, x)
            errs.append(float(np.abs(y.numpy() - ref).max() / np.abs(ref).max()))
    oc = sp.SequentialCache(model.L, be.n_local, model.k, cache_rate=0.5, num_predict=0)
    for l, ids in be.reported:
        oc.report_layer(l, ids)
    out_q.put((rank, max(errs), be.cache.events == oc.events, len(be.cache.events), ep.bytes_dispatched))
    dist.destroy_process_group()


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 3])
def test_two_rank_exchange_matches_single_process_oracle(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, 7, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    for rank, err, log_ok, n_events, sent in results:
        assert err < 1e-5, f"rank {rank}: output differs from the oracle ({err})"
        assert log_ok and n_events > 0
        assert sent > 0


def test_bounds_and_splits():
    assert expert_bounds(64, 8) == [0, 8, 16, 24, 32, 40, 48, 56, 64]
    assert expert_bounds(60, 8) == [0, 7, 15, 22, 30, 37, 45, 52, 60]   # uneven blocks of 7 or 8
    counts = torch.tensor([1, 0, 2, 3, 0, 0, 4, 1])
    assert split_counts(counts, expert_bounds(8, 2)) == [6, 5]
    assert split_counts(counts, expert_bounds(8, 1)) == [11]
