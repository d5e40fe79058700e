"""Two (or more) GPU check of the expert-parallel layer, launched with torchrun:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        --master-port 29511 tests/ep_gpu_check.py

Every rank routes its own tokens, the experts are sharded in blocks, and the outputs must equal
the single-process oracle on that rank's tokens; every rank's cache log must equal a single cache
over its block fed with the ids that arrived and with the prefetches its summed predictor scores
rank. NVLS is switched off for the run (a rank that exits early must not leave multicast bindings
behind). Prints one line per rank and exits non-zero on a mismatch."""
import os
import sys
from pathlib import Path

os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import numpy as np
import torch
import torch.distributed as dist

from oracle import moe_math as om
from oracle import srs_policy as sp
from tests.ep_common import build_rank, oracle_replay


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    pool_tag = f"c{os.environ.get('MASTER_PORT', '0')}" if "--pool" in sys.argv else None   # pooled miss fetch
    model, preds, ep, be, cache = build_rank(rank, world, with_pred=True, pool_tag=pool_tag)
    rng = np.random.default_rng(50 + rank)
    worst, xs = 0.0, []
    for step in range(5):
        x = om.bf16_round(rng.standard_normal((6, model.H)).astype(np.float32))
        xs.append(x)
        for l in range(model.L):
            y = ep.forward(l, torch.from_numpy(x).to(torch.bfloat16).cuda())
            torch.cuda.synchronize()
            ref, _, _ = model.oracle_forward(l, x)
            got = y.float().cpu().numpy()
            worst = max(worst, float(np.linalg.norm(got - ref) / np.linalg.norm(ref)))
    gathered = [None] * world
    dist.all_gather_object(gathered, xs)
    oc = oracle_replay(model, preds, gathered, rank, world)
    ok_log = cache.events() == oc.events
    ok = worst < 5e-3 and ok_log and int(be.unpack_err.item()) == 0
    pooled = f" pool exchanges {be.pool['exchanges']} pulled {cache.get('pool_bytes_pulled')} B" if be.pool else ""
    print(f"rank {rank}/{world}: rel_err {worst:.2e} cache_log_equal {ok_log} events {len(oc.events)} "
          f"dispatched {ep.bytes_dispatched} B{pooled} {'OK' if ok else 'MISMATCH'}", flush=True)
    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    cache.close()
    dist.destroy_process_group()
    sys.exit(1 if int(flag.item()) else 0)


if __name__ == "__main__":
    main()
