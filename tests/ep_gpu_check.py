"""Two (or more) GPU check of the expert-parallel layer, launched with torchrun:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        --master-port 29511 tests/ep_gpu_check.py

Every rank routes its own tokens, the experts are sharded in blocks, and the outputs must equal
the single-process oracle on that rank's tokens; every rank's cache log must equal a single cache
over its block fed with the ids that arrived. NVLS is switched off for the run (a rank that exits
early must not leave multicast bindings behind). Prints one line per rank and exits non-zero on
a mismatch."""
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
from promoe_b200.engine import ExpertCache
from promoe_b200.ep import CudaBackend, ExpertParallelMoE, expert_bounds
from tests.helpers import TinyModel, dev, dev_bf16


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    model = TinyModel(seed=11, L=3, E=16, H=256, I=128, k=4, shared_I=256, shared_gate=True)
    b = expert_bounds(model.E, world)
    e0, n_local = b[rank], b[rank + 1] - b[rank]
    cache = ExpertCache(model.L, n_local, num_expert_per_token=model.k, cache_rate=0.5, num_predict_expert_per_layer=0)
    cache.set_param_list(["gate_proj.weight", "up_proj.weight", "down_proj.weight"])
    for l in range(model.L):
        for e in range(n_local):
            cache.register_expert(l, e, [om.to_bf16_bits(w) for w in model.experts[l][e0 + e]])
    cache.pin_all()
    cache.build_slab()
    cache.enable_event_log(True)
    layers = []
    for l in range(model.L):
        cache.set_layer_weights(l, None, model.I, 1, False, hidden=model.H)
        layers.append(dict(gate_w=dev_bf16(model.gate_w[l]), gate_bias=dev(model.gate_bias[l]),
                           shared=[dev_bf16(w) for w in model.shared[l]], shared_gate_w=dev_bf16(model.shared_gate_w[l]),
                           top_k=model.k, norm_topk=model.norm_topk, routed_scale=1.0, inter=model.I))
    ep = ExpertParallelMoE(model.E, CudaBackend(cache, layers, torch.device("cuda")))
    rng = np.random.default_rng(50 + rank)
    worst = 0.0
    arrived = []   # (layer, sorted unique local ids) in call order, rebuilt from all ranks' routing
    for step in range(5):
        x = om.bf16_round(rng.standard_normal((6 + rank, model.H)).astype(np.float32))
        for l in range(model.L):
            y = ep.forward(l, dev_bf16(x))
            torch.cuda.synchronize()
            ref, ids, _ = model.oracle_forward(l, x)
            got = y.float().cpu().numpy()
            worst = max(worst, float(np.linalg.norm(got - ref) / np.linalg.norm(ref)))
            mine = torch.zeros(model.E, dtype=torch.int32, device="cuda")
            mine[torch.from_numpy(np.unique(ids)).cuda()] = 1
            dist.all_reduce(mine)   # which experts anyone activated in this layer call
            act = np.nonzero(mine.cpu().numpy())[0]
            arrived.append((l, [int(e - e0) for e in act if e0 <= e < e0 + n_local]))
    oc = sp.SequentialCache(model.L, n_local, model.k, cache_rate=0.5, num_predict=0)
    for l, ids in arrived:
        if ids:
            oc.report_layer(l, ids)
    ok_log = cache.events() == oc.events
    ok = worst < 5e-3 and ok_log
    print(f"rank {rank}/{world}: rel_err {worst:.2e} cache_log_equal {ok_log} events {len(oc.events)} "
          f"dispatched {ep.bytes_dispatched} B {'OK' if ok else 'MISMATCH'}", flush=True)
    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    cache.close()
    dist.destroy_process_group()
    sys.exit(1 if int(flag.item()) else 0)


if __name__ == "__main__":
    main()
