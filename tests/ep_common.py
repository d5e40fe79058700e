"""Shared by the expert-parallel GPU checks: one rank's cache, backend and layer over a small
model, and the single-process replay its cache log is compared with."""
import numpy as np
import torch

from oracle import moe_math as om
from oracle import srs_policy as sp
from promoe_b200.engine import ExpertCache
from promoe_b200.ep import CudaBackend, ExpertParallelMoE, Geometry
from tests.helpers import TinyModel, dev, dev_bf16

N_PREDICT = 2


def make_preds(model, seed=3, D=32):
    rng = np.random.default_rng(seed)
    preds = {}
    for src in range(model.L - 1):                  # index l predicts layer l + 1
        w1 = om.bf16_round((rng.standard_normal((D, model.H)) * 0.1).astype(np.float32))
        w2 = om.bf16_round((rng.standard_normal((model.E, D)) * 0.3).astype(np.float32))
        b2 = (rng.standard_normal(model.E) * 0.1).astype(np.float32)
        preds[(src, src + 1)] = (w1, None, w2, b2)
    return preds


def build_rank(rank, world, with_pred, tokens=6, seed=11, pool_tag=None):
    """pool_tag: a string shared by all ranks of the run switches the pooled miss fetch on."""
    model = TinyModel(seed=seed, L=3, E=16, H=256, I=128, k=4, shared_I=256, shared_gate=True)
    preds = make_preds(model) if with_pred else {}
    geo = Geometry(model.E, world, max_tokens_per_rank=tokens, top_k=model.k, hidden=model.H, n_pred=1 if with_pred else 0)
    e0, n_local = geo.bounds[rank], geo.bounds[rank + 1] - geo.bounds[rank]
    cache = ExpertCache(model.L, n_local, num_expert_per_token=model.k, cache_rate=0.5,
                        num_predict_expert_per_layer=N_PREDICT if with_pred else 0)
    cache.set_param_list(["gate_proj.weight", "up_proj.weight", "down_proj.weight"])
    for l in range(model.L):
        for e in range(n_local):
            cache.register_expert(l, e, [om.to_bf16_bits(w) for w in model.experts[l][e0 + e]])
    if pool_tag is not None:
        cache.set("shared_arena", f"/pm_{pool_tag}_{rank}")
    cache.pin_all()
    cache.build_slab()
    cache.enable_event_log(True)
    layers = []
    for l in range(model.L):
        cache.set_layer_weights(l, None, model.I, 1, False, hidden=model.H)
        layers.append(dict(gate_w=dev_bf16(model.gate_w[l]), gate_bias=dev(model.gate_bias[l]),
                           shared=[dev_bf16(w) for w in model.shared[l]], shared_gate_w=dev_bf16(model.shared_gate_w[l]),
                           top_k=model.k, norm_topk=model.norm_topk, routed_scale=1.0, inter=model.I))
    dev_preds = {key: (dev_bf16(w1), None, dev_bf16(w2), torch.from_numpy(b2).cuda()) for key, (w1, _, w2, b2) in preds.items()}
    pmap = [(l + 1, l + 2) if l + 1 < model.L else (model.L, model.L) for l in range(model.L)]
    be = CudaBackend(cache, layers, torch.device("cuda"), geo, rank, predictors=dev_preds, predict_map=pmap,
                     global_tokens=tokens * world, n_predict=N_PREDICT if with_pred else 0)
    if pool_tag is not None:
        be.enable_pool([f"/pm_{pool_tag}_{r}" for r in range(world)],
                       [geo.bounds[r + 1] - geo.bounds[r] for r in range(world)], f"/pm_{pool_tag}_mail")
    return model, preds, ExpertParallelMoE(geo, be), be, cache


def oracle_replay(model, preds, xs_by_rank, rank, world):
    """What this rank's cache must have decided: per layer call, the prefetch of those of the globally
    best-ranked experts (predictor scores summed over every rank's tokens) that this rank holds, then
    the ascending unique ids that arrived."""
    geo_bounds = [r * model.E // world for r in range(world + 1)]
    e0, n_local = geo_bounds[rank], geo_bounds[rank + 1] - geo_bounds[rank]
    oc = sp.SequentialCache(model.L, n_local, model.k, cache_rate=0.5, num_predict=N_PREDICT if preds else 0)
    for step in range(len(xs_by_rank[0])):
        for l in range(model.L):
            for (s, d), (w1, b1, w2, b2) in sorted(preds.items()):
                if s == l:
                    # each rank adds its bias-free partial sums; the output bias enters once per token
                    total = sum(om.predictor_scores(xs_by_rank[r][step], w1, b1, w2, b2) for r in range(world))
                    mine = [int(e) - e0 for e in om.rank_experts(total, N_PREDICT) if e0 <= e < e0 + n_local][: oc.num_predict]
                    if mine:
                        oc.prefetch_layer(d, mine)
            act = set()
            for r in range(world):
                ids, _ = model.canonical_routing(l, xs_by_rank[r][step])
                act |= set(int(v) for v in ids.reshape(-1))
            local = sorted(e - e0 for e in act if e0 <= e < e0 + n_local)
            if local:
                oc.report_layer(l, local)
    return oc
