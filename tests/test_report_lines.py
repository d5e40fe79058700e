"""The per-forward counter series and the end-of-run `key:value` report of the reference's profiler
(src/cpp_worker/profiler.hpp:262-319, src/cpp_worker/prefetcher.cpp:327-402), over a policy-only
context (no GPU): per-iteration hits and misses must equal what the oracle's event log gives for
the same request stream, and the report must average exactly the iterations the reference keeps."""
import numpy as np

from oracle import srs_policy as sp
from promoe_b200 import cpp_worker as cw
from promoe_b200.engine import ExpertCache


def drive(L=3, E=8, k=2, iters=16, seed=3):
    cache = ExpertCache(L, E, num_expert_per_token=k, cache_rate=0.5, num_predict_expert_per_layer=2)
    cache.build_policy_only()
    oc = sp.SequentialCache(L, E, k, cache_rate=0.5, num_predict=2)
    rng = np.random.default_rng(seed)
    prof, stats = cw.TimeProfiler(cache), cw.CacheStatistics(cache)
    per_iter = []                       # oracle: [hit, miss, prefetch_hit, prefetch_miss, activated]
    # four warm-up requests (prompt + one decode step each), then two real requests
    seq_lens = [7, 1, 7, 1, 7, 1, 7, 1, 7, 1, 1, 1, 9, 1, 1, 1][:iters]
    for it in range(iters):
        n0 = len(oc.events)
        activated = 0
        prof.push("seq_len", seq_lens[it])
        prof.push(cw.TimeType.kModelForward, 1000 * (it + 1))
        for l in range(L):
            n_ids = k if seq_lens[it] == 1 else 5
            ids = sorted(int(v) for v in rng.choice(E, size=n_ids, replace=False))
            if l + 1 < L:
                guess = [int(v) for v in rng.choice(E, size=2, replace=False)]
                cache.prefetch_layer(l + 1, guess)
                oc.prefetch_layer(l + 1, guess)
            stats.forward()
            cache.report_layer(l, ids)
            oc.report_layer(l, ids)
            for e in ids:          # the oracle's report_layer already includes the per-expert hooks
                cache.report_expert(l, e)
                cache.expert_done(l, e)
            cache.layer_done(l)
            activated += len(ids)
        kinds = [e[0] for e in oc.events[n0:]]
        per_iter.append([kinds.count(sp.PRECISE_HIT), kinds.count(sp.PRECISE_MISS), kinds.count(sp.PREFETCH_HIT),
                         kinds.count(sp.PREFETCH_MISS), activated])
    return cache, prof, stats, np.array(per_iter), np.array(seq_lens)


def test_series_match_the_oracle_per_iteration():
    cache, prof, stats, per_iter, _ = drive()
    for col, kind in enumerate(("hit", "miss", "prefetch_hit", "prefetch_miss", "activated")):
        assert prof.to_tensor(kind).tolist() == per_iter[:, col].tolist(), kind
    # ready / unready: one count per demanded expert, and the per-layer rows add up to them
    assert (prof.to_tensor("ready") + prof.to_tensor("unready")).tolist() == per_iter[:, 4].tolist()
    rows = stats.to_tensor()
    assert rows.shape == (16 * 3, 2) and rows.sum().item() == per_iter[:, 4].sum()
    cache.close()


def test_report_lines_average_the_iterations_the_reference_keeps():
    cache, prof, _, per_iter, seq = drive()
    lines = dict(ln.split(":") for ln in prof.report_lines())
    # the first four prompts are warm-up: everything before the fifth prefill iteration (index 8) is dropped
    keep = np.arange(len(seq)) >= 8
    dec, pre = keep & (seq <= 1), keep & (seq > 1)
    assert int(lines["num_prefill_iter"]) == pre.sum() == 2 and int(lines["num_decode_iter"]) == dec.sum() == 6
    hit, miss = per_iter[dec, 0].mean(), per_iter[dec, 1].mean()
    assert abs(float(lines["decode_stage_hit_cnt"]) - hit) < 1e-4
    assert abs(float(lines["decode_stage_miss_cnt"]) - miss) < 1e-4
    assert abs(float(lines["decode_stage_hit_rate"]) - hit / (hit + miss)) < 1e-4
    ph, pm = per_iter[pre, 2].mean(), per_iter[pre, 3].mean()
    assert abs(float(lines["prefill_stage_prefetch_hit_cnt"]) - ph) < 1e-4
    assert abs(float(lines["prefill_stage_prefetch_miss_cnt"]) - pm) < 1e-4
    fwd = 1000.0 * (np.arange(len(seq)) + 1)
    assert abs(float(lines["decode_stage_forward_time"]) - fwd[dec].mean() / 1000.0) < 1e-3
    assert float(lines["decode_stage_wait_time"]) == 0.0
    # every key the reference's sweep parser reads is present
    for key in ("decode_stage_ready_rate", "prefill_stage_ready_rate", "decode_stage_prefetch_hit_rate",
                "prefill_stage_hit_rate", "prefill_stage_forward_time", "predict_time"):
        assert key in lines
    cache.close()


def test_report_with_too_few_prompts_keeps_nothing():
    cache, prof, _, _, _ = drive(iters=6)
    lines = dict(ln.split(":") for ln in prof.report_lines())
    assert lines["num_prefill_iter"] == "0" and lines["num_decode_iter"] == "0"
    cache.close()
