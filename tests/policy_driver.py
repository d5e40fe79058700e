"""Drives the same request stream through the product's cache engine (C ABI, no GPU needed)
and through the oracle, and returns both event logs."""
from __future__ import annotations

import ctypes as C

import numpy as np

from oracle import srs_policy as sp
from promoe_b200 import _lib


def make_stream(seed, num_layer, num_expert, top_k, steps, batch=1, zipf=1.1, prefill_first=False,
                n_predict=0):
    """A synthetic request stream: per step and layer, the ascending unique expert ids that a
    batch of tokens activates (skewed popularity, temporal reuse), optionally preceded by a
    prefetch request (noisy guess of the same ids)."""
    rng = np.random.default_rng(seed)
    pop = 1.0 / np.arange(1, num_expert + 1) ** zipf
    perms = [rng.permutation(num_expert) for _ in range(num_layer)]
    prev = [[None] * batch for _ in range(num_layer)]
    stream = []
    for t in range(steps):
        for l in range(num_layer):
            ids = set()
            if prefill_first and t == 0:
                ids = set(rng.choice(num_expert, size=min(num_expert, top_k * 12), replace=False).tolist())
            else:
                for b in range(batch):
                    if prev[l][b] is not None and rng.random() < 0.6:
                        keep = rng.choice(prev[l][b], size=max(1, top_k // 2), replace=False).tolist()
                    else:
                        keep = []
                    p = pop[np.argsort(perms[l])]
                    p = p / p.sum()
                    pick = set(keep)
                    while len(pick) < top_k:
                        pick.add(int(rng.choice(num_expert, p=p)))
                    prev[l][b] = sorted(pick)
                    ids |= pick
            ids = sorted(ids)
            if n_predict > 0 and not (prefill_first and t == 0):
                guess = list(rng.permutation(ids)[: max(1, n_predict - 1)])
                while len(guess) < n_predict:
                    c = int(rng.integers(num_expert))
                    if c not in guess:
                        guess.append(c)
                stream.append(("prefetch", l, [int(g) for g in guess[:n_predict]]))
            stream.append(("layer", l, ids))
    return stream


def run_oracle(stream, traces=None, **kw):
    cache = sp.SequentialCache(**kw)
    for (seq, layer, expert), times in (traces or {}).items():
        cache.add_use_times(seq, layer, expert, times)
    out_orders = []
    for kind, layer, ids in stream:
        if kind == "prefetch":
            cache.prefetch_layer(layer, ids[: cache.num_predict])
        elif kind == "priority":
            cache.update_priority(ids, layer)
        elif kind == "seq":
            cache.set_cur_seq(layer)
        else:
            out_orders.append(cache.report_layer(layer, ids))
    return cache.events, out_orders, cache


def config_text(**kw) -> bytes:
    return "\n".join(f"{k}={v}" for k, v in kw.items()).encode()


def run_product(stream, num_layer, num_expert, num_expert_per_token, cache_rate=0.5, cache_policy="lru",
                num_predict=None, reorder_experts=None, early_preempt=None, chunk_prefetch=None,
                per_layer_cache=True, promote_hit_in_prefetch=True, num_per_expert_param=3, traces=None):
    lib = _lib.load()
    cfg = dict(num_expert_per_token=num_expert_per_token, cache_rate=repr(float(cache_rate)),
               cache_policy=cache_policy, num_predict_expert_per_layer=num_predict,
               reorder_experts=reorder_experts, early_preempt=early_preempt, chunk_prefetch=chunk_prefetch,
               per_layer_cache=per_layer_cache, promote_hit_in_prefetch=promote_hit_in_prefetch)
    ctx = C.c_void_p()
    _lib.call("pm_ctx_create", C.byref(ctx), num_layer, num_expert, config_text(**cfg))
    try:
        names = "\n".join(f"p{i}" for i in range(num_per_expert_param)).encode()
        _lib.call("pm_ctx_set_param_list", ctx, names)
        _lib.call("pm_build_policy_only", ctx)
        _lib.call("pm_event_log_enable", ctx, 1)
        buf = C.create_string_buffer(64)
        _lib.call("pm_ctx_get", ctx, b"num_predict_expert_per_layer", buf, 64)
        n_pred = int(buf.value)
        _lib.call("pm_ctx_get", ctx, b"early_preempt", buf, 64)
        early = buf.value == b"true"
        if traces:
            for (seq, layer, expert), times in traces.items():
                arr = (C.c_int64 * len(times))(*times)
                _lib.call("pm_oracle_add_use_times", ctx, seq, layer, expert, arr, len(times))
        out_orders = []
        for kind, layer, ids in stream:
            if kind == "prefetch":
                ids = ids[:n_pred]
                arr = (C.c_int64 * len(ids))(*ids)
                _lib.call("pm_prefetch_layer", ctx, layer, arr, len(ids))
            elif kind == "priority":
                p = np.ascontiguousarray(ids, np.float32)
                _lib.call("pm_update_priority", ctx, p.ctypes.data_as(C.POINTER(C.c_float)), p.shape[0], layer)
            elif kind == "seq":
                _lib.call("pm_set_cur_seq", ctx, layer)
            else:
                arr = (C.c_int64 * len(ids))(*ids)
                _lib.call("pm_report_layer", ctx, layer, arr, len(ids))
                order = list(arr)
                if not early:
                    for i in order:
                        _lib.call("pm_report_expert", ctx, layer, i)
                for i in order:
                    _lib.call("pm_expert_done", ctx, layer, i)
                _lib.call("pm_layer_done", ctx, layer)
                out_orders.append(order)
        n = C.c_size_t()
        _lib.call("pm_event_log_read", ctx, None, 0, C.byref(n))
        evs = (_lib.pm_event * max(1, n.value))()
        _lib.call("pm_event_log_read", ctx, evs, n.value, C.byref(n))
        events = [(e.kind, e.layer, e.expert, e.slot, e.evicted, e.evicted_layer) for e in evs[: n.value]]
        stats = _lib.pm_stats()
        _lib.call("pm_stats_read", ctx, C.byref(stats))
        _lib.call("pm_iter_marks_read", ctx, None, 0, C.byref(n))
        marks = (_lib.pm_stats * max(1, n.value))()
        _lib.call("pm_iter_marks_read", ctx, marks, n.value, C.byref(n))
        series = {name: [] for name in ("activated", "hit", "miss", "prefetch_hit", "prefetch_miss")}
        prev = dict.fromkeys(series, 0)
        for m in marks[: n.value]:   # per-forward values = differences of the end-of-iteration snapshots
            now = {"activated": m.activated_experts, "hit": m.precise_hit, "miss": m.precise_miss,
                   "prefetch_hit": m.prefetch_hit, "prefetch_miss": m.prefetch_miss}
            for k in series:
                series[k].append(now[k] - prev[k])
            prev = now
        stats.series = series
        return events, out_orders, stats
    finally:
        _lib.call("pm_ctx_destroy", ctx)
