"""The product's cache engine (through the C ABI, host only) against the policy oracle:
event logs (kind, layer, expert, slot, evicted), reordered id lists and counters must be
identical on the same request stream."""
import numpy as np
import pytest

from oracle import srs_policy as sp
from tests.policy_driver import make_stream, run_oracle, run_product

CASES = [
    # L, E, k, rate, policy, n_predict, batch, per_layer
    (1, 64, 6, 0.375, "lru", 0, 32, True),     # C1: more unique experts than lines per call
    (24, 60, 4, 0.375, "lru", 0, 8, True),     # C2 shape, no prefetch
    (24, 60, 4, 0.375, "lru", 4, 8, True),     # C2 shape with prefetch, reorder, early preempt
    (8, 8, 2, 0.5, "lru", 2, 16, True),        # C3 shape (Mixtral)
    (4, 64, 8, 0.375, "fifo", 0, 4, True),
    (4, 64, 8, 0.375, "fifo", 8, 4, True),
    (6, 16, 2, 0.4, "static-1", 0, 2, True),
    (6, 16, 2, 0.4, "static-2", 2, 2, True),
    (5, 32, 4, 0.3, "lru", 4, 2, False),       # one pool shared by all layers
    (5, 32, 4, 0.3, "lru", 0, 2, False),
    (27, 64, 6, 1.0 / 64, "lru", 0, 1, True),  # one line per layer
    (3, 8, 2, 1.0, "lru", 2, 4, True),         # everything fits
]


@pytest.mark.parametrize("L,E,k,rate,policy,n_pred,batch,per_layer", CASES)
def test_event_log_matches_oracle(lib, L, E, k, rate, policy, n_pred, batch, per_layer):
    stream = make_stream(11 + L + E, L, E, k, steps=12, batch=batch, prefill_first=True, n_predict=n_pred)
    kw = dict(num_layer=L, num_expert=E, num_expert_per_token=k, cache_rate=rate, cache_policy=policy,
              num_predict=n_pred, per_layer_cache=per_layer)
    ev_o, ord_o, cache = run_oracle(stream, **kw)
    ev_p, ord_p, stats = run_product(stream, **kw)
    assert len(ev_p) == len(ev_o) > 0
    assert ev_p == ev_o
    assert ord_p == ord_o
    assert (stats.precise_hit, stats.precise_miss, stats.prefetch_hit, stats.prefetch_miss) == (
        cache.counters["hit"], cache.counters["miss"], cache.counters["prefetch_hit"],
        cache.counters["prefetch_miss"])


@pytest.mark.parametrize("reorder,early,chunk,promote", [(True, False, False, True), (False, True, True, False),
                                                        (False, False, True, True), (True, True, False, False)])
def test_flag_combinations(lib, reorder, early, chunk, promote):
    L, E, k = 6, 32, 4
    stream = make_stream(5, L, E, k, steps=10, batch=3, n_predict=4)
    kw = dict(num_layer=L, num_expert=E, num_expert_per_token=k, cache_rate=0.375, num_predict=4,
              reorder_experts=reorder, early_preempt=early, chunk_prefetch=chunk,
              promote_hit_in_prefetch=promote)
    ev_o, ord_o, _ = run_oracle(stream, **kw)
    ev_p, ord_p, _ = run_product(stream, **kw)
    assert ev_p == ev_o and ord_p == ord_o


def test_nn_policy_with_priority_updates(lib):
    L, E, k = 6, 32, 4
    rng = np.random.default_rng(3)
    base = make_stream(9, L, E, k, steps=10, batch=2, n_predict=4)
    stream = []
    for item in base:
        if item[0] == "prefetch":
            # the predictor's scores for that layer arrive just before its prefetch (worker.cpp:19-21)
            stream.append(("priority", item[1], rng.random((1, E)).astype(np.float32) * 50))
        stream.append(item)
    stream.insert(0, ("priority", 0, rng.random((L, E)).astype(np.float32)))
    kw = dict(num_layer=L, num_expert=E, num_expert_per_token=k, cache_rate=0.375, cache_policy="nn",
              num_predict=4)
    ev_o, ord_o, _ = run_oracle(stream, **kw)
    ev_p, ord_p, _ = run_product(stream, **kw)
    assert ev_p == ev_o and ord_p == ord_o
    assert any(e[4] >= 0 for e in ev_p), "the stream must force evictions"


def test_min_policy_follows_trace(lib):
    """Belady: the trace is the stream itself, so every precise access matches the recorded time."""
    L, E, k = 4, 16, 2
    traces, stream = {}, []
    for seq in range(3):
        s = make_stream(100 + seq, L, E, k, steps=8, batch=1)
        use = {}
        time = 0
        for kind, layer, ids in s:
            for i in ids:
                use.setdefault((seq, layer, i), []).append(time)
            time += 1
        for l in range(L):
            for e in range(E):
                traces[(seq, l, e)] = use.get((seq, l, e), []) + [sp.INT64_MAX]
        stream.append(("seq", seq, None))
        stream += s
    kw = dict(num_layer=L, num_expert=E, num_expert_per_token=k, cache_rate=0.375, cache_policy="min",
              num_predict=0)
    ev_o, ord_o, _ = run_oracle(stream, traces=traces, **kw)
    ev_p, ord_p, _ = run_product(stream, traces=traces, **kw)
    assert ev_p == ev_o and ord_p == ord_o
    # MIN never does worse than LRU on the same stream
    kw_lru = dict(kw, cache_policy="lru")
    ev_l, _, _ = run_oracle([s for s in stream if s[0] != "seq"], **kw_lru)
    assert sum(e[0] == sp.PRECISE_MISS for e in ev_o) <= sum(e[0] == sp.PRECISE_MISS for e in ev_l)


def test_line_plan_matches_oracle(lib):
    import ctypes as C
    from promoe_b200 import _lib
    from tests.policy_driver import config_text
    for L, E, rate in [(24, 60, 0.375), (27, 64, 0.375), (32, 8, 0.5), (28, 64, 0.375), (26, 64, 0.25),
                       (7, 10, 0.33), (2, 5, 0.5), (1, 64, 0.375), (13, 9, 0.41)]:
        ctx = C.c_void_p()
        _lib.call("pm_ctx_create", C.byref(ctx), L, E, config_text(num_expert_per_token=2, cache_rate=repr(rate)))
        lens = (C.c_int32 * L)()
        n = C.c_int()
        _lib.call("pm_plan_slots", ctx, lens, L, C.byref(n))
        _lib.call("pm_ctx_destroy", ctx)
        assert n.value == L
        assert list(lens) == sp.plan_lines(L, sp.total_lines(rate, L, E))
    # Qwen1.5-MoE shape: 540 lines over 24 layers, 12 layers get 23
    assert sorted(i for i, v in enumerate(sp.plan_lines(24, 540)) if v == 23) == [0, 1, 3, 4, 6, 7, 9, 10, 13, 16, 19, 22]


def test_config_errors_are_returned_not_fatal(lib):
    import ctypes as C
    from promoe_b200 import _lib
    ctx = C.c_void_p()
    for bad in (b"cache_rate=0.5", b"num_expert_per_token=2\nbogus_key=1",
                b"num_expert_per_token=2\ncache_policy=clock", b"num_expert_per_token=abc"):
        with pytest.raises(_lib.PromoeError):
            _lib.call("pm_ctx_create", C.byref(ctx), 2, 4, bad)
    # dialect aliases, "None" = default, '-' in keys (utils.cpp:147-172)
    _lib.call("pm_ctx_create", C.byref(ctx), 27, 64,
              b"num_expert_per_token=6\nmoe-cache-rate=0.25\nnum_predict=None\nmodel_arch_string=DeepSeek-x\ncross_token_pred=True")
    buf = C.create_string_buffer(64)
    for key, want in ((b"cache_rate", b"0.25"), (b"num_predict_expert_per_layer", b"6"), (b"reorder_experts", b"true"),
                      (b"limit_layer_0_window", b"3"), (b"max_prefetch_layer_distance", b"26"),
                      (b"cross_token_pred", b"true")):
        _lib.call("pm_ctx_get", ctx, key, buf, 64)
        assert buf.value == want, (key, buf.value)
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_report_layer", ctx, 0, (C.c_int64 * 1)(1), 1)  # cache not built yet
    _lib.call("pm_ctx_destroy", ctx)
