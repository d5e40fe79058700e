"""GPU parity of the fused MoE layer (pm_moe_forward: route, permute, cache bookkeeping, copies
into VMM-mapped lines, grouped SwiGLU FFN by slot, combine) against the oracles:
routing ids bit-exact, cache event log bit-exact, layer output within bf16 tolerance."""
import numpy as np
import pytest
import torch

from oracle import moe_math as om
from oracle import srs_policy as sp
from tests.helpers import TinyModel, dev_bf16

pytestmark = pytest.mark.gpu

RTOL = 2e-2  # bf16 layer outputs vs the float64 oracle on the same bf16 inputs


def check_output(y_dev, ref):
    got = y_dev.float().cpu().numpy()
    scale = np.abs(ref).max()
    np.testing.assert_allclose(got, ref, rtol=RTOL, atol=RTOL * scale * 0.25)
    # and tight in aggregate: relative Frobenius error well below one bf16 ulp
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 5e-3


def run_stack(model, cache, oracle_cache, batch, steps, prefetch_rng=None, n_predict=0):
    cache.enable_event_log(True)
    cache.set("keep_routing", 1)
    for x in model.hidden_stream(batch, steps):
        xd = dev_bf16(x)
        for l in range(model.L):
            if prefetch_rng is not None:
                guess = [int(v) for v in prefetch_rng.choice(model.E, size=n_predict, replace=False)]
                cache.prefetch_layer(l, guess)
                oracle_cache.prefetch_layer(l, guess)
            y = cache.forward(l, xd)
            torch.cuda.synchronize()
            ids, w = cache.last_routing(l, batch, model.k)
            ref_ids, ref_w = model.canonical_routing(l, x)
            assert np.array_equal(ids, ref_ids.astype(np.int32)), "routing must be bit-exact"
            np.testing.assert_allclose(w, ref_w, rtol=1e-4, atol=1e-7)
            orders = []
            ref_y, ids64, _ = model.oracle_forward(
                l, x, report_experts=lambda u: np.asarray(orders.append(oracle_cache.report_layer(l, u)) or orders[-1]))
            assert np.array_equal(ids64, ref_ids), "seed gives a routing gap below float32 resolution"
            check_output(y, ref_y)
    return cache.events()


CASES = [
    # name, model kwargs, config, batch, steps
    ("slots_lt_unique", dict(L=2, E=8, H=128, I=64, k=2, shared_I=128), dict(cache_rate=0.5, num_predict_expert_per_layer=0), 6, 6),
    ("qwen_like", dict(L=3, E=12, H=256, I=96, k=4, shared_I=192, shared_gate=True), dict(cache_rate=0.375, num_predict_expert_per_layer=0), 4, 5),
    ("deepseek_like", dict(L=2, E=16, H=128, I=64, k=6, shared_I=128, routed_scale=2.5), dict(cache_rate=0.375, num_predict_expert_per_layer=0), 5, 5),
    ("mixtral_like", dict(L=2, E=8, H=256, I=160, k=2, norm_topk=True, zipf_bias=False, gate_std=0.2), dict(cache_rate=0.5, num_predict_expert_per_layer=0), 16, 4),
    ("all_resident", dict(L=2, E=8, H=128, I=64, k=2), dict(cache_rate=1.0, num_predict_expert_per_layer=0), 3, 4),
    ("one_line", dict(L=2, E=8, H=128, I=64, k=2), dict(cache_rate=0.125, num_predict_expert_per_layer=0), 3, 4),
    ("global_pool", dict(L=3, E=8, H=128, I=64, k=2), dict(cache_rate=0.4, num_predict_expert_per_layer=0, per_layer_cache=False), 2, 5),
    ("fifo", dict(L=2, E=8, H=128, I=64, k=2), dict(cache_rate=0.5, num_predict_expert_per_layer=0, cache_policy="fifo"), 3, 5),
]


@pytest.mark.parametrize("name,mk,cfg,batch,steps", CASES, ids=[c[0] for c in CASES])
def test_stack_parity(lib, name, mk, cfg, batch, steps):
    model = TinyModel(seed=17, **mk)
    cache = model.make_cache(**cfg)
    oc = sp.SequentialCache(model.L, model.E, model.k, cache_rate=cfg["cache_rate"],
                            cache_policy=cfg.get("cache_policy", "lru"), num_predict=0,
                            per_layer_cache=cfg.get("per_layer_cache", True))
    events = run_stack(model, cache, oc, batch, steps)
    assert events == oc.events
    st = cache.stats()
    assert st["precise_miss"] > 0 and st["h2d_copies"] == st["precise_miss"] + st["prefetch_miss"]
    assert cache.get("slab_impl") == "vmm"
    cache.close()


def test_prefetch_requests_interleaved(lib):
    """Prefetches (wrong and right guesses) go through the copy stream while layers compute."""
    model = TinyModel(seed=5, L=3, E=12, H=128, I=64, k=3, shared_I=64)
    cfg = dict(cache_rate=0.5, num_predict_expert_per_layer=3)
    cache = model.make_cache(**cfg)
    oc = sp.SequentialCache(model.L, model.E, model.k, cache_rate=0.5, num_predict=3)
    events = run_stack(model, cache, oc, batch=4, steps=6, prefetch_rng=np.random.default_rng(1), n_predict=3)
    assert events == oc.events
    kinds = [e[0] for e in events]
    assert kinds.count(sp.PREFETCH_MISS) > 0 and kinds.count(sp.PREFETCH_HIT) > 0
    cache.close()


@pytest.mark.parametrize("device_topn", [True, False])
def test_predictor_inside_forward(lib, device_topn):
    """With predict_from_moe_input the forward runs the predictor MLP on its own input, ranks
    the scores (on the device: the host reads the best ids; or on the host from all scores) and
    prefetches the predicted layers before it reports its own."""
    model = TinyModel(seed=9, L=5, E=12, H=128, I=64, k=3)
    cfg = dict(cache_rate=0.5, num_predict_expert_per_layer=3, predict_from_moe_input=True)
    cache = model.make_cache(**cfg)
    cache.set("device_topn", "1" if device_topn else "0")
    rng = np.random.default_rng(2)
    D = 32
    mapping = []  # (src, dst) pairs of the default window: 0 -> [0,1), 1 -> [1,4), l>=2 -> l+2
    L = model.L
    stops = [0] * (L + 1)
    stop = 0
    for l in range(L):
        window = 1 if l == 0 else 3
        stops[l] = stop
        stops[l + 1] = min(l + window, L)
        stop = stops[l + 1]
    for l in range(1, L + 1):
        stops[l] = max(stops[l], stops[l - 1])
    preds = {}
    for src in range(L):
        for dst in range(stops[src], stops[src + 1]):
            w1 = om.bf16_round((rng.standard_normal((D, model.H)) * 0.1).astype(np.float32))
            w2 = om.bf16_round((rng.standard_normal((model.E, D)) * 0.3).astype(np.float32))
            b1 = (rng.standard_normal(D) * 0.1).astype(np.float32)
            b2 = (rng.standard_normal(model.E) * 0.1).astype(np.float32)
            preds[(src, dst)] = (w1, b1, w2, b2)
            cache.set_predictor(src, dst, dev_bf16(w1), torch.from_numpy(b1).cuda(), dev_bf16(w2),
                                torch.from_numpy(b2).cuda())
    assert sorted(preds) == [(0, 0), (1, 1), (1, 2), (1, 3), (2, 4)]
    oc = sp.SequentialCache(L, model.E, model.k, cache_rate=0.5, num_predict=3)
    cache.enable_event_log(True)
    for x in model.hidden_stream(4, 5):
        xd = dev_bf16(x)
        for l in range(L):
            for (src, dst), (w1, b1, w2, b2) in sorted(preds.items()):
                if src == l:
                    oc.prefetch_layer(dst, om.rank_experts(om.predictor_scores(x, w1, b1, w2, b2), oc.num_predict))
            y = cache.forward(l, xd)
            ref_y, _, _ = model.oracle_forward(l, x, report_experts=lambda u: np.asarray(oc.report_layer(l, u)))
            check_output(y, ref_y)
    assert cache.events() == oc.events
    assert cache.stats()["prefetch_miss"] > 0
    assert (int(cache.get("topn_launches")) > 0) == device_topn
    cache.close()


def test_deepseek_layer_shape_c1(lib):
    """Config C1 shape (DeepSeek-MoE-16B layer): 32 sequences activate more experts than the 24 lines."""
    model = TinyModel(seed=3, L=1, E=64, H=2048, I=1408, k=6, shared_I=2816)
    cache = model.make_cache(cache_rate=0.375, num_predict_expert_per_layer=0)
    assert cache.plan_slots() == [24]
    oc = sp.SequentialCache(1, 64, 6, cache_rate=0.375, num_predict=0)
    events = run_stack(model, cache, oc, batch=32, steps=3)
    assert events == oc.events
    cache.close()


def test_forward_host_round_trip_and_errors(lib):
    from promoe_b200 import _lib
    model = TinyModel(seed=4, L=1, E=8, H=128, I=64, k=2)
    cache = model.make_cache(cache_rate=0.5, num_predict_expert_per_layer=0)
    x = model.hidden_stream(5, 1)[0]
    xh = torch.from_numpy(x).to(torch.bfloat16).pin_memory()
    y = cache.forward_host(0, xh)
    ref, _, _ = model.oracle_forward(0, x)
    check_output(y.cuda(), ref)
    # empty batch is a no-op; bad layer and missing weights are errors, not aborts
    cache.forward(0, torch.empty((0, 128), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(_lib.PromoeError):
        cache.forward(3, dev_bf16(x))
    cache.close()
    from promoe_b200.engine import ExpertCache
    c2 = ExpertCache(1, 4, num_expert_per_token=2)
    with pytest.raises(_lib.PromoeError):
        c2.forward(0, dev_bf16(x))
    c2.close()


def test_report_hidden_hook_path(lib):
    """The hook route of the predictor (MoeLayerHook -> report_moe_layer_logits -> pm_report_hidden):
    hidden states entering index l are given to the library, which runs the MLPs of that index on
    the device, ranks on the host and prefetches; prefill-shaped input (seq > 1) is ignored."""
    model = TinyModel(seed=12, L=4, E=12, H=128, I=64, k=3)
    cache = model.make_cache(cache_rate=0.5, num_predict_expert_per_layer=3)
    rng = np.random.default_rng(6)
    D = 32
    preds = {}
    for src, dst in [(0, 0), (1, 1), (1, 2), (1, 3)]:  # default window for 4 layers
        w1 = om.bf16_round((rng.standard_normal((D, model.H)) * 0.1).astype(np.float32))
        w2 = om.bf16_round((rng.standard_normal((model.E, D)) * 0.3).astype(np.float32))
        preds[(src, dst)] = (w1, None, w2, None)
        cache.set_predictor(src, dst, dev_bf16(w1), None, dev_bf16(w2), None)
    oc = sp.SequentialCache(model.L, model.E, model.k, cache_rate=0.5, num_predict=3)
    cache.enable_event_log(True)
    for x in model.hidden_stream(3, 4):
        xd = dev_bf16(x)
        cache.report_hidden(0, torch.zeros((3, 5, model.H), dtype=torch.bfloat16, device="cuda"))  # prefill: ignored
        for l in range(model.L):
            cache.report_hidden(l, xd.view(3, 1, model.H))
            for (src, dst), (w1, b1, w2, b2) in sorted(preds.items()):
                if src == l:
                    oc.prefetch_layer(dst, om.rank_experts(om.predictor_scores(x, w1, b1, w2, b2), oc.num_predict))
            y = cache.forward(l, xd)
            ref_y, _, _ = model.oracle_forward(l, x, report_experts=lambda u: np.asarray(oc.report_layer(l, u)))
            check_output(y, ref_y)
    assert cache.events() == oc.events
    assert cache.stats()["prefetch_miss"] > 0
    cache.close()


def test_routed_rows_reject_an_expert_id_out_of_range(lib):
    """pm_moe_forward_routed takes the caller's expert id per row: an id equal to num_expert is an
    error, not a silently dropped row, and the context stays usable."""
    from promoe_b200 import _lib
    model = TinyModel(seed=8, L=1, E=8, H=128, I=64, k=2)
    cache = model.make_cache(cache_rate=0.5, num_predict_expert_per_layer=0)
    x = model.hidden_stream(4, 1)[0]
    xd = dev_bf16(x)
    out = torch.full((4, 128), float("nan"), dtype=torch.float32, device="cuda")
    bad = torch.tensor([0, 3, 8, 1], dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.PromoeError) as e:
        _lib.call("pm_moe_forward_routed", cache.handle, 0, xd.data_ptr(), 4, bad.data_ptr(), out.data_ptr(), 0, None,
                  None, 0, 0, 0, 0, None)
    assert "expert id" in str(e.value)
    # -1 marks a padding row: no expert runs on it and its output row is zeros
    good = torch.tensor([0, 3, -1, 1], dtype=torch.int32, device="cuda")
    _lib.call("pm_moe_forward_routed", cache.handle, 0, xd.data_ptr(), 4, good.data_ptr(), out.data_ptr(), 4, None,
              None, 0, 0, 0, 0, None)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    for r, e_id in enumerate([0, 3, -1, 1]):
        if e_id < 0:
            assert (got[r] == 0).all()
            continue
        ref = om.swiglu_mlp(x[r:r + 1], *model.experts[0][e_id], round_h_bf16=True)
        np.testing.assert_allclose(got[r:r + 1], ref, rtol=RTOL, atol=RTOL * np.abs(ref).max() * 0.25)
    cache.close()
