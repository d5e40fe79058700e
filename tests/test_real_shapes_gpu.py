"""The fused layer at the dimensions of the benchmark configurations (one or two layers each, a few
decode steps), against the oracles: routing ids and cache event log exact, outputs within the bf16
tolerance. The small-shape tests elsewhere cover the logic; these cover what only shows at size:
tile counts that do not divide, segments that mix a few rows with many, 60 experts on 22 or 23 lines,
8192-token prefill over 64 experts, 14336-wide uint4 matrices."""
import numpy as np
import pytest
import torch

from oracle import moe_math as om
from oracle import quant4 as oq
from oracle import srs_policy as sp
from promoe_b200 import synth
from tests.helpers import ShapeModel, dev_bf16

pytestmark = pytest.mark.gpu
RTOL = 2e-2      # bf16 experts
RTOL_Q4 = 3e-2   # uint4 experts, same dequantised weights on both sides


def check(y_dev, ref, rtol=RTOL):
    got = y_dev.float().cpu().numpy()
    np.testing.assert_allclose(got, ref, rtol=rtol, atol=rtol * np.abs(ref).max() * 0.25)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 5e-3


def decode_steps(model, cache, oc, batch, steps, preds=None, rtol=RTOL):
    """Decode steps through every layer; returns the library's event log."""
    cache.enable_event_log(True)
    cache.set("keep_routing", 1)
    for x in model.hidden_stream(batch, steps):
        xd = dev_bf16(x)
        for l in range(model.L):
            for (src, dst), (w1, b1, w2, b2) in sorted((preds or {}).items()):
                if src == l:
                    oc.prefetch_layer(dst, om.rank_experts(om.predictor_scores(x, w1, b1, w2, b2), oc.num_predict))
            y = cache.forward(l, xd)
            torch.cuda.synchronize()
            ids, w = cache.last_routing(l, batch, model.k)
            ref_ids, ref_w = model.canonical_routing(l, x)
            assert np.array_equal(ids, ref_ids.astype(np.int32)), "routing must be bit-exact"
            np.testing.assert_allclose(w, ref_w, rtol=1e-4, atol=1e-7)
            ref, ids64, _ = model.oracle_forward(l, x, report_experts=lambda u: np.asarray(oc.report_layer(l, u)))
            assert np.array_equal(ids64, ref_ids), "seed gives a routing gap below float32 resolution"
            check(y, ref, rtol)
    return cache.events()


def test_c2_qwen15_two_layers_with_predictor(lib):
    """Qwen1.5-MoE-A2.7B shape: 60 experts on 23 and 22 lines, top-4, batch 8, shared expert 5632 with a
    sigmoid gate, predictor MLP 2048-512-60 run inside the forward, four experts per predicted layer."""
    model = ShapeModel(seed=102, L=2, E=60, H=2048, I=1408, k=4, shared_I=5632, shared_gate=True)
    cache = model.make_cache(cache_rate=0.375, num_predict_expert_per_layer=4, predict_from_moe_input=True)
    assert cache.plan_slots() == [23, 22]
    rng = np.random.default_rng(7)
    preds = {}
    for src, dst in ((0, 0), (1, 1)):   # default window of a two-layer stack
        w1 = om.bf16_round((rng.standard_normal((512, model.H)) * 0.02).astype(np.float32))
        w2 = om.bf16_round((rng.standard_normal((model.E, 512)) * 0.02).astype(np.float32))
        preds[(src, dst)] = (w1, None, w2, None)
        cache.set_predictor(src, dst, dev_bf16(w1), None, dev_bf16(w2), None)
    oc = sp.SequentialCache(model.L, model.E, model.k, cache_rate=0.375, num_predict=4)
    events = decode_steps(model, cache, oc, batch=8, steps=4, preds=preds)
    assert events == oc.events
    kinds = [e[0] for e in events]
    assert kinds.count(sp.PREFETCH_MISS) > 0 and kinds.count(sp.PRECISE_HIT) > 0
    cache.close()


def test_c4_qwen2_57b_layer_mixed_rows(lib):
    """Qwen2-57B-A14B shape, batch 64 x top-8: 512 routed rows over 64 experts on 24 lines. Zipf routing
    gives some experts more than 16 rows and others one or two, so a launch mixes both kinds."""
    model = ShapeModel(seed=104, L=1, E=64, H=3584, I=2560, k=8, shared_I=20480, shared_gate=True)
    cache = model.make_cache(cache_rate=0.375, num_predict_expert_per_layer=0)
    assert cache.plan_slots() == [24]
    oc = sp.SequentialCache(1, 64, 8, cache_rate=0.375, num_predict=0)
    x0 = model.hidden_stream(64, 1)[0]
    counts = np.bincount(model.canonical_routing(0, x0)[0].reshape(-1), minlength=64)
    assert counts.max() > 16 and (counts[counts > 0] <= 4).any(), "the case must mix large and small experts"
    events = decode_steps(model, cache, oc, batch=64, steps=3)
    assert events == oc.events
    cache.close()


def test_c4_small_batch_device_planned(lib):
    """Same shape with 8 tokens: the device-planned launch for resident experts at hidden 3584, inter 2560."""
    model = ShapeModel(seed=105, L=1, E=64, H=3584, I=2560, k=8, shared_I=20480, shared_gate=True)
    cache = model.make_cache(cache_rate=0.375, num_predict_expert_per_layer=0)
    oc = sp.SequentialCache(1, 64, 8, cache_rate=0.375, num_predict=0)
    events = decode_steps(model, cache, oc, batch=8, steps=4)
    assert events == oc.events
    cache.close()


@pytest.mark.parametrize("rate", [0.25, 1.0])
def test_c5_prefill_8192_tokens(lib, rate):
    """DeepSeek-V2-Lite shape, one prompt pass of 4 x 2048 tokens over 64 experts (top-6, two shared experts
    as one of width 2816), with 16 lines (segments are cut when lines run out) and with every expert resident.
    The oracle's matmuls run in float32 torch on the host cores (float64 numpy would take minutes)."""
    T = 8192
    model = ShapeModel(seed=105, L=1, E=64, H=2048, I=1408, k=6, shared_I=2816)
    cache = model.make_cache(cache_rate=rate, num_predict_expert_per_layer=0)
    cache.enable_event_log(True)
    cache.set("keep_routing", 1)
    cache.set("seq_len", T)
    oc = sp.SequentialCache(1, 64, 6, cache_rate=rate, num_predict=0)
    x = om.bf16_round(model.rng.standard_normal((T, model.H)).astype(np.float32))
    y = cache.forward(0, dev_bf16(x))
    torch.cuda.synchronize()
    assert cache.get("tc_error") == "0" and int(cache.get("tc_launches")) > 0
    ids, w = cache.last_routing(0, T, model.k)
    ref_ids, ref_w = model.canonical_routing(0, x)
    assert np.array_equal(ids, ref_ids.astype(np.int32)), "routing must be bit-exact"
    assert om.routing_consistent(x, model.gate_w[0], model.gate_bias[0], ref_ids, model.k)
    order = np.asarray(oc.report_layer(0, om.unique_sorted_experts(ref_ids)))
    ref = om.moe_block_forward_f32(x, ref_ids, ref_w, model.experts[0], shared=model.shared[0], expert_order=order)
    check(y, ref)
    assert cache.events() == oc.events
    cache.close()


def test_c3_mixtral_uint4_decode_and_prefill(lib):
    """Mixtral-8x7B shape with uint4 group-128 experts (hidden 4096, inter 14336, 8 experts on 4 lines,
    top-2 renormalised): two decode steps of batch 16, then a 512-token prompt pass. The oracle computes
    with the weights its own unpacker dequantises from the same packed bytes."""
    from promoe_b200.engine import ExpertCache
    L, E, H, I, k = 1, 8, 4096, 14336, 2
    model = ShapeModel(seed=103, L=L, E=0, H=H, I=I, k=k, norm_topk=True, zipf_bias=False, gate_std=0.2)
    model.E = E
    g = torch.Generator(device="cuda").manual_seed(1031)
    model.gate_w = [(torch.randn((E, H), generator=g, device="cuda") * 0.2).to(torch.bfloat16).float().cpu().numpy()]
    cache = ExpertCache(L, E, num_expert_per_token=k, cache_rate=0.5, num_predict_expert_per_layer=0)
    cache.set_param_list(["w1.qweight", "w1.scale_zero", "w3.qweight", "w3.scale_zero", "w2.qweight", "w2.scale_zero"])
    packed = []

    class Dequantised:
        """Dequantises an expert when the oracle first touches it (float32, 3 x 235 MB)."""
        def __init__(self):
            self.memo = {}

        def __getitem__(self, e):
            if e not in self.memo:
                self.memo[e] = tuple(oq.dequantize(p, s) for p, s in packed[e])
            return self.memo[e]

    for e in range(E):
        mats = []
        for shape in ((I, H), (I, H), (H, I)):
            wm = torch.randn(shape, generator=g, device="cuda") * 0.02
            word, sz = synth.quantize_pack_torch(wm)
            mats.append((word.cpu().numpy().view(np.uint8).reshape(shape[0], shape[1] // 2), sz.cpu().numpy()))
        packed.append(mats)
        cache.register_expert(0, e, [a for pair in mats for a in pair])
    model.experts = [Dequantised()]
    cache.pin_all()
    cache.build_slab()
    assert cache.plan_slots() == [4]
    cache.set_layer_weights(0, dev_bf16(model.gate_w[0]), I, k, True, quant4=True)
    oc = sp.SequentialCache(L, E, k, cache_rate=0.5, num_predict=0, num_per_expert_param=6)
    decode_steps(model, cache, oc, batch=16, steps=2, rtol=RTOL_Q4)
    # prompt pass: 1024 routed rows over 8 experts
    T = 512
    x = om.bf16_round(model.rng.standard_normal((T, H)).astype(np.float32))
    cache.set("seq_len", T)
    y = cache.forward(0, dev_bf16(x))
    torch.cuda.synchronize()
    ids, w = cache.last_routing(0, T, k)
    ref_ids, ref_w = model.canonical_routing(0, x)
    assert np.array_equal(ids, ref_ids.astype(np.int32))
    assert om.routing_consistent(x, model.gate_w[0], None, ref_ids, k)
    order = np.asarray(oc.report_layer(0, om.unique_sorted_experts(ref_ids)))
    ref = om.moe_block_forward_f32(x, ref_ids, ref_w, model.experts[0], expert_order=order)
    check(y, ref, RTOL_Q4)
    assert int(cache.get("q4_expanded")) >= E      # the prompt pass ran on the tensor cores from expanded weights
    assert cache.events() == oc.events
    cache.close()
