"""Pins the MoE arithmetic oracle against outputs of the stock HuggingFace transformers blocks
(tests/golden/moe_hf_*.npz, written by tests/golden/make_moe_golden.py)."""
from pathlib import Path

import numpy as np
import pytest

from oracle import moe_math as om

GOLDEN = sorted((Path(__file__).parent / "golden").glob("moe_hf_*.npz"))


def load(path):
    z = np.load(path)
    d = {k: z[k] for k in z.files}
    for k in ("w_gate", "w_up", "w_down", "shared_w_gate", "shared_w_up", "shared_w_down"):
        if k in d:
            d[k] = om.from_bf16_bits(d[k])
    return d


def test_fixtures_exist():
    assert len(GOLDEN) >= 5


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem.replace("moe_hf_", ""))
def test_block_matches_stock_transformers(path):
    d = load(path)
    E = d["w_gate"].shape[0]
    experts = [(d["w_gate"][e], d["w_up"][e], d["w_down"][e]) for e in range(E)]
    shared = (d["shared_w_gate"], d["shared_w_up"], d["shared_w_down"]) if "shared_w_gate" in d else None
    seen = []

    def report(ids):  # the hook point the reference replaces (utils/__init__.py:82-89)
        seen.append(ids.copy())
        return ids

    y, ids, w = om.moe_block_forward(d["x"], d["gate_w"], experts, int(d["top_k"]), bool(d["norm_topk"]),
                                     float(d["routed_scale"]), shared=shared,
                                     shared_gate_w=d.get("shared_gate_w"), report_experts=report)
    # stock DeepseekV2 uses topk(sorted=False): compare as sets per token, and weights by expert id
    ref_ids, ref_w = d["ids"], d["weights"]
    order_ref = np.argsort(ref_ids, axis=1)
    order_got = np.argsort(ids, axis=1)
    assert np.array_equal(np.take_along_axis(ref_ids, order_ref, 1), np.take_along_axis(ids, order_got, 1))
    np.testing.assert_allclose(np.take_along_axis(w, order_got, 1), np.take_along_axis(ref_w, order_ref, 1),
                               rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(y, d["y"], rtol=2e-4, atol=2e-5)
    assert len(seen) == 1 and np.array_equal(seen[0], np.unique(ids))
    if str(d["family"]) != "deepseek_v2":  # sorted top-k: descending probability
        assert np.array_equal(ids, ref_ids)


def test_report_experts_may_reorder_without_changing_the_output():
    d = load(GOLDEN[0])
    E = d["w_gate"].shape[0]
    experts = [(d["w_gate"][e], d["w_up"][e], d["w_down"][e]) for e in range(E)]
    y0, _, _ = om.moe_block_forward(d["x"], d["gate_w"], experts, int(d["top_k"]), False)
    y1, _, _ = om.moe_block_forward(d["x"], d["gate_w"], experts, int(d["top_k"]), False,
                                    report_experts=lambda ids: ids[::-1].copy())
    np.testing.assert_allclose(y0, y1, rtol=1e-12, atol=1e-12)


def test_canonical_logits_equal_float64_logits_closely():
    rng = np.random.default_rng(0)
    for T, H, E in [(3, 64, 8), (5, 2048, 60), (2, 3584, 64), (4, 72, 5)]:
        x = om.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
        w = om.bf16_round((rng.standard_normal((E, H)) * 0.02).astype(np.float32))
        b = rng.standard_normal(E).astype(np.float32)
        a = om.gate_logits_canonical(x, w, b)
        ref = om.gate_logits(x, w, b)
        assert a.dtype == np.float32
        np.testing.assert_allclose(a, ref, rtol=1e-4, atol=1e-5)


def test_topk_ties_and_permute():
    s = np.array([[0.5, 0.9, 0.9, 0.1], [0.2, 0.2, 0.2, 0.2]])
    assert om.topk_desc(s, 2).tolist() == [[1, 2], [0, 1]]
    ids = np.array([[2, 0], [1, 2], [0, 1]], np.int32)
    counts, offsets, row_token, pos = om.permute(ids, 4)
    assert counts.tolist() == [2, 2, 2, 0] and offsets.tolist() == [0, 2, 4, 6, 6]
    assert row_token.tolist() == [0, 2, 1, 2, 0, 1]
    assert pos.reshape(3, 2).tolist() == [[4, 0], [2, 5], [1, 3]]


def test_bf16_round_trip():
    rng = np.random.default_rng(1)
    a = rng.standard_normal(1000).astype(np.float32)
    r = om.bf16_round(a)
    assert np.array_equal(om.from_bf16_bits(om.to_bf16_bits(a)), r)
    assert np.all(np.abs(r - a) <= np.abs(a) * 2.0 ** -8)
    import torch
    assert np.array_equal(r, torch.from_numpy(a).to(torch.bfloat16).float().numpy())


def test_uint4_packers_agree():
    """The numpy packer, the torch packer of the synthetic stacks and the oracle's independent unpacker
    describe the same layout."""
    import torch
    from oracle import quant4 as oq
    from promoe_b200 import quant4 as pq
    from promoe_b200.synth import quantize_pack_torch
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((12, 384)) * 0.02).astype(np.float32)
    packed, sz = pq.quantize_pack(w)
    word, sz_t = quantize_pack_torch(torch.from_numpy(w))
    assert np.array_equal(word.numpy().view(np.uint8).reshape(12, -1), packed)
    assert np.array_equal(sz_t.numpy(), sz)
    deq = oq.dequantize(packed, sz)
    assert np.abs(deq - w).max() <= np.abs(w).max() / 15 + 1e-6      # within one quantisation step
    q, s, z = pq.quantize(w)
    ref = (q.reshape(12, 3, 128).astype(np.float32) - z.astype(np.float32)[..., None]) * s.astype(np.float32)[..., None]
    assert np.array_equal(deq, ref.reshape(12, 384))
