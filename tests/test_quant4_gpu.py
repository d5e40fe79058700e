"""uint4 group-128 experts: the fused dequantising GEMV against the float64 oracle fed with the
SAME dequantised weights (tolerance rtol 3e-2), at kernel level and through the fused layer."""
import numpy as np
import pytest
import torch

from oracle import moe_math as om
from oracle import quant4 as oq
from oracle import srs_policy as sp
from promoe_b200 import _lib
from promoe_b200 import quant4 as pq
from tests.helpers import TinyModel, bf16_weights, dev, dev_bf16, ptr

pytestmark = pytest.mark.gpu
RTOL_Q4 = 3e-2


def q4_expert(rng, H, I):
    """Three quantised matrices: device tensors for the kernel, dequantised float32 for the oracle."""
    out_dev, out_deq, raw = [], [], []
    for shape in ((I, H), (I, H), (H, I)):
        packed, sz = pq.quantize_pack(bf16_weights(rng, shape))
        out_dev += [dev(packed), dev(sz)]
        out_deq.append(oq.dequantize(packed, sz))
        raw += [packed, sz]
    return out_dev, out_deq, raw


@pytest.mark.parametrize("H,inters,rows", [(128, [128], [1]), (256, [128, 256], [5, 8]),
                                           (1024, [512, 512, 1024], [3, 16, 9]), (4096, [1792], [2]),
                                           # 132 chunks of 16 rows: more than the one-launch kernel's chunk
                                           # table holds, so the gate/up + down launch pair runs
                                           (128, [128], [2100])])
def test_q4_ffn_matches_oracle(lib, H, inters, rows):
    rng = np.random.default_rng(3 + H)
    T = 16
    x = om.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    xd = dev_bf16(x)
    arr = (_lib.pm_ffn_group * len(inters))()
    keep, deq, row_token, start = [], [], [], 0
    for i, (inter, r) in enumerate(zip(inters, rows)):
        d, q, _ = q4_expert(rng, H, inter)
        keep += d
        deq.append(q)
        arr[i] = _lib.pm_ffn_group(ptr(d[0]), ptr(d[2]), ptr(d[4]), ptr(d[1]), ptr(d[3]), ptr(d[5]), start, r, inter, 0)
        row_token += list(rng.integers(0, T, size=r))
        start += r
    rt = dev(np.array(row_token, np.int32))
    nbytes = _lib.call("pm_k_swiglu_ffn_scratch_bytes", len(inters), start, max(inters), H)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    yexp = torch.full((start, H), float("nan"), dtype=torch.float32, device="cuda")
    _lib.call("pm_k_swiglu_ffn", arr, len(inters), 1, ptr(xd), H, ptr(rt), start, ptr(yexp), ptr(scratch), nbytes, None)
    torch.cuda.synchronize()
    y = yexp.cpu().numpy()
    assert np.isfinite(y).all()
    s0 = 0
    for (wg, wu, wd), r in zip(deq, rows):
        ref = om.swiglu_mlp(x[row_token[s0:s0 + r]], wg, wu, wd, round_h_bf16=True)
        np.testing.assert_allclose(y[s0:s0 + r], ref, rtol=RTOL_Q4, atol=RTOL_Q4 * np.abs(ref).max() * 0.1)
        assert np.linalg.norm(y[s0:s0 + r] - ref) / np.linalg.norm(ref) < 5e-3
        s0 += r


def test_q4_rejects_bad_shapes(lib):
    arr = (_lib.pm_ffn_group * 1)()
    arr[0] = _lib.pm_ffn_group(8, 8, 8, 8, 8, 8, 0, 1, 64, 0)       # inter % 128 != 0
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_swiglu_ffn", arr, 1, 1, 8, 128, 8, 1, 8, 8, 1 << 20, None)
    arr[0] = _lib.pm_ffn_group(8, 8, 8, None, None, None, 0, 1, 128, 0)  # scale/zero tensors missing
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_swiglu_ffn", arr, 1, 1, 8, 128, 8, 1, 8, 8, 1 << 20, None)


def test_q4_fused_layer_mixtral_like(lib):
    """Mixtral-shaped tiny stack with uint4 experts in the cache: outputs vs the oracle on the
    dequantised weights, routing and cache log exact."""
    from promoe_b200.engine import ExpertCache
    model = TinyModel(seed=21, L=2, E=8, H=256, I=128, k=2, norm_topk=True, zipf_bias=False, gate_std=0.2)
    rng = np.random.default_rng(4)
    cache = ExpertCache(model.L, model.E, num_expert_per_token=model.k, cache_rate=0.5, num_predict_expert_per_layer=0)
    cache.set_param_list(["w1.qweight", "w1.scale_zero", "w3.qweight", "w3.scale_zero", "w2.qweight", "w2.scale_zero"])
    for l in range(model.L):
        for e in range(model.E):
            _, deq, raw = q4_expert(rng, model.H, model.I)
            model.experts[l][e] = tuple(deq)          # the oracle computes with the dequantised weights
            cache.register_expert(l, e, raw)
    cache.pin_all()
    cache.build_slab()
    for l in range(model.L):
        cache.set_layer_weights(l, dev_bf16(model.gate_w[l]), model.I, model.k, True, quant4=True)
    cache.enable_event_log(True)
    cache.set("keep_routing", 1)
    oc = sp.SequentialCache(model.L, model.E, model.k, cache_rate=0.5, num_predict=0, num_per_expert_param=6)
    for x in model.hidden_stream(6, 4):
        for l in range(model.L):
            y = cache.forward(l, dev_bf16(x))
            torch.cuda.synchronize()
            ids, _ = cache.last_routing(l, 6, model.k)
            ref_ids, _ = model.canonical_routing(l, x)
            assert np.array_equal(ids, ref_ids.astype(np.int32))
            ref, _, _ = model.oracle_forward(l, x, report_experts=lambda u: np.asarray(oc.report_layer(l, u)))
            got = y.float().cpu().numpy()
            np.testing.assert_allclose(got, ref, rtol=RTOL_Q4, atol=RTOL_Q4 * np.abs(ref).max() * 0.25)
    assert int(cache.get("q4_expanded")) == 0          # decode batches stay on the split-K tiles
    # a prompt pass: 640 tokens x top-2 over 8 experts = 160 rows per expert on average, so every segment's
    # experts are expanded to bf16 once and run on the tensor cores
    T = 640
    x = om.bf16_round(rng.standard_normal((T, model.H)).astype(np.float32))
    cache.set("seq_len", T)
    for l in range(model.L):
        y = cache.forward(l, dev_bf16(x))
        torch.cuda.synchronize()
        ids, _ = cache.last_routing(l, T, model.k)
        ref_ids, _ = model.canonical_routing(l, x)
        assert np.array_equal(ids, ref_ids.astype(np.int32))
        ref, _, _ = model.oracle_forward(l, x, report_experts=lambda u: np.asarray(oc.report_layer(l, u)))
        got = y.float().cpu().numpy()
        np.testing.assert_allclose(got, ref, rtol=RTOL_Q4, atol=RTOL_Q4 * np.abs(ref).max() * 0.25)
    assert int(cache.get("q4_expanded")) >= model.E * model.L and int(cache.get("tc_launches")) >= model.L
    assert cache.events() == oc.events
    cache.close()


def test_gptq_checkpoint_layout_through_inject_model(lib):
    """A Mixtral-style model whose experts carry AutoGPTQ tensors (qweight / qzeros / scales / g_idx):
    adapt_quantised_linear rewrites them to the library layout, inject_model registers and moves
    them, the fused layer computes with them; the oracle uses its own GPTQ dequantiser."""
    from dataclasses import dataclass
    from torch import nn
    from promoe_b200.utils import inject_model
    from tests.test_quant_layouts import gptq_tensors

    @dataclass
    class Cfg:
        _name_or_path: str = "mistralai/Mixtral-8x7B-Instruct-v0.1"
        num_experts_per_tok: int = 2

    class QLinear(nn.Module):
        def __init__(self, rng, in_f, out_f):
            super().__init__()
            qw, qz, sc, _, _ = gptq_tensors(rng, in_f, out_f)
            self.register_buffer("qweight", torch.from_numpy(qw))
            self.register_buffer("qzeros", torch.from_numpy(qz))
            self.register_buffer("scales", torch.from_numpy(sc))
            self.register_buffer("g_idx", torch.arange(in_f, dtype=torch.int32) // 128)
            self.dense = oq.dequantize_gptq(qw, qz, sc)          # [out, in] float32, oracle side

    class Expert(nn.Module):
        def __init__(self, rng, H, I):
            super().__init__()
            self.w1, self.w3, self.w2 = QLinear(rng, H, I), QLinear(rng, H, I), QLinear(rng, I, H)

    class Block(nn.Module):
        def __init__(self, rng, H, E, I):
            super().__init__()
            self.gate = nn.Linear(H, E, bias=False)
            self.experts = nn.ModuleList([Expert(rng, H, I) for _ in range(E)])

        def report_experts(self, ids):
            return ids

    class Layer(nn.Module):
        def __init__(self, rng, H, E, I):
            super().__init__()
            self.block_sparse_moe = Block(rng, H, E, I)

        def forward(self, h):
            return (self.block_sparse_moe(h),)

    class Model(nn.Module):
        def __init__(self, L, H, E, I):
            super().__init__()
            rng = np.random.default_rng(9)
            self.config = Cfg()
            self.model = nn.Module()
            self.model.layers = nn.ModuleList([Layer(rng, H, E, I) for _ in range(L)])

        def forward(self, h):
            return [layer(h)[0] for layer in self.model.layers]

    L, H, E, I, k = 2, 256, 8, 128, 2
    torch.manual_seed(3)
    model = Model(L, H, E, I).eval()
    gates, dense = [], []
    for layer in model.model.layers:
        blk = layer.block_sparse_moe
        with torch.no_grad():
            blk.gate.weight.copy_((blk.gate.weight * 3).to(torch.bfloat16).float())
        gates.append(blk.gate.weight.detach().numpy().copy())
        dense.append([(e.w1.dense, e.w3.dense, e.w2.dense) for e in blk.experts])
        for e in blk.experts:
            for lin in (e.w1, e.w3, e.w2):
                pq.adapt_quantised_linear(lin, "gptq")
                assert set(lin._buffers) == {"qweight", "scale_zero"}
    mngr = inject_model(model, num_moe_layer=L, num_expert_per_layer=E, num_expert_per_token=k, cache_rate=0.5,
                        num_predict_expert_per_layer=0)
    model.to("cuda")
    rng = np.random.default_rng(4)
    for _ in range(3):
        x = om.bf16_round(rng.standard_normal((5, H)).astype(np.float32))
        with torch.no_grad():
            ys = model(dev_bf16(x).view(5, 1, H))
        torch.cuda.synchronize()
        for l in range(L):
            ref, _, _ = om.moe_block_forward(x, gates[l], dense[l], k, True, round_h_bf16=True)
            got = ys[l].float().cpu().numpy().reshape(5, H)
            np.testing.assert_allclose(got, ref, rtol=RTOL_Q4, atol=RTOL_Q4 * np.abs(ref).max() * 0.25)
    assert mngr.metas.cache.stats()["precise_miss"] > 0
