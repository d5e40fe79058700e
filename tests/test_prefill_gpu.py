"""Prefill-size batches: the tcgen05 / TMEM grouped GEMM path (more than 16 rows per expert) through
the fused layer, against the float64 oracle; routing and cache log exact."""
import numpy as np
import pytest
import torch

from oracle import srs_policy as sp
from tests.helpers import TinyModel, dev_bf16

pytestmark = pytest.mark.gpu
RTOL = 2e-2


def run_prefill(model, cfg, T, steps=2, tc=True):
    cache = model.make_cache(**cfg)
    cache.set("tc_prefill", int(tc))
    cache.set("keep_routing", 1)
    cache.enable_event_log(True)
    oc = sp.SequentialCache(model.L, model.E, model.k, cache_rate=cfg["cache_rate"], num_predict=0)
    worst = 0.0
    for x in model.hidden_stream(T, steps):
        xd = dev_bf16(x)
        for l in range(model.L):
            cache.set("seq_len", T)
            y = cache.forward(l, xd)
            torch.cuda.synchronize()
            assert cache.get("tc_error") == "0"
            ids, _ = cache.last_routing(l, T, model.k)
            ref_ids, _ = model.canonical_routing(l, x)
            assert np.array_equal(ids, ref_ids.astype(np.int32))
            ref, _, _ = model.oracle_forward(l, x, report_experts=lambda u: np.asarray(oc.report_layer(l, u)))
            got = y.float().cpu().numpy()
            np.testing.assert_allclose(got, ref, rtol=RTOL, atol=RTOL * np.abs(ref).max() * 0.25)
            worst = max(worst, float(np.linalg.norm(got - ref) / np.linalg.norm(ref)))
    assert cache.events() == oc.events
    launches = int(cache.get("tc_launches"))
    cache.close()
    return worst, launches


@pytest.mark.parametrize("T,rate", [(300, 1.0), (300, 0.5), (129, 0.25), (1024, 0.5)])
def test_prefill_matches_oracle(lib, T, rate):
    model = TinyModel(seed=31, L=2, E=8, H=256, I=128, k=2, shared_I=256, shared_gate=True)
    worst, launches = run_prefill(model, dict(cache_rate=rate, num_predict_expert_per_layer=0), T)
    assert launches > 0, "the tensor-core path must have been taken"
    assert worst < 5e-3


def test_prefill_wide_shapes(lib):
    """K loops longer than the stage ring and inter that is not a multiple of the 128-column tile."""
    model = TinyModel(seed=32, L=1, E=4, H=1024, I=320, k=2, shared_I=0)
    worst, launches = run_prefill(model, dict(cache_rate=1.0, num_predict_expert_per_layer=0), 200, steps=1)
    assert launches > 0 and worst < 5e-3


def test_prefill_paths_agree(lib):
    """Same inputs with the tensor-core path switched off (staged mma.sync kernel): both within tolerance."""
    model = TinyModel(seed=33, L=1, E=8, H=256, I=128, k=2)
    w1, n1 = run_prefill(model, dict(cache_rate=0.5, num_predict_expert_per_layer=0), 200, steps=1, tc=False)
    assert n1 == 0 and w1 < 5e-3
