"""History-based predictor inputs and the NN cache policy driven by them (the reference's
weighted_decode_cumsum / decode_cumsum / last_use_distance modes, src/cpp_worker/predictor.cpp:48-80,
143-175,351-365; fed from src/cpp_worker/prefetcher.cpp:462-479), on a policy-only context: the input
tensor equals a numpy restatement after every iteration, and the cache decisions equal the oracle's
NN policy given the same scores."""
import numpy as np
import pytest
import torch

from oracle import srs_policy as sp
from promoe_b200 import cpp_worker as cw

L, E, K = 3, 8, 2


def make_mngr(mode, **cfg):
    meta = cw.ModuleMeta(L, E)
    meta.init_param_list(["w"])
    conf = {"cache_rate": "0.5", "num_expert_per_token": str(K), "num_predict_expert_per_layer": "0",
            "cache_policy": "nn", "predict_input_mode": mode}
    conf.update({k: str(v) for k, v in cfg.items()})
    meta.init_from_map(conf)
    meta.cache.build_policy_only()
    meta.cache.enable_event_log(True)
    return cw.PrefetchMngr(meta, cw.ModelLoader(meta), cw.PredictorBase.create(meta)), meta.cache


def skewed_ids(rng, n):
    p = 1.0 / (np.arange(E) + 1.0) ** 1.2
    return sorted(int(v) for v in rng.choice(E, size=n, replace=False, p=p / p.sum()))


class NumpyHistory:
    def __init__(self, mode, decay=2, dmax=10):
        self.mode, self.decay, self.dmax = mode, decay, dmax
        self.cnt, self.dist, self.wsum = (np.zeros((L, E), np.float32) for _ in range(3))

    def add(self, l, ids):
        if len(ids) > K:
            if l == 0 and self.mode != "one_token":
                self.cnt[:], self.dist[:], self.wsum[:] = 0, 0, 0
            return
        self.dist[l] += 1
        self.wsum[l] /= np.float32(self.decay)
        for e in ids:
            self.cnt[l, e] += 1
            self.dist[l, e] = 0
            self.wsum[l, e] += 1

    def input(self):
        if self.mode == "decode_cumsum":
            s = self.cnt.sum(1, keepdims=True)
            return np.where(s > 0, self.cnt / np.maximum(s, 1), 0).astype(np.float32)
        if self.mode == "last_use_distance":
            return (np.maximum(self.dmax - self.dist, 0) / np.float32(self.dmax)).astype(np.float32)
        return self.wsum if self.mode == "weighted_decode_cumsum" else self.cnt


@pytest.mark.parametrize("mode", ["weighted_decode_cumsum", "decode_cumsum", "last_use_distance"])
def test_history_input_and_nn_policy(mode):
    mngr, cache = make_mngr(mode)
    oc = sp.SequentialCache(L, E, K, cache_rate=0.5, cache_policy="nn", num_predict=0)
    hist = NumpyHistory(mode)
    rng = np.random.default_rng(11)
    for it in range(24):
        prompt = it in (0, 12)                        # two sequences: a prompt pass, then decode steps
        for l in range(L):
            ids = skewed_ids(rng, 5 if prompt else K)
            t = torch.tensor(ids, dtype=torch.int64)
            mngr.report_one_layer(l, t)
            oc.report_layer(l, ids)
            for e in t.tolist():
                mngr.report_one_expert(l, e)
                mngr.one_expert_done(l, e)
            hist.add(l, ids)
            mngr.one_moe_layer_done(l)
        np.testing.assert_allclose(cache.history_input(), hist.input(), rtol=1e-6, atol=0)
        oc.update_priority(hist.input(), 0)           # what the iteration's prediction handed the policy
    assert cache.events() == oc.events
    assert any(ev[4] >= 0 for ev in oc.events)
    assert len(mngr.profiler.to_tensor("predict_time")) == 24
    cache.close()


def test_history_model_file_and_prefetch(tmp_path):
    """A TorchScript model file for the history modes (one file, applied to the rows, summed over
    them) and prefetching of the top-n experts it ranks."""
    class Shift(torch.nn.Module):            # scores of every layer = twice the summed history rows
        def forward(self, x):
            return (2.0 * x).repeat(1, 3)    # [rows, 3 * E] -> reshaped to [rows, 3, E], summed over rows
    path = tmp_path / "history-model.pt"
    torch.jit.script(Shift()).save(str(path))
    mngr, cache = make_mngr("weighted_decode_cumsum", num_predict_expert_per_layer=2, cache_policy="lru",
                            predictor_model_path=str(path))
    mngr.predictor.load_model()
    assert mngr.predictor.history_model is not None
    rng = np.random.default_rng(2)
    for it in range(6):
        for l in range(L):
            ids = skewed_ids(rng, K)
            mngr.report_one_layer(l, torch.tensor(ids, dtype=torch.int64))
            mngr.one_moe_layer_done(l)
    scores, start = mngr.predictor.history_scores(torch.from_numpy(cache.history_input()))
    assert scores.shape == (3, E) and start == 0
    np.testing.assert_allclose(scores.numpy(), 2.0 * cache.history_input().sum(0, keepdims=True).repeat(3, 0), rtol=1e-6)
    kinds = [ev[0] for ev in cache.events()]
    assert kinds.count(sp.PREFETCH_MISS) + kinds.count(sp.PREFETCH_HIT) > 0
    cache.close()
