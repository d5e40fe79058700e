"""The two trace formats of the Belady (MIN) policy, CacheOracle.load_from_tensor and
load_from_file (src/cpp_worker/cache.cpp:431-489,592-644), on a policy-only context: both loaders
must give the library the use times the format defines, checked by replaying the traced requests
through the library and through the oracle fed with use times computed here independently."""
import json

import numpy as np
import pytest
import torch

from oracle import srs_policy as sp
from promoe_b200 import cpp_worker as cw
from promoe_b200.engine import ExpertCache

L, E, K = 2, 6, 2


def make_trace(seed=5):
    rng = np.random.default_rng(seed)
    seqs = []
    for prompt_len, reply_len in ((3, 4), (2, 5)):
        prompt = [[sorted(int(v) for v in rng.choice(E, size=K, replace=False)) for _ in range(prompt_len)] for _ in range(L)]
        reply = [[[int(v) for v in rng.choice(E, size=K, replace=False)] for _ in range(L)] for _ in range(reply_len)]
        seqs.append((prompt_len, reply_len, prompt, reply))
    return seqs


def expected_use_times(seq):
    """use times of one sequence: one tick per (iteration, layer), prompt first."""
    prompt_len, reply_len, prompt, reply = seq
    use, t = {}, 0
    for l in range(L):
        for e in sorted({e for tok in prompt[l] for e in tok}):
            use.setdefault((l, e), []).append(t)
        t += 1
    for r in range(reply_len):
        for l in range(L):
            for e in reply[r][l]:
                use.setdefault((l, e), []).append(t)
            t += 1
    return use


def requests(seq):
    prompt_len, reply_len, prompt, reply = seq
    out = [[(l, sorted({e for tok in prompt[l] for e in tok})) for l in range(L)]]
    for r in range(reply_len):
        out.append([(l, sorted(reply[r][l])) for l in range(L)])
    return out


def replay(cache, seqs):
    cache.enable_event_log(True)
    oc = sp.SequentialCache(L, E, K, cache_rate=0.5, cache_policy="min", num_predict=0)
    for s, seq in enumerate(seqs):
        use = expected_use_times(seq)
        for l in range(L):
            for e in range(E):
                oc.add_use_times(s, l, e, use.get((l, e), []))
    for s, seq in enumerate(seqs):
        cache.set_cur_seq(s)
        oc.set_cur_seq(s)
        for it in requests(seq):
            for l, ids in it:
                cache.report_layer(l, ids)
                oc.report_layer(l, ids)
                for e in ids:      # ExpertHook around every expert (the oracle's report_layer includes it)
                    cache.report_expert(l, e)
                    cache.expert_done(l, e)
                cache.layer_done(l)
    assert cache.events() == oc.events and len(oc.events) > 20
    assert any(ev[4] >= 0 for ev in oc.events), "the replay must evict"


def min_cache():
    cache = ExpertCache(L, E, num_expert_per_token=K, cache_rate=0.5, cache_policy="min", num_predict_expert_per_layer=0)
    cache.build_policy_only()
    return cache


def test_load_from_tensor():
    seqs = make_trace()
    max_pre = max(len({e for tok in s[2][l] for e in tok}) for s in seqs for l in range(L))
    pre_len = torch.zeros((len(seqs), L), dtype=torch.int32)
    pre_sel = torch.zeros((len(seqs), L, max_pre), dtype=torch.int32)
    metas, dec = [], []
    for s, (prompt_len, reply_len, prompt, reply) in enumerate(seqs):
        for l in range(L):
            ids = sorted({e for tok in prompt[l] for e in tok})
            pre_len[s, l] = len(ids)
            pre_sel[s, l, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        for r in range(reply_len):
            metas.append([s, r])
            dec.append(reply[r])
    cache = min_cache()
    cw.CacheOracle(cache, L, E).load_from_tensor(torch.tensor(metas), pre_len, pre_sel, torch.tensor(dec, dtype=torch.int32))
    replay(cache, seqs)
    cache.close()
    bad = torch.tensor(metas)
    bad[1, 1] = 7                                  # a reply token out of order: refused like the reference's CHECK
    with pytest.raises(ValueError):
        cw.CacheOracle(min_cache(), L, E).load_from_tensor(bad, pre_len, pre_sel, torch.tensor(dec, dtype=torch.int32))


def test_load_from_file(tmp_path):
    seqs = make_trace(seed=6)
    doc = {}
    for s, (prompt_len, reply_len, prompt, reply) in enumerate(seqs):
        entry = {"prompt_len": prompt_len}
        for l in range(L):
            entry[str(l)] = {str(t): prompt[l][t] for t in range(prompt_len)}
            entry[str(l)].update({str(prompt_len + r): reply[r][l] for r in range(reply_len)})
        doc[str(s)] = entry
    path = tmp_path / "trace.json"
    path.write_text(json.dumps(doc))
    cache = min_cache()
    cw.CacheOracle(cache, L, E).load_from_file(str(path))
    replay(cache, seqs)
    cache.close()
