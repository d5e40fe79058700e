"""Writes tests/golden/policy_ref_*.json: cache event logs produced by the REFERENCE's own
compiled classes (oracle/_ref/ref_policy, built by `make -C oracle/ref_build` from the
reference checkout) on seeded synthetic request streams. The fixtures pin oracle/srs_policy.py
(tests/test_oracle_policy.py) and, through it, the product's cache engine.

Run from the repository root, on a machine that holds the reference checkout:
    make -C oracle/ref_build && python tests/golden/make_policy_golden.py
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from tests.policy_driver import make_stream  # noqa: E402

REF_BIN = ROOT / "oracle" / "_ref" / "ref_policy"
INT64_MAX = (1 << 63) - 1

# name, L, E, k, rate, policy, n_predict, batch, per_layer, steps, extra config
CASES = [
    ("c1_deepseek_layer_lru", 1, 64, 6, 0.375, "lru", 0, 32, True, 16, {}),
    ("c2_qwen_lru_nopred", 24, 60, 4, 0.375, "lru", 0, 8, True, 6, {}),
    ("c2_qwen_lru_pred4", 24, 60, 4, 0.375, "lru", 4, 8, True, 6, {}),
    ("c3_mixtral_lru_pred2", 32, 8, 2, 0.5, "lru", 2, 16, True, 6, {}),
    ("c5_dsv2_lru_rate025", 26, 64, 6, 0.25, "lru", 6, 4, True, 5, {}),
    ("fifo_pred", 4, 64, 8, 0.375, "fifo", 8, 4, True, 10, {}),
    ("static1", 6, 16, 2, 0.4, "static-1", 0, 2, True, 12, {}),
    ("static2_pred", 6, 16, 2, 0.4, "static-2", 2, 2, True, 12, {}),
    ("global_pool_lru_pred", 5, 32, 4, 0.3, "lru", 4, 2, False, 10, {}),
    ("one_line_per_layer", 27, 64, 6, 1.0 / 64, "lru", 0, 1, True, 4, {}),
    ("flags_reorder_only", 6, 32, 4, 0.375, "lru", 4, 3, True, 8,
     {"reorder_experts": True, "early_preempt": False, "chunk_prefetch": False}),
    ("flags_early_chunk_nopromote", 6, 32, 4, 0.375, "lru", 4, 3, True, 8,
     {"reorder_experts": False, "early_preempt": True, "chunk_prefetch": True, "promote_hit_in_prefetch": False}),
    ("nn_priority", 6, 32, 4, 0.375, "nn", 4, 2, True, 8, {}),
    ("min_trace", 4, 16, 2, 0.375, "min", 0, 1, True, 8, {}),
]


def add_nn_priorities(stream, L, E, seed):
    rng = np.random.default_rng(seed)
    out = [("priority", 0, np.round(rng.random((L, E)), 4).astype(np.float32).tolist())]
    for item in stream:
        if item[0] == "prefetch":
            out.append(("priority", item[1], np.round(rng.random((1, E)) * 50, 3).astype(np.float32).tolist()))
        out.append(item)
    return out


def add_min_traces(L, E, k, steps):
    traces, stream = [], []
    for seq in range(3):
        s = make_stream(100 + seq, L, E, k, steps=steps, batch=1)
        use, time = {}, 0
        for _, layer, ids in s:
            for i in ids:
                use.setdefault((layer, i), []).append(time)
            time += 1
        for l in range(L):
            for e in range(E):
                traces.append([seq, l, e, use.get((l, e), []) + [INT64_MAX]])
        stream.append(("seq", seq, None))
        stream += s
    return traces, stream


def run_reference(cfg: dict, L: int, E: int, n_param: int, stream, traces):
    lines = ["config " + " ".join(f"{k}={v}" for k, v in cfg.items()), f"init {L} {E} {n_param}"]
    for seq, l, e, times in traces:
        lines.append(f"trace {seq} {l} {e} {len(times)} " + " ".join(map(str, times)))
    for kind, a, b in stream:
        if kind == "layer":
            lines.append(f"layer {a} {len(b)} " + " ".join(map(str, b)))
        elif kind == "prefetch":
            lines.append(f"prefetch {a} {len(b)} " + " ".join(map(str, b)))
        elif kind == "priority":
            flat = [v for row in b for v in row]
            lines.append(f"priority {a} {len(b)} " + " ".join(repr(float(np.float32(v))) for v in flat))
        elif kind == "seq":
            lines.append(f"seq {a}")
    env = dict(os.environ, SPARSE_CACHE_LOG_LEVEL="FATAL")
    r = subprocess.run([str(REF_BIN)], input="\n".join(lines) + "\n", capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"reference harness failed ({r.returncode}):\n{r.stderr[-2000:]}")
    plan, events, orders, series = None, [], [], {}
    for ln in r.stdout.splitlines():
        tok = ln.split()
        if not tok:
            continue
        if tok[0] == "plan":
            plan = [int(v) for v in tok[1:]]
        elif tok[0] == "ev":
            events.append([int(v) for v in tok[1:]])
        elif tok[0] == "order":
            orders.append([int(v) for v in tok[2:]])
        elif tok[0] == "series":
            series[tok[1]] = [int(v) for v in tok[2:]]
    return plan, events, orders, series


def main():
    if not REF_BIN.exists():
        raise SystemExit("build the reference harness first: make -C oracle/ref_build")
    out_dir = Path(__file__).resolve().parent
    for name, L, E, k, rate, policy, n_pred, batch, per_layer, steps, extra in CASES:
        traces = []
        if policy == "min":
            traces, stream = add_min_traces(L, E, k, steps)
        else:
            stream = make_stream(11 + L + E, L, E, k, steps=steps, batch=batch, prefill_first=True, n_predict=n_pred)
            if policy == "nn":
                stream = add_nn_priorities(stream, L, E, 3)
        cfg = {"num_expert_per_token": k, "cache_rate": repr(float(rate)), "cache_policy": policy,
               "num_predict_expert_per_layer": n_pred, "per_layer_cache": per_layer}
        cfg.update(extra)
        # the harness issues each prefetch with min(n_predict, lines of pool 0) ids, as PredictWorker does
        plan, events, orders, series = run_reference(cfg, L, E, 3, clamp_prefetch(stream, L, E, rate, per_layer, n_pred),
                                                     traces)
        fixture = {"name": name, "num_layer": L, "num_expert": E, "num_expert_per_token": k, "cache_rate": rate,
                   "cache_policy": policy, "num_predict": n_pred, "per_layer_cache": per_layer, "extra": extra,
                   "num_per_expert_param": 3, "stream": [[a, b, c] for a, b, c in stream], "traces": traces,
                   "plan": plan, "events": [v for ev in events for v in ev], "orders": orders, "series": series}
        path = out_dir / f"policy_ref_{name}.json"
        path.write_text(json.dumps(fixture, separators=(",", ":")))
        print(f"{path.name}: {len(events)} events, {path.stat().st_size / 1024:.0f} KiB")


def clamp_prefetch(stream, L, E, rate, per_layer, n_pred):
    from oracle.srs_policy import plan_lines, total_lines
    lens = plan_lines(L if per_layer else 1, total_lines(rate, L, E))
    n = min(n_pred, lens[0])  # cache.cpp:130-131
    return [(a, b, c[:n]) if a == "prefetch" else (a, b, c) for a, b, c in stream]


if __name__ == "__main__":
    main()
