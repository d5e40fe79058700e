"""Pins the policy oracle (and the product's engine) against event logs that the REFERENCE's
own compiled classes produced (tests/golden/policy_ref_*.json, written by
tests/golden/make_policy_golden.py from oracle/_ref/ref_policy)."""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import srs_policy as sp
from tests.policy_driver import run_oracle, run_product

GOLDEN = sorted((Path(__file__).parent / "golden").glob("policy_ref_*.json"))


def load(path):
    fx = json.loads(path.read_text())
    stream = []
    for kind, a, b in fx["stream"]:
        if kind == "priority":
            b = np.asarray(b, np.float32)
        stream.append((kind, a, b))
    traces = {(seq, l, e): times for seq, l, e, times in fx["traces"]}
    kw = dict(num_layer=fx["num_layer"], num_expert=fx["num_expert"],
              num_expert_per_token=fx["num_expert_per_token"], cache_rate=fx["cache_rate"],
              cache_policy=fx["cache_policy"], num_predict=fx["num_predict"],
              per_layer_cache=fx["per_layer_cache"], num_per_expert_param=fx["num_per_expert_param"])
    kw.update(fx["extra"])
    ev = np.asarray(fx["events"], np.int64).reshape(-1, 6)
    return fx, stream, traces, kw, [tuple(int(v) for v in r) for r in ev]


def test_fixtures_exist():
    assert len(GOLDEN) >= 14


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem.replace("policy_ref_", ""))
def test_oracle_reproduces_reference(path):
    fx, stream, traces, kw, ref_events = load(path)
    events, orders, cache = run_oracle(stream, traces=traces, **kw)
    assert cache.lens == fx["plan"]
    assert events == ref_events
    assert orders == fx["orders"]


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem.replace("policy_ref_", ""))
def test_product_reproduces_reference(lib, path):
    fx, stream, traces, kw, ref_events = load(path)
    events, orders, stats = run_product(stream, traces=traces, **kw)
    assert events == ref_events
    assert orders == fx["orders"]
    kinds = [e[0] for e in ref_events]
    assert (stats.precise_hit, stats.precise_miss, stats.prefetch_hit, stats.prefetch_miss) == tuple(
        kinds.count(k) for k in range(4))
    # the per-forward series the reference's own TimeProfiler recorded for the same requests
    assert stats.series == fx["series"]


def test_heap_remove_never_sifts_up():
    """utils.hpp:341-349: after swapping the last node into the hole only heapify_down runs, so a
    node smaller than its new parent stays below it. The oracle keeps that behaviour."""
    h = sp.MinHeap()
    nodes = [[p, 0, i] for i, p in enumerate([1.0, 10.0, 2.0, 11.0, 12.0, 3.0, 4.0])]
    for n in nodes:
        h.push(n)
    h.remove(nodes[3])                   # hole under the 10.0 branch, filled by the 4.0 node
    assert h.buf[3][0] == 4.0 and h.buf[1][0] == 10.0   # 4.0 sits under 10.0: heap order is broken
