"""CPU oracle for the expert cache policy and fetch schedule. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference leg may
import this module, and only as the checker; the product path never calls it.

It restates, in plain Python, the single-threaded core of the reference's cache:
  * CacheMngr (src/cpp_worker/cache.cpp:57-132 line planning, :236-312 hit/miss),
  * the policies FIFO / LRU / Static-n / NN / MIN (src/cpp_worker/cache.hpp:24-224,
    src/cpp_worker/cache.cpp:313-399,490-583) with the reference's DoubleLinkedList and
    MinHeap (src/cpp_worker/utils.hpp:213-357; `remove` sifts down only),
  * the FetchScheduleWorker state machine (src/cpp_worker/prefetcher.cpp:6-161,494-659)
    run as a *sequential schedule*: every queued copy task is processed, and its copy taken
    as complete, before the next request is looked at. Without prefetching the reference is
    deterministic and this schedule is exactly what it does; with prefetching the reference's
    outcome depends on thread timing and this schedule is the timing in which the copy engine
    always keeps up.

Pinning. tests/golden/policy_ref_*.json hold event logs produced by the reference's own
compiled classes (oracle/ref_build builds them from the reference checkout into oracle/_ref/);
tests/test_oracle_policy.py replays them through this file.
"""
from __future__ import annotations

import math
from collections import deque

import numpy as np

PRECISE_HIT, PRECISE_MISS, PREFETCH_HIT, PREFETCH_MISS = 0, 1, 2, 3
K_IDLE, K_FETCHING, K_READY, K_LAUNCHING, K_USING = range(5)
INT64_MAX = (1 << 63) - 1
FLT_MIN = float(np.finfo(np.float32).tiny)


def f32(v) -> float:
    return float(np.float32(v))


# ----------------------------------------------------------------------------- containers
class MinHeap:
    """src/cpp_worker/utils.hpp:270-357, nodes are [priority, index, data] lists."""

    def __init__(self):
        self.buf = []

    def _swap(self, i, j):
        b = self.buf
        b[i], b[j] = b[j], b[i]
        b[i][1] = i
        b[j][1] = j

    def heapify_down(self, i):
        b = self.buf
        left, right, smallest = 2 * i + 1, 2 * i + 2, i
        if left < len(b) and b[left][0] < b[smallest][0]:
            smallest = left
        if right < len(b) and b[right][0] < b[smallest][0]:
            smallest = right
        if smallest != i:
            self._swap(i, smallest)
            self.heapify_down(smallest)

    def heapify_up(self, i):
        b = self.buf
        while i > 0:
            parent = (i - 1) // 2
            if b[parent][0] > b[i][0]:
                self._swap(parent, i)
                i = parent
            else:
                break

    def rebuild(self):
        for i in range(len(self.buf) // 2, -1, -1):
            self.heapify_down(i)

    def push(self, node):
        node[1] = len(self.buf)
        self.buf.append(node)
        self.heapify_up(len(self.buf) - 1)

    def update_priority(self, node, new_priority):
        old = node[0]
        node[0] = new_priority
        if new_priority < old:
            self.heapify_up(node[1])
        else:
            self.heapify_down(node[1])

    def remove(self, node):
        i = node[1]
        self._swap(i, len(self.buf) - 1)
        self.buf.pop()
        if i < len(self.buf):
            self.heapify_down(i)  # never sifts up: kept as in the reference
        return node

    def front(self):
        return self.buf[0]


# ----------------------------------------------------------------------------- policies
class PolicyBase:
    def select_for_evict(self): raise NotImplementedError
    def evict(self, e): pass
    def access_on_hit(self, e, is_precise): pass
    def access_on_miss(self, e, is_precise): pass
    def update_all_priority(self): pass
    def update_priority(self, e, p): pass
    def set_cur_seq(self, seq): pass


class PolicyFIFO(PolicyBase):
    def __init__(self, cache): self.q = deque()
    def select_for_evict(self): return self.q[0]

    def evict(self, e):
        assert e == self.q[0]
        self.q.popleft()

    def access_on_miss(self, e, is_precise): self.q.append(e)


class PolicyLRU(PolicyBase):
    """List front = victim; hit moves to the back; miss appends (cache.cpp:321-339)."""

    def __init__(self, cache): self.order = []  # small pools: a list is enough
    def select_for_evict(self): return self.order[0]
    def evict(self, e): self.order.remove(e)

    def access_on_hit(self, e, is_precise):
        self.order.remove(e)
        self.order.append(e)

    def access_on_miss(self, e, is_precise):
        assert e not in self.order
        self.order.append(e)


class PolicyStatic(PolicyBase):
    """cache.cpp:340-381: a rotating buffer of n entrants, older ones persist for good."""

    def __init__(self, cache, n):
        self.n, self.alt, self.persisted = n, [], set()

    def select_for_evict(self): return self.alt[0]

    def evict(self, e):
        assert e not in self.persisted
        self.alt.remove(e)

    def access_on_miss(self, e, is_precise):
        if len(self.alt) == self.n:
            self.persisted.add(self.alt.pop(0))
        self.alt.append(e)


class PolicyNN(PolicyBase):
    """cache.hpp:81-126, cache.cpp:383-399."""

    def __init__(self, cache):
        self.cache, self.heap, self.map = cache, MinHeap(), {}

    def select_for_evict(self): return self.heap.front()[2]

    def evict(self, e):
        self.heap.remove(self.map.pop(e))

    def access_on_hit(self, e, is_precise): assert e in self.map

    def access_on_miss(self, e, is_precise):
        assert e not in self.map
        node = [self.cache.priority_get(e), 0, e]
        self.map[e] = node
        self.heap.push(node)

    def update_all_priority(self):
        for e, node in self.map.items():
            node[0] = self.cache.priority_get(e)
        self.heap.rebuild()

    def update_priority(self, e, p): self.heap.update_priority(self.map[e], p)


class PolicyMIN(PolicyBase):
    """cache.hpp:148-224, cache.cpp:490-583. use_times per (seq, expert) end with INT64_MAX."""

    def __init__(self, cache):
        self.cache, self.heap, self.map = cache, MinHeap(), {}
        self.next_idx, self.seq, self.now = {}, None, -1

    def _times(self, e): return self.cache.traces[self.seq][e]
    def select_for_evict(self): return self.heap.front()[2]

    def evict(self, e):
        self.heap.remove(self.map.pop(e))

    def set_cur_seq(self, seq):
        self.seq, self.now = seq, -1
        for k in self.next_idx:
            self.next_idx[k] = 0
        for e, node in self.map.items():
            node[0] = f32(-self._times(e)[0])
        self.heap.rebuild()

    def _advance(self, e):
        t = self._times(e)
        i = self.next_idx.setdefault(e, 0)
        assert i < len(t) and self.now <= t[i]
        self.now = t[i]
        self.next_idx[e] = i + 1

    def access_on_hit(self, e, is_precise):
        self.next_idx.setdefault(e, 0)
        if is_precise:
            self._advance(e)
        self.heap.update_priority(self.map[e], f32(-self._times(e)[self.next_idx[e]]))

    def access_on_miss(self, e, is_precise):
        self.next_idx.setdefault(e, 0)
        if is_precise:
            self._advance(e)
        assert e not in self.map
        node = [f32(-self._times(e)[self.next_idx[e]]), 0, e]
        self.map[e] = node
        self.heap.push(node)


# ----------------------------------------------------------------------------- line planning
def bi_traverse(arr, ret):
    """cache.cpp:9-53."""
    if not arr:
        return
    q = deque([(0, len(arr))])
    while q:
        l, r = q.popleft()
        if l == r:
            continue
        if r - l == 1:
            if not q:
                ret.append(arr[l])
                return
            remaining = list(arr[l:r])
            while q:
                l2, r2 = q.popleft()
                remaining += arr[l2:r2]
            bi_traverse(remaining, ret)
            return
        mid = (l + r) // 2
        ret.append(arr[mid])
        if l < mid:
            q.append((l, mid))
        if mid + 1 < r:
            q.append((mid + 1, r))


def plan_lines(n_pools: int, total: int):
    """cache.cpp:57-94: lines per pool."""
    cand = list(range(n_pools))
    if n_pools > 2:
        order = [0, 1]
        bi_traverse(cand[2:], order)
    else:
        order = cand
    base, rem = divmod(total, n_pools)
    out = [0] * n_pools
    for i in range(n_pools):
        out[order[i]] = base + (1 if i < rem else 0)
    return out


def total_lines(cache_rate: float, num_layer: int, num_expert: int) -> int:
    """prefetcher.cpp:168-174: round(float cache_rate * L * E) in float arithmetic."""
    v = np.float32(np.float32(np.float32(cache_rate) * np.float32(num_layer)) * np.float32(num_expert))
    return int(math.floor(float(v) + 0.5)) if v >= 0 else -int(math.floor(-float(v) + 0.5))


# ----------------------------------------------------------------------------- the schedule
class Expert:
    __slots__ = ("layer", "idx", "line", "num_ready", "status")

    def __init__(self, layer, idx):
        self.layer, self.idx, self.line, self.num_ready, self.status = layer, idx, None, 0, K_IDLE


class SequentialCache:
    """CacheMngr + FetchScheduleWorker under the sequential schedule."""

    def __init__(self, num_layer, num_expert, num_expert_per_token, cache_rate=0.5, cache_policy="lru",
                 num_predict=None, reorder_experts=None, early_preempt=None, chunk_prefetch=None,
                 per_layer_cache=True, promote_hit_in_prefetch=True, num_per_expert_param=3):
        self.L, self.E, self.N = num_layer, num_expert, num_per_expert_param
        self.num_predict = num_expert_per_token if num_predict in (None, -1) else num_predict
        on = self.num_predict > 0  # utils.cpp:93-100
        self.reorder = on if reorder_experts is None else reorder_experts
        self.early_preempt = on if early_preempt is None else early_preempt
        self.chunk_prefetch = on if chunk_prefetch is None else chunk_prefetch
        self.per_layer, self.promote, self.policy_name = per_layer_cache, promote_hit_in_prefetch, cache_policy
        self.experts = [[Expert(l, e) for e in range(num_expert)] for l in range(num_layer)]
        n_pools = num_layer if per_layer_cache else 1
        self.lens = plan_lines(n_pools, total_lines(cache_rate, num_layer, num_expert))
        self.unused = [list(range(n)) for n in self.lens]  # slots in creation order; taken from the back
        self.priority = np.zeros((num_layer, num_expert), np.float32) if cache_policy == "nn" else None
        self.max_priority = np.float32(FLT_MIN)  # cache.hpp:267
        self.traces = {}
        mk = {"fifo": lambda: PolicyFIFO(self), "lru": lambda: PolicyLRU(self),
              "static-1": lambda: PolicyStatic(self, 1), "static-2": lambda: PolicyStatic(self, 2),
              "nn": lambda: PolicyNN(self), "min": lambda: PolicyMIN(self)}[cache_policy]
        self.policies = [mk() for _ in range(n_pools)]
        self.num_predict = min(self.num_predict, self.lens[0])  # cache.cpp:130-131
        self.precise_q, self.layer_q = deque(), [deque() for _ in range(num_layer)]
        self.events = []
        self.counters = dict(hit=0, miss=0, prefetch_hit=0, prefetch_miss=0)

    # -- helpers
    def pool(self, layer): return layer if self.per_layer else 0
    def priority_get(self, e): return float(self.priority[e.layer, e.idx]) if self.priority is not None else 0.0

    def _priority_set(self, e, p):
        if self.priority is not None:
            self.priority[e.layer, e.idx] = p

    def _log(self, kind, e, victim):
        self.counters[("hit", "miss", "prefetch_hit", "prefetch_miss")[kind]] += 1
        self.events.append((kind, e.layer, e.idx, e.line, -1 if victim is None else victim.idx,
                            -1 if victim is None else victim.layer))

    # -- CacheMngr::hit / miss (cache.cpp:236-312)
    def cache_hit(self, e, is_precise):
        pol = self.policies[self.pool(e.layer)]
        pol.access_on_hit(e, is_precise)
        if is_precise:
            self.max_priority = np.float32(self.max_priority + np.float32(1))
            pol.update_priority(e, float(self.max_priority))
            self._priority_set(e, self.max_priority)
        self._log(PRECISE_HIT if is_precise else PREFETCH_HIT, e, None)

    def cache_miss(self, e, is_precise):
        p = self.pool(e.layer)
        pol = self.policies[p]
        if is_precise:
            self.max_priority = np.float32(self.max_priority + np.float32(1))
            self._priority_set(e, self.max_priority)
        victim = None
        if self.unused[p]:
            e.line = self.unused[p].pop()
            pol.access_on_miss(e, is_precise)
        else:
            victim = pol.select_for_evict()
            assert victim is not e
            pol.evict(victim)
            pol.access_on_miss(e, is_precise)
            e.line, victim.line = victim.line, None
            victim.status, victim.num_ready = K_IDLE, 0
        self._log(PRECISE_MISS if is_precise else PREFETCH_MISS, e, victim)

    # -- scheduler (prefetcher.cpp)
    def _reorder(self, layer, ids):
        done, partial, miss = [], [], []
        for i in ids:
            e = self.experts[layer][i]
            if e.line is None:
                miss.append(i)
            elif e.num_ready == self.N:
                done.append(i)
            else:
                partial.append(i)
        ids[:] = done + partial + miss  # no copy is ever "current" between two requests

    def _preempt_layer(self, layer, ids):
        preceding_in_cache = True
        for i in ids:
            e = self.experts[layer][i]
            if e.line is None:
                preceding_in_cache = False
                self.precise_q.append([e, 0, self.N, True])
            elif not preceding_in_cache:
                self.precise_q.append([e, 0, self.N, True])
            elif e.num_ready == self.N:
                e.status = K_LAUNCHING
                self.cache_hit(e, True)
            else:
                self.precise_q.append([e, e.num_ready, self.N, True])

    def _send(self, task):
        e, start, stop, precise = task
        if e.line is None:
            assert start == 0 and e.num_ready == 0
            self.cache_miss(e, precise)
            e.status = K_FETCHING
        else:
            if precise or start == 0:
                self.cache_hit(e, precise)
            if e.num_ready >= stop:
                if precise and e.status == K_READY:
                    e.status = K_LAUNCHING
                return
            start = max(start, e.num_ready)
        # copy [start, stop) is sent and, under the sequential schedule, done (FetchDoneTask)
        e.num_ready = stop
        if stop == self.N:
            e.status = K_LAUNCHING if precise else K_READY

    def _drain(self):
        while True:
            if self.precise_q:
                task = self.precise_q.popleft()
            else:
                for q in self.layer_q:
                    if q:
                        task = q.popleft()
                        break
                else:
                    return
            self._send(task)

    # -- public requests
    def report_layer(self, layer, ids):
        """PrefetchMngr::report_one_layer; returns the (possibly reordered) id list."""
        ids = [int(i) for i in ids]
        if self.reorder:
            self._reorder(layer, ids)
        if self.early_preempt:
            self._preempt_layer(layer, ids)
        self.layer_q[layer].clear()
        self._drain()
        if not self.early_preempt:  # the per-expert hook path: report_one_expert in list order
            for i in ids:
                self.report_expert(layer, i)
        for i in ids:
            self.expert_done(layer, i)
        return ids

    def report_expert(self, layer, i):
        e = self.experts[layer][i]
        if e.line is None:
            self.precise_q.append([e, 0, self.N, True])
        elif e.num_ready == self.N:
            e.status = K_LAUNCHING
            self.cache_hit(e, True)
        else:
            self.precise_q.append([e, e.num_ready, self.N, True])
        self._drain()

    def expert_done(self, layer, i):
        e = self.experts[layer][i]
        if e.status in (K_LAUNCHING, K_USING):
            e.status = K_READY

    def prefetch_layer(self, layer, ids):
        assert not self.layer_q[layer]
        for i in ids:
            e = self.experts[layer][int(i)]
            if self.promote and e.line is not None:
                self.cache_hit(e, False)
            if self.chunk_prefetch:
                for c in range(self.N):
                    self.layer_q[layer].append([e, c, c + 1, False])
            else:
                self.layer_q[layer].append([e, 0, self.N, False])
        self._drain()

    def update_priority(self, prob, start_layer):
        """CacheMngr::update_priority (cache.cpp:400-430,584-591); prob [n_layers, E] float32."""
        prob = np.asarray(prob, np.float32)
        n = prob.shape[0]
        self.priority[start_layer:start_layer + n] = prob
        self.max_priority = np.float32(self.priority.max())
        pools = range(len(self.policies)) if n == self.L else sorted({self.pool(l) for l in range(start_layer, start_layer + n)})
        for p in pools:
            self.policies[p].update_all_priority()

    def set_cur_seq(self, seq):
        for pol in self.policies:
            pol.set_cur_seq(seq)

    def add_use_times(self, seq, layer, expert, times):
        t = [int(v) for v in times]
        if not t or t[-1] != INT64_MAX:
            t.append(INT64_MAX)
        self.traces.setdefault(seq, {})[self.experts[layer][expert]] = t
