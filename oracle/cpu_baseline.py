"""The reference's CPU code path for the MoE block, timed as the baseline. TEST / BENCH
INFRASTRUCTURE ONLY (bench.py's cpu_baseline leg and `--impl reference`).

It is the float32 torch MoE block in the layout the reference actually drives (HF 4.x: a
`gate` linear, a ModuleList of SwiGLU expert modules visited in a Python loop over the ids
that `report_experts` returns, weighted index_add, shared expert; Qwen: sigmoid shared gate)
with the cache bookkeeping of the sequential schedule attached (decisions only: there is no
device to copy to). The reference's own block lives in a transformers fork that is not
available (install.md:23-27), so this restatement, checked against the stock transformers
blocks through oracle/moe_math.py, stands in for it (kind "port").
"""
from __future__ import annotations

import time

import torch

from . import srs_policy as sp


class ExpertMLP(torch.nn.Module):
    def __init__(self, w_gate, w_up, w_down):
        super().__init__()
        self.gate_proj = torch.nn.Linear(w_gate.shape[1], w_gate.shape[0], bias=False)
        self.up_proj = torch.nn.Linear(w_up.shape[1], w_up.shape[0], bias=False)
        self.down_proj = torch.nn.Linear(w_down.shape[1], w_down.shape[0], bias=False)
        with torch.no_grad():
            self.gate_proj.weight.copy_(w_gate)
            self.up_proj.weight.copy_(w_up)
            self.down_proj.weight.copy_(w_down)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class SparseMoeBlock(torch.nn.Module):
    """HF 4.x style block with the report_experts hook point (utils/__init__.py:82-89)."""

    def __init__(self, gate_w, gate_bias, experts, top_k, norm_topk, shared=None, shared_gate_w=None):
        super().__init__()
        self.top_k, self.norm_topk = top_k, norm_topk
        self.gate_w, self.gate_bias = gate_w, gate_bias
        self.experts = torch.nn.ModuleList([ExpertMLP(*w) for w in experts])
        self.shared_expert = ExpertMLP(*shared) if shared is not None else None
        self.shared_gate_w = shared_gate_w
        self.report_experts = lambda ids: ids

    @torch.no_grad()
    def forward(self, x):
        logits = torch.nn.functional.linear(x, self.gate_w)
        if self.gate_bias is not None:
            logits = logits + self.gate_bias
        probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
        w, ids = torch.topk(probs, self.top_k, dim=-1)
        if self.norm_topk:
            w = w / w.sum(dim=-1, keepdim=True)
        expert_list = self.report_experts(torch.unique(ids))
        y = torch.zeros_like(x)
        for e in expert_list.tolist():
            tok, slot = torch.where(ids == e)
            y.index_add_(0, tok, self.experts[e](x[tok]) * w[tok, slot, None])
        if self.shared_expert is not None:
            s = self.shared_expert(x)
            if self.shared_gate_w is not None:
                s = s * torch.sigmoid(x @ self.shared_gate_w)[:, None]
            y = y + s
        return y


def time_stack_sample(blocks, xs, num_layer_total, cache_rate, top_k, num_expert, threads, warmup_steps=1):
    """Runs `blocks` (the first len(blocks) layers of the stack) over the hidden-state stream xs
    [steps, B, H] on the CPU with `threads` threads and returns tokens/s scaled to the whole
    stack: B / (mean seconds per layer-step * num_layer_total)."""
    torch.set_num_threads(threads)
    n_sample = len(blocks)
    cache = sp.SequentialCache(n_sample, num_expert, top_k, cache_rate=cache_rate, num_predict=0)
    for l, blk in enumerate(blocks):
        blk.report_experts = (lambda layer: lambda ids: torch.as_tensor(cache.report_layer(layer, ids.tolist())))(l)
    steps, B = xs.shape[0], xs.shape[1]
    t_total, n_timed = 0.0, 0
    for t in range(steps):
        x = xs[t]
        for blk in blocks:
            t0 = time.perf_counter()
            blk(x)
            dt = time.perf_counter() - t0
            if t >= warmup_steps:
                t_total += dt
                n_timed += 1
    per_layer_step = t_total / max(1, n_timed)
    hits = cache.counters["hit"]
    return {"tokens_per_s": B / (per_layer_step * num_layer_total), "seconds_per_layer_step": per_layer_step,
            "layer_steps_timed": n_timed, "hit_rate": hits / max(1, hits + cache.counters["miss"]),
            "cpu_seconds": t_total}
