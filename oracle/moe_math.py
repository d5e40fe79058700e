"""CPU oracle for the MoE block arithmetic. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference leg may
import this module, and only as the checker; the product path never calls it.

What it restates. The reference (huwf5/promoe) does not contain the MoE block arithmetic: it
lives in a private fork of HuggingFace transformers plus patched trust_remote_code model files
(install.md:23-27, README.md:13-14), cloned without a pinned version (the only hints are
`transformers>=4.40.1,<5.0.0`, docker/requirements.txt:9, and the TGI 2.2.0 base image,
docker/Dockerfile.transformers:2). The reference touches that code only through
`module.report_experts(experts)` (src/sparse_llm_cache/utils/__init__.py:82-89), the per-expert
module hooks (src/sparse_llm_cache/utils/hooks.py:187-198) and the zero-sized stand-in model
eval/demo-simulate/transformers-deepseek-moe.py:27-88. This file therefore restates the
PUBLISHED algorithm of the HF 4.x sparse MoE blocks the fork patches (Qwen2MoeSparseMoeBlock,
MixtralSparseMoeBlock, DeepseekMoE): gate linear -> softmax in float32 -> top-k -> optional
renormalisation -> unique expert list -> report_experts -> loop over experts, SwiGLU MLP each
-> weighted index_add -> + shared expert (Qwen: scaled by sigmoid(shared_expert_gate . x)).

Pinning. The reference has no test or golden vector at this boundary, so parity with the
reference itself is UNPINNED. The restatement is pinned instead against the stock
transformers 5.5.0 blocks of this container (tests/golden/make_moe_golden.py writes
tests/golden/moe_hf_*.npz; tests/test_oracle_math.py replays them).
"""
from __future__ import annotations

import numpy as np


# ----------------------------------------------------------------------------- bf16 helpers
def bf16_round(a: np.ndarray) -> np.ndarray:
    """Rounds float32 values to the nearest bfloat16 (ties to even); returns float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(a), a, out).reshape(a.shape)


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> uint16 bfloat16 bit patterns (round to nearest even)."""
    return (bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ----------------------------------------------------------------------------- routing
def gate_logits(x: np.ndarray, w_gate: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    """Router logits in float64 (x [T,H], w_gate [E,H]); the plain restatement of `gate(x)`."""
    out = x.astype(np.float64) @ w_gate.astype(np.float64).T
    if bias is not None:
        out = out + bias.astype(np.float64)
    return out


def gate_logits_canonical(x: np.ndarray, w_gate: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    """Router logits in float32 with the exact summation order the device router documents.

    The hidden dimension is cut into 8-element vectors; lane j of 32 accumulates the vectors
    v with v % 32 == j in ascending v, elements in order, acc = acc + w*x (products of
    bf16-representable values are exact in float32); lanes are merged by a butterfly over
    lane ^ 16, 8, 4, 2, 1. Inputs must already be bf16-representable float32.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w_gate, dtype=np.float32)
    T, H = x.shape
    E = w.shape[0]
    assert H % 8 == 0
    nvec = H // 8
    rounds = (nvec + 31) // 32
    pad = rounds * 32 * 8 - H
    if pad:
        x = np.concatenate([x, np.zeros((T, pad), np.float32)], axis=1)
        w = np.concatenate([w, np.zeros((E, pad), np.float32)], axis=1)
    xr = x.reshape(T, 1, rounds, 32, 8)
    wr = w.reshape(1, E, rounds, 32, 8)
    acc = np.zeros((T, E, 32), np.float32)
    for r in range(rounds):
        # A padded (absent) vector adds exact zeros, which leaves acc unchanged bit for bit.
        for i in range(8):
            prod = (xr[:, :, r, :, i] * wr[:, :, r, :, i]).astype(np.float32)
            acc = (acc + prod).astype(np.float32)
    lanes = np.arange(32)
    for m in (16, 8, 4, 2, 1):
        acc = (acc + acc[:, :, lanes ^ m]).astype(np.float32)
    out = acc[:, :, 0]
    if bias is not None:
        out = (out + bias.astype(np.float32)[None, :]).astype(np.float32)
    return out


def topk_desc(scores: np.ndarray, k: int) -> np.ndarray:
    """Indices of the k largest entries per row, descending, ties -> lower index."""
    order = np.argsort(-scores, axis=-1, kind="stable")
    return order[:, :k].astype(np.int64)


def route(logits: np.ndarray, k: int, norm_topk: bool, routed_scale: float = 1.0):
    """softmax(float) -> top-k -> optional renormalisation. Returns (ids [T,k], weights [T,k]).

    Selection is made on the logits: softmax is strictly monotonic, so this equals top-k over
    the probabilities whenever the probabilities are distinct.
    """
    lg = logits.astype(np.float64)
    p = np.exp(lg - lg.max(axis=-1, keepdims=True))
    p = p / p.sum(axis=-1, keepdims=True)
    ids = topk_desc(logits, k)
    w = np.take_along_axis(p, ids, axis=-1)
    if norm_topk:
        w = w / (w.sum(axis=-1, keepdims=True) + 1e-20)
    return ids, (w * routed_scale)


def unique_sorted_experts(topk_ids: np.ndarray) -> np.ndarray:
    """The id list handed to report_experts: ascending unique ids (int64)."""
    return np.unique(topk_ids.reshape(-1)).astype(np.int64)


def permute(topk_ids: np.ndarray, num_expert: int):
    """Expert-sorted row order, stable in t*k + j. Returns counts, offsets, row_token, pos."""
    flat = topk_ids.reshape(-1)
    k = topk_ids.shape[1]
    counts = np.bincount(flat, minlength=num_expert).astype(np.int32)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    order = np.argsort(flat, kind="stable")
    row_token = (order // k).astype(np.int32)
    pos = np.empty(flat.shape[0], np.int32)
    pos[order] = np.arange(flat.shape[0], dtype=np.int32)
    return counts, offsets, row_token, pos


# ----------------------------------------------------------------------------- expert FFN
def silu(v: np.ndarray) -> np.ndarray:
    return v / (1.0 + np.exp(-v))


def swiglu_mlp(x: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray,
               round_h_bf16: bool = False) -> np.ndarray:
    """down(silu(gate(x)) * up(x)) with [out, in] weight matrices, float64 accumulation."""
    xd = x.astype(np.float64)
    h = silu(xd @ w_gate.astype(np.float64).T) * (xd @ w_up.astype(np.float64).T)
    if round_h_bf16:
        h = bf16_round(h.astype(np.float32)).astype(np.float64)
    return h @ w_down.astype(np.float64).T


def moe_block_forward(x, gate_w, experts, top_k, norm_topk, routed_scale=1.0, gate_bias=None,
                      shared=None, shared_gate_w=None, report_experts=None, round_h_bf16=False):
    """One MoE block forward in the HF 4.x layout.

    x [T,H]; gate_w [E,H]; experts: sequence of (w_gate [I,H], w_up [I,H], w_down [H,I]);
    shared: optional (w_gate, w_up, w_down); shared_gate_w: optional [H] (sigmoid gate).
    report_experts: optional callable(int64 array) -> int64 array (may reorder), the hook point
    of src/sparse_llm_cache/utils/__init__.py:82-89. Returns (y [T,H] float64, ids, weights).
    """
    T, H = x.shape
    logits = gate_logits(x, gate_w, gate_bias)
    ids, w = route(logits, top_k, norm_topk, routed_scale)
    expert_list = unique_sorted_experts(ids)
    if report_experts is not None:
        expert_list = report_experts(expert_list)
    y = np.zeros((T, H), np.float64)
    for e in expert_list:
        tok, slot = np.nonzero(ids == e)
        if tok.size == 0:
            continue
        wg, wu, wd = experts[int(e)]
        out = swiglu_mlp(x[tok], wg, wu, wd, round_h_bf16)
        np.add.at(y, tok, out * w[tok, slot][:, None])
    if shared is not None:
        s = swiglu_mlp(x, shared[0], shared[1], shared[2], round_h_bf16)
        if shared_gate_w is not None:
            gate = 1.0 / (1.0 + np.exp(-(x.astype(np.float64) @ shared_gate_w.astype(np.float64))))
            s = s * gate[:, None]
        y = y + s
    return y, ids, w


# ----------------------------------------------------------------------------- predictor
def predictor_scores(x, w1, b1, w2, b2):
    """sum over the batch of W2 relu(W1 x + b1) + b2 (src/cpp_worker/predictor.cpp:596-605)."""
    xd = x.astype(np.float64)
    h = np.maximum(xd @ w1.astype(np.float64).T + (0 if b1 is None else b1.astype(np.float64)), 0.0)
    out = h @ w2.astype(np.float64).T + (0 if b2 is None else b2.astype(np.float64))
    return out.sum(axis=0)


def rank_experts(scores: np.ndarray, n: int) -> np.ndarray:
    """Descending sort, first n (src/cpp_worker/predictor.hpp:24-28); ties -> lower id."""
    n = min(n, scores.shape[-1])
    return np.argsort(-scores, kind="stable")[:n].astype(np.int64)


# ----------------------------------------------------------------------------- large batches
def routing_consistent(x, gate_w, gate_bias, ids, top_k, gap=1e-4) -> bool:
    """True when `ids` (descending order, selected on the float32 canonical logits) is a valid
    top-k of the float64 logits up to `gap`: no expert left out beats a chosen one by more than
    `gap`, and the chosen ones are in non-increasing order up to `gap`. (Where two float64 logits
    lie closer than float32 resolves, either order is a correct selection.)"""
    lg = gate_logits(x, gate_w, gate_bias)
    chosen = np.take_along_axis(lg, ids, axis=1)
    masked = lg.copy()
    np.put_along_axis(masked, ids, -np.inf, axis=1)
    if (masked.max(axis=1) - chosen.min(axis=1) > gap).any():
        return False
    return not ((chosen[:, 1:] - chosen[:, :-1]) > gap).any()


def moe_block_forward_f32(x, ids, w, experts, shared=None, shared_gate_w=None, expert_order=None):
    """The same block for prefill-size batches with the routing given: float32 torch matmuls on the
    host cores, grouped per expert, intermediate rows rounded to bf16 as the device stores them.
    (float64 numpy needs minutes for 8192 tokens x 64 experts; the tolerance of the parity tests,
    rtol 2e-2, is four orders of magnitude above float32 rounding.) Returns y [T, H] float32."""
    import torch
    T, H = x.shape
    xt = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32))
    y = torch.zeros((T, H), dtype=torch.float32)
    wt = torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32))
    idt = torch.from_numpy(np.ascontiguousarray(ids, dtype=np.int64))

    def mlp(rows, wg, wu, wd):
        g = rows @ torch.from_numpy(wg).T
        h = torch.nn.functional.silu(g) * (rows @ torch.from_numpy(wu).T)
        return h.to(torch.bfloat16).float() @ torch.from_numpy(wd).T

    order = unique_sorted_experts(ids) if expert_order is None else expert_order
    for e in order:
        tok, slot = torch.nonzero(idt == int(e), as_tuple=True)
        if tok.numel() == 0:
            continue
        out = mlp(xt[tok], *experts[int(e)])
        y.index_add_(0, tok, out * wt[tok, slot][:, None])
    if shared is not None:
        s = mlp(xt, *shared)
        if shared_gate_w is not None:
            s = s * torch.sigmoid(xt @ torch.from_numpy(np.ascontiguousarray(shared_gate_w, dtype=np.float32)))[:, None]
        y += s
    return y.numpy()
