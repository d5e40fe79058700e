"""The MoE-block replacement: swaps the forward of an HF 4.x style sparse MoE module for one call
into the fused B200 path (route -> permute -> cache bookkeeping and copies -> grouped SwiGLU
FFN by cache slot -> combine).

The reference ships this piece as a patch to the transformers modelling files (its fork:
install.md:23-27), whose forward computes the routing, calls `self.report_experts(ids)`
(src/sparse_llm_cache/utils/__init__.py:82-89) and loops over the expert modules. Here the
module keeps its structure (`gate`, `experts`, shared expert children, so the name patterns of
utils/common_metas.py still match) and only `forward` changes.
"""
from __future__ import annotations

import torch


def _first(module, names):
    for n in names:
        child = getattr(module, n, None)
        if child is not None:
            return child
    return None


def _bf16_dev(t: torch.Tensor, device) -> torch.Tensor:
    return t.detach().to(device=device, dtype=torch.bfloat16).contiguous()


def describe_block(block: torch.nn.Module, config=None) -> dict:
    """Extracts what the fused layer needs from an HF 4.x style MoE block:
    Qwen2-MoE (`gate`, `experts[i].{gate,up,down}_proj`, `shared_expert`, `shared_expert_gate`),
    DeepSeek-MoE / V2 (`gate.weight`, `shared_experts`, routed_scaling_factor),
    Mixtral (`gate`, `experts[i].{w1,w3,w2}`, top-k renormalised)."""
    gate = block.gate
    gate_w = gate.weight
    first = block.experts[0]
    mixtral = hasattr(first, "w1")
    proj = first.w1 if mixtral else first.gate_proj
    # uint4 experts in this library's layout (promoe_b200.quant4.adapt_quantised_linear): packed rows
    quant4 = getattr(proj, "qweight", None) is not None and getattr(proj, "scale_zero", None) is not None
    inter = proj.qweight.shape[0] if quant4 else proj.weight.shape[0]
    method = getattr(gate, "topk_method", getattr(block, "topk_method", "greedy"))
    if method not in (None, "greedy"):
        raise ValueError(f"the fused router selects the k largest probabilities (greedy); this block uses {method!r}")
    shared = _first(block, ("shared_expert", "shared_experts"))
    shared_gate = getattr(block, "shared_expert_gate", None)
    cfg = config if config is not None else getattr(block, "config", None)
    top_k = (getattr(block, "top_k", None) or getattr(gate, "top_k", None)
             or getattr(cfg, "num_experts_per_tok", None))
    if top_k is None:
        raise ValueError("cannot find the number of experts per token on the block or its config")
    if mixtral:
        norm = True
    else:
        norm = bool(getattr(block, "norm_topk_prob", getattr(gate, "norm_topk_prob", getattr(cfg, "norm_topk_prob", False))))
    scale = float(getattr(block, "routed_scaling_factor", getattr(gate, "routed_scaling_factor", 1.0)) or 1.0)
    return dict(gate_w=gate_w, inter=inter, top_k=int(top_k), norm_topk=norm, routed_scale=scale,
                shared=shared, shared_gate=shared_gate, quant4=quant4)


def install_fused_forward(block: torch.nn.Module, cache, layer_id: int, device="cuda", config=None,
                          returns_router_logits: bool = False):
    """Uploads the block's resident weights (router, shared expert) and replaces `block.forward`.
    `cache` is the promoe_b200.engine.ExpertCache that already holds the block's experts."""
    d = describe_block(block, config)
    dev = torch.device(device)
    shared = None
    if d["shared"] is not None:
        s = d["shared"]
        shared = [_bf16_dev(s.gate_proj.weight, dev), _bf16_dev(s.up_proj.weight, dev), _bf16_dev(s.down_proj.weight, dev)]
    sgw = None
    if d["shared_gate"] is not None:
        sgw = _bf16_dev(d["shared_gate"].weight.reshape(-1), dev)
    cache.set_layer_weights(layer_id, _bf16_dev(d["gate_w"], dev), d["inter"], d["top_k"], d["norm_topk"],
                            d["routed_scale"], shared=shared, shared_gate_w=sgw, quant4=d["quant4"])
    block._promoe_layer_id = layer_id
    block._promoe_cache = cache
    if not hasattr(block, "_unfused_forward"):
        block._unfused_forward = block.forward

    def fused_forward(hidden_states, *args, **kwargs):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1])
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        x = x.contiguous()
        cache.set("seq_len", shape[1] if len(shape) == 3 else 1)
        y = cache.forward(layer_id, x).view(shape).to(hidden_states.dtype)
        return (y, None) if returns_router_logits else y

    block.forward = fused_forward
    return block
