"""Attaches the expert cache to a stock HuggingFace transformers 5.x MoE model.

The reference hooks into a transformers 4.x fork whose MoE blocks hold one module per expert
(`...mlp.experts.N`, src/sparse_llm_cache/utils/common_metas.py). Stock transformers 5.x keeps the
experts of a block in two 3-D parameters instead (`experts.gate_up_proj [E, 2I, H]`,
`experts.down_proj [E, H, I]`), so name-pattern injection finds nothing there. This module does the
same job for that layout: every expert's three matrices are sliced out of the fused tensors and
registered with the cache, the fused tensors are released, and the block's forward becomes one call
into the fused device path. Supported blocks: Qwen2-MoE (shared expert with sigmoid gate),
Mixtral (renormalised top-k), DeepSeek-V2 with greedy top-k (shared experts, routed scaling).
"""
from __future__ import annotations

import torch

from .engine import ExpertCache


def find_moe_blocks(model: torch.nn.Module) -> list[tuple[str, torch.nn.Module]]:
    """MoE blocks in forward order: modules that own `experts.gate_up_proj` and a `gate`."""
    out = []
    for name, mod in model.named_modules():
        experts = getattr(mod, "experts", None)
        if experts is not None and hasattr(experts, "gate_up_proj") and hasattr(mod, "gate"):
            out.append((name, mod))
    return out


def _describe(block) -> dict:
    gate = block.gate
    experts = block.experts
    E, two_i, H = experts.gate_up_proj.shape
    top_k = getattr(gate, "top_k", None) or getattr(block, "top_k", None)
    if top_k is None:
        raise ValueError("cannot find top_k on the MoE block")
    kind = type(block).__name__.lower()
    if "mixtral" in kind:
        norm = True
    else:
        norm = bool(getattr(gate, "norm_topk_prob", getattr(block, "norm_topk_prob", False)))
    if getattr(block, "topk_method", "greedy") != "greedy":
        raise ValueError("only greedy top-k routing is supported (group-limited routing is not)")
    return dict(E=E, H=H, I=two_i // 2, top_k=int(top_k), norm_topk=norm,
                routed_scale=float(getattr(block, "routed_scaling_factor", 1.0) or 1.0),
                shared=getattr(block, "shared_expert", None) or getattr(block, "shared_experts", None),
                shared_gate=getattr(block, "shared_expert_gate", None))


def inject_hf_fused_model(model: torch.nn.Module, cache_rate: float = 0.375, cache_policy: str = "lru",
                          num_predict_expert_per_layer: int = 0, device="cuda", **config) -> ExpertCache:
    """Moves every routed expert of `model` into a pinned host record + cache lines and replaces the
    MoE blocks' forwards. The rest of the model is left where it is (move it to `device` yourself).
    Returns the ExpertCache; it is also stored as `model._promoe_cache`."""
    blocks = find_moe_blocks(model)
    if not blocks:
        raise ValueError("no MoE block with fused expert tensors found")
    d0 = _describe(blocks[0][1])
    model_id = getattr(getattr(model, "config", None), "_name_or_path", "") or type(model).__name__
    cache = ExpertCache(len(blocks), d0["E"], num_expert_per_token=d0["top_k"], cache_rate=repr(float(cache_rate)),
                        cache_policy=cache_policy, num_predict_expert_per_layer=num_predict_expert_per_layer,
                        model_arch_string=model_id, **config)
    cache.set_param_list(["gate_proj.weight", "up_proj.weight", "down_proj.weight"])
    descs = []
    for layer, (name, block) in enumerate(blocks):
        d = _describe(block)
        if (d["E"], d["H"], d["I"], d["top_k"]) != (d0["E"], d0["H"], d0["I"], d0["top_k"]):
            raise ValueError(f"MoE block {name} has a different shape than the first one")
        gu = block.experts.gate_up_proj.detach().to("cpu", torch.bfloat16)
        dn = block.experts.down_proj.detach().to("cpu", torch.bfloat16)
        for e in range(d["E"]):
            cache.register_expert(layer, e, [gu[e, : d["I"]].contiguous(), gu[e, d["I"]:].contiguous(), dn[e].contiguous()])
        descs.append(d)
    cache.pin_all()
    cache.build_slab()
    dev = torch.device(device)
    to_dev = lambda t: t.detach().to(dev, torch.bfloat16).contiguous()  # noqa: E731
    for layer, ((name, block), d) in enumerate(zip(blocks, descs)):
        shared = None
        if d["shared"] is not None:
            s = d["shared"]
            shared = [to_dev(s.gate_proj.weight), to_dev(s.up_proj.weight), to_dev(s.down_proj.weight)]
        sgw = to_dev(d["shared_gate"].weight.reshape(-1)) if d["shared_gate"] is not None else None
        cache.set_layer_weights(layer, to_dev(block.gate.weight), d["I"], d["top_k"], d["norm_topk"], d["routed_scale"],
                                shared=shared, shared_gate_w=sgw)
        # the fused tensors are no longer needed: the experts live in the cache now
        block.experts.gate_up_proj = torch.nn.Parameter(torch.empty(0, dtype=torch.bfloat16), requires_grad=False)
        block.experts.down_proj = torch.nn.Parameter(torch.empty(0, dtype=torch.bfloat16), requires_grad=False)
        _replace_forward(block, cache, layer)
    model._promoe_cache = cache
    return cache


def _replace_forward(block, cache: ExpertCache, layer: int):
    block._unfused_forward = block.forward

    def fused_forward(hidden_states, *args, **kwargs):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1])
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        cache.set("seq_len", shape[1] if len(shape) == 3 else 1)
        return cache.forward(layer, x.contiguous()).view(shape).to(hidden_states.dtype)

    block.forward = fused_forward
