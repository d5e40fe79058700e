"""Per-model metadata: number of MoE layers, experts per layer, experts per token and the
name patterns that locate experts, MoE blocks, attention blocks and decoder layers
(counterpart of the reference's src/sparse_llm_cache/utils/common_metas.py:9-190; same model
ids, same numbers, same patterns, so a model prepared for the reference is found the same way).
"""
from __future__ import annotations

import re
from dataclasses import asdict, dataclass
from typing import Callable

from .filter import RegexFilter


@dataclass
class ModelMetas:
    num_moe_layer: int
    num_expert_per_layer: int
    num_expert_per_token: int
    expert_meta_parser: Callable
    expert_name_filter: Callable
    moe_attn_name_filter: Callable
    moe_mlp_name_filter: Callable
    moe_layer_name_filter: Callable


def _parser(layer_offset: int, block: str):
    """(moe layer id, expert id) from a module name; either is None when the name has no such part."""
    layer_re = re.compile(r".*layers\.(\d+).*")
    expert_re = re.compile(r".*layers\.\d+\." + block + r"experts\.(\d+).*$")

    def parse(name: str):
        lm, em = layer_re.match(name), expert_re.match(name)
        return (int(lm.group(1)) - layer_offset if lm else None, int(em.group(1)) if em else None)

    return parse


def _build(layers, experts, top_k, block="mlp", first_moe_layer=0, all_layers_pattern=r"(\d+)"):
    moe_idx = r"([1-9]\d*)" if first_moe_layer == 1 else all_layers_pattern
    b = re.escape(block)
    return ModelMetas(
        num_moe_layer=layers, num_expert_per_layer=experts, num_expert_per_token=top_k,
        expert_meta_parser=_parser(first_moe_layer, b + r"\."),
        expert_name_filter=RegexFilter(r".*layers\.(\d+)\." + b + r"\.experts\.(\d+)$"),
        moe_attn_name_filter=RegexFilter(r".*layers\." + moe_idx + r"\.self_attn$"),
        moe_mlp_name_filter=RegexFilter(r".*layers\." + moe_idx + r"\." + b + "$"),
        moe_layer_name_filter=RegexFilter(r".*layers\." + moe_idx + "$"))


def _simulate():
    # the zero-sized stand-in model of eval/demo-simulate: experts hang directly off the layer
    m = _build(27, 64, 6)
    m.expert_meta_parser = _parser(0, "")
    m.expert_name_filter = RegexFilter(r".*layers\.(\d+)\.experts\.(\d+)$")
    m.moe_attn_name_filter = RegexFilter(r".*layers\.([1-9]\d*)\.self_attn$")
    m.moe_mlp_name_filter = RegexFilter(r".*layers\.(\d+).mlp$")
    return m


predefined_metas = {
    "deepseek-ai/deepseek-moe-16b-chat": lambda: _build(27, 64, 6, first_moe_layer=1),
    "deepseek-ai/deepseek-moe-16b-chat-simulate": _simulate,
    "deepseek-ai/DeepSeek-V2-Lite-Chat": lambda: _build(26, 64, 6, first_moe_layer=1),
    "Qwen/Qwen1.5-MoE-A2.7B-Chat": lambda: _build(24, 60, 4),
    "Qwen/Qwen2-57B-A14B-Instruct": lambda: _build(28, 64, 8),
    "Qwen/Qwen2-57B-A14B-Instruct-GPTQ-Int4": lambda: _build(28, 64, 8),
    "mistralai/Mixtral-8x7B-Instruct-v0.1": lambda: _build(32, 8, 2, block="block_sparse_moe"),
    "TheBloke/Mixtral-8x7B-Instruct-v0.1-GPTQ": lambda: _build(32, 8, 2, block="block_sparse_moe"),
}


def auto_infer_model_metas(model_id: str, return_dict: bool = True):
    if model_id not in predefined_metas:
        raise ValueError(f"model {model_id} is not supported")
    metas = predefined_metas[model_id]()
    return asdict(metas) if return_dict else metas
