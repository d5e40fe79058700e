"""Writes tests/golden/moe_hf_*.npz: inputs, weights and outputs of the stock HuggingFace
transformers 5.5.0 sparse-MoE blocks of this container (Qwen2MoeSparseMoeBlock,
MixtralSparseMoeBlock, DeepseekV2Moe), run in float32 on the CPU at small shapes. The MoE
arithmetic of the reference lives in a transformers fork that is not available, so these
blocks are the nearest executable statement of the same published algorithm; the fixtures pin
oracle/moe_math.py (tests/test_oracle_math.py).

Weights are stored per expert in the HF 4.x layout the reference hooks into
(gate_proj / up_proj [I, H], down_proj [H, I]); the stock 5.x blocks get them copied into
their fused gate_up_proj tensors.

Run from the repository root:  python tests/golden/make_moe_golden.py
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
OUT = Path(__file__).resolve().parent


def bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16-representable float32 tensor -> its uint16 bfloat16 bit patterns (halves the file)."""
    return (t.contiguous().view(torch.int32) >> 16).to(torch.int16).numpy().view(np.uint16)


def rand_expert_weights(g, E, H, I):
    wg = bf16(torch.randn(E, I, H, generator=g) * 0.05)
    wu = bf16(torch.randn(E, I, H, generator=g) * 0.05)
    wd = bf16(torch.randn(E, H, I, generator=g) * 0.05)
    return wg, wu, wd


def fill_experts(experts_module, wg, wu, wd):
    with torch.no_grad():
        experts_module.gate_up_proj.copy_(torch.cat([wg, wu], dim=1))
        experts_module.down_proj.copy_(wd)


def qwen_case(name, T, H, E, k, I, I_sh, norm, seed):
    from transformers.models.qwen2_moe.configuration_qwen2_moe import Qwen2MoeConfig
    from transformers.models.qwen2_moe.modeling_qwen2_moe import Qwen2MoeSparseMoeBlock
    g = torch.Generator().manual_seed(seed)
    cfg = Qwen2MoeConfig(hidden_size=H, num_experts=E, num_experts_per_tok=k, moe_intermediate_size=I,
                         shared_expert_intermediate_size=I_sh, norm_topk_prob=norm, hidden_act="silu")
    blk = Qwen2MoeSparseMoeBlock(cfg).float().eval()
    wg, wu, wd = rand_expert_weights(g, E, H, I)
    gate = bf16(torch.randn(E, H, generator=g) * 0.3)
    sg, su = bf16(torch.randn(I_sh, H, generator=g) * 0.05), bf16(torch.randn(I_sh, H, generator=g) * 0.05)
    sd = bf16(torch.randn(H, I_sh, generator=g) * 0.05)
    sgate = bf16(torch.randn(1, H, generator=g) * 0.2)
    x = bf16(torch.randn(1, T, H, generator=g))
    with torch.no_grad():
        fill_experts(blk.experts, wg, wu, wd)
        blk.gate.weight.copy_(gate)
        blk.shared_expert.gate_proj.weight.copy_(sg)
        blk.shared_expert.up_proj.weight.copy_(su)
        blk.shared_expert.down_proj.weight.copy_(sd)
        blk.shared_expert_gate.weight.copy_(sgate)
        y = blk(x)
        _, rw, ri = blk.gate(x.view(-1, H))
    np.savez_compressed(OUT / f"moe_hf_{name}.npz", family="qwen2_moe", x=x[0].numpy(), gate_w=gate.numpy(),
                        w_gate=bits(wg), w_up=bits(wu), w_down=bits(wd), shared_w_gate=bits(sg),
                        shared_w_up=bits(su), shared_w_down=bits(sd), shared_gate_w=sgate[0].numpy(),
                        top_k=k, norm_topk=int(norm), routed_scale=1.0, y=y[0].numpy(), ids=ri.numpy(),
                        weights=rw.numpy())


def mixtral_case(name, T, H, E, k, I, seed):
    from transformers.models.mixtral.configuration_mixtral import MixtralConfig
    from transformers.models.mixtral.modeling_mixtral import MixtralSparseMoeBlock
    g = torch.Generator().manual_seed(seed)
    cfg = MixtralConfig(hidden_size=H, num_local_experts=E, num_experts_per_tok=k, intermediate_size=I,
                        hidden_act="silu")
    blk = MixtralSparseMoeBlock(cfg).float().eval()
    wg, wu, wd = rand_expert_weights(g, E, H, I)
    gate = bf16(torch.randn(E, H, generator=g) * 0.3)
    x = bf16(torch.randn(1, T, H, generator=g))
    with torch.no_grad():
        fill_experts(blk.experts, wg, wu, wd)
        blk.gate.weight.copy_(gate)
        y = blk(x)
        _, rw, ri = blk.gate(x.view(-1, H))
    np.savez_compressed(OUT / f"moe_hf_{name}.npz", family="mixtral", x=x[0].numpy(), gate_w=gate.numpy(),
                        w_gate=bits(wg), w_up=bits(wu), w_down=bits(wd), top_k=k, norm_topk=1,
                        routed_scale=1.0, y=y[0].numpy(), ids=ri.numpy(), weights=rw.numpy())


def deepseek_case(name, T, H, E, k, I, n_shared, scale, seed):
    from transformers.models.deepseek_v2.configuration_deepseek_v2 import DeepseekV2Config
    from transformers.models.deepseek_v2.modeling_deepseek_v2 import DeepseekV2Moe
    g = torch.Generator().manual_seed(seed)
    cfg = DeepseekV2Config(hidden_size=H, n_routed_experts=E, num_experts_per_tok=k, moe_intermediate_size=I,
                           n_shared_experts=n_shared, routed_scaling_factor=scale, topk_method="greedy",
                           hidden_act="silu", n_group=1, topk_group=1)
    blk = DeepseekV2Moe(cfg).float().eval()
    wg, wu, wd = rand_expert_weights(g, E, H, I)
    gate = bf16(torch.randn(E, H, generator=g) * 0.3)
    I_sh = I * n_shared
    sg, su = bf16(torch.randn(I_sh, H, generator=g) * 0.05), bf16(torch.randn(I_sh, H, generator=g) * 0.05)
    sd = bf16(torch.randn(H, I_sh, generator=g) * 0.05)
    x = bf16(torch.randn(1, T, H, generator=g))
    with torch.no_grad():
        fill_experts(blk.experts, wg, wu, wd)
        blk.gate.weight.copy_(gate)
        blk.shared_experts.gate_proj.weight.copy_(sg)
        blk.shared_experts.up_proj.weight.copy_(su)
        blk.shared_experts.down_proj.weight.copy_(sd)
        y = blk(x)
        logits = torch.nn.functional.linear(x, gate)
        ri, rw = blk.route_tokens_to_experts(logits)
    np.savez_compressed(OUT / f"moe_hf_{name}.npz", family="deepseek_v2", x=x[0].numpy(), gate_w=gate.numpy(),
                        w_gate=bits(wg), w_up=bits(wu), w_down=bits(wd), shared_w_gate=bits(sg),
                        shared_w_up=bits(su), shared_w_down=bits(sd), top_k=k, norm_topk=0,
                        routed_scale=scale, y=y[0].numpy(), ids=ri.numpy(), weights=rw.numpy())


if __name__ == "__main__":
    torch.set_num_threads(4)
    qwen_case("qwen_small", T=6, H=64, E=12, k=4, I=32, I_sh=64, norm=False, seed=1)
    qwen_case("qwen_norm", T=9, H=64, E=10, k=3, I=64, I_sh=32, norm=True, seed=2)
    mixtral_case("mixtral_small", T=7, H=64, E=8, k=2, I=96, seed=3)
    deepseek_case("deepseek_small", T=8, H=64, E=16, k=6, I=32, n_shared=2, scale=1.0, seed=4)
    deepseek_case("deepseek_scaled", T=5, H=64, E=16, k=3, I=32, n_shared=1, scale=2.5, seed=5)
    for p in sorted(OUT.glob("moe_hf_*.npz")):
        print(p.name, f"{p.stat().st_size / 1024:.0f} KiB")
