"""Stock transformers 5.x MoE models (fused expert tensors): inject_hf_fused_model keeps the logits of a
tiny random Qwen2-MoE causal LM, through a prefill and decode steps with a cache smaller than the
set of activated experts, and a Mixtral block keeps its output."""
import copy

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def tiny_qwen():
    from transformers.models.qwen2_moe.configuration_qwen2_moe import Qwen2MoeConfig
    from transformers.models.qwen2_moe.modeling_qwen2_moe import Qwen2MoeForCausalLM
    cfg = Qwen2MoeConfig(vocab_size=128, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, moe_intermediate_size=64,
                         shared_expert_intermediate_size=128, num_experts=8, num_experts_per_tok=2,
                         decoder_sparse_step=1, max_position_embeddings=64, norm_topk_prob=False)
    torch.manual_seed(0)
    model = Qwen2MoeForCausalLM(cfg).to(torch.bfloat16).eval()
    with torch.no_grad():  # spread the router so that top-k is not a coin toss at bf16 resolution
        for layer in model.model.layers:
            layer.mlp.gate.weight.mul_(20.0)
    return model


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm())


def test_qwen2_moe_causal_lm_keeps_its_logits(lib):
    from promoe_b200.hf_fused import find_moe_blocks, inject_hf_fused_model
    model = tiny_qwen()
    ref = copy.deepcopy(model).cuda()
    assert len(find_moe_blocks(model)) == 2
    cache = inject_hf_fused_model(model, cache_rate=0.5, num_predict_expert_per_layer=0)
    model.cuda()
    assert model.model.layers[0].mlp.experts.gate_up_proj.numel() == 0
    ids = torch.randint(0, 128, (2, 9), device="cuda")
    with torch.no_grad():
        want = ref(input_ids=ids).logits
        got = model(input_ids=ids).logits           # prefill: 18 tokens per block call
        assert rel_err(got, want) < 3e-2
        step = torch.randint(0, 128, (2, 1), device="cuda")     # decode-sized call
        want1 = ref(input_ids=step).logits
        got1 = model(input_ids=step).logits
        assert rel_err(got1, want1) < 3e-2
    st = cache.stats()
    assert st["precise_miss"] > 0 and st["layer_calls"] == 4
    assert cache.plan_slots() == [4, 4]
    cache.close()


def test_mixtral_block_keeps_its_output(lib):
    from transformers.models.mixtral.configuration_mixtral import MixtralConfig
    from transformers.models.mixtral.modeling_mixtral import MixtralSparseMoeBlock
    from promoe_b200.hf_fused import inject_hf_fused_model
    torch.manual_seed(1)
    cfg = MixtralConfig(hidden_size=128, num_local_experts=8, num_experts_per_tok=2, intermediate_size=192)

    class Wrapper(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.block = MixtralSparseMoeBlock(cfg)

    w = Wrapper().to(torch.bfloat16).eval()
    with torch.no_grad():
        w.block.experts.gate_up_proj.normal_(0, 0.05)
        w.block.experts.down_proj.normal_(0, 0.05)
        w.block.gate.weight.normal_(0, 0.5)
    ref = copy.deepcopy(w).cuda()
    cache = inject_hf_fused_model(w, cache_rate=0.5)
    w.cuda()
    x = torch.randn(1, 7, 128, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        assert rel_err(w.block(x), ref.block(x)) < 3e-2
    cache.close()
