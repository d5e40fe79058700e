"""hack_transformers: `from_pretrained` loads on the CPU, injects the cache, moves the rest to the
device the caller named (src/sparse_llm_cache/utils/__init__.py:369-392 in the reference). The CPU
test checks the loader wiring with the injection stubbed out; the GPU test loads a saved tiny
Qwen2-MoE through the patched loader and compares its logits with the plain model."""
import inspect

import pytest
import torch


def tiny_qwen():
    from transformers.models.qwen2_moe.configuration_qwen2_moe import Qwen2MoeConfig
    from transformers.models.qwen2_moe.modeling_qwen2_moe import Qwen2MoeForCausalLM
    cfg = Qwen2MoeConfig(vocab_size=128, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, moe_intermediate_size=64,
                         shared_expert_intermediate_size=128, num_experts=8, num_experts_per_tok=2,
                         decoder_sparse_step=1, max_position_embeddings=64, norm_topk_prob=False)
    torch.manual_seed(0)
    model = Qwen2MoeForCausalLM(cfg).to(torch.bfloat16).eval()
    with torch.no_grad():
        for layer in model.model.layers:
            layer.mlp.gate.weight.mul_(20.0)
    return model


def test_loader_wiring_on_cpu(tmp_path, monkeypatch):
    from transformers.modeling_utils import PreTrainedModel
    from transformers.models.qwen2_moe.modeling_qwen2_moe import Qwen2MoeForCausalLM
    import promoe_b200.utils as U
    model = tiny_qwen()
    model.save_pretrained(tmp_path)
    before_loader = inspect.getattr_static(PreTrainedModel, "_load_pretrained_model")
    before_from = inspect.getattr_static(PreTrainedModel, "from_pretrained")
    seen = []

    def fake_inject(m, device="cuda", **kw):
        # the model is complete (finalised weights) and entirely on the CPU when the injection runs
        assert all(p.device.type == "cpu" for p in m.parameters())
        seen.append((device, kw, m.model.layers[1].mlp.experts.down_proj.detach().clone()))
        m._promoe_fused_layout = True     # nothing to launch

    monkeypatch.setattr(U, "_inject_loaded", fake_inject)
    U.hack_transformers(cache_rate=0.5, cache_policy="lru")
    try:
        U.hack_transformers(cache_rate=0.25)          # a second call changes nothing
        loaded = Qwen2MoeForCausalLM.from_pretrained(tmp_path, device_map={"": "cpu"}, dtype=torch.bfloat16)
        with pytest.raises(AssertionError, match="single device"):
            Qwen2MoeForCausalLM.from_pretrained(tmp_path, dtype=torch.bfloat16)       # no device_map
    finally:
        U.unhack_transformers()
    assert len(seen) == 1
    device, kw, down = seen[0]
    assert device == "cpu" and kw == {"cache_rate": 0.5, "cache_policy": "lru"}
    assert torch.equal(down, model.model.layers[1].mlp.experts.down_proj)
    assert isinstance(loaded, Qwen2MoeForCausalLM)
    assert inspect.getattr_static(PreTrainedModel, "_load_pretrained_model") is before_loader
    assert inspect.getattr_static(PreTrainedModel, "from_pretrained") is before_from
    assert not hasattr(PreTrainedModel, "_old_load_pretrained_model")


@pytest.mark.gpu
def test_from_pretrained_with_the_cache_keeps_the_logits(lib, tmp_path):
    from transformers.models.qwen2_moe.modeling_qwen2_moe import Qwen2MoeForCausalLM
    import promoe_b200.utils as U
    model = tiny_qwen()
    model.save_pretrained(tmp_path)
    U.hack_transformers(cache_rate=0.5, num_predict_expert_per_layer=0)
    try:
        loaded = Qwen2MoeForCausalLM.from_pretrained(tmp_path, device_map={"": "cuda:0"}, dtype=torch.bfloat16)
    finally:
        U.unhack_transformers()
    assert loaded.model.layers[0].mlp.experts.gate_up_proj.numel() == 0        # experts live in the cache
    assert next(loaded.model.embed_tokens.parameters()).device.type == "cuda"
    ref = model.cuda()
    ids = torch.randint(0, 128, (2, 7), device="cuda")
    with torch.no_grad():
        want, got = ref(input_ids=ids).logits.float(), loaded(input_ids=ids).logits.float()
    assert float((got - want).norm() / want.norm()) < 3e-2
    st = loaded._promoe_cache.stats()
    assert st["layer_calls"] == 2 and st["precise_miss"] > 0
    loaded._promoe_cache.close()
