"""Small helpers shared by the GPU parity tests (device memory comes from torch)."""
from __future__ import annotations

import numpy as np
import torch

from oracle import moe_math as om


def bf16_weights(rng: np.random.Generator, shape, std=0.02) -> np.ndarray:
    """float32 array whose values are bf16-representable."""
    return om.bf16_round((rng.standard_normal(shape) * std).astype(np.float32))


def dev_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).cuda()


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


class TinyModel:
    """Random MoE stack in the HF 4.x layout (per-expert gate/up/down matrices), values
    bf16-representable, plus the synthetic AR(1) hidden-state stream of the benchmark."""

    def __init__(self, seed, L, E, H, I, k, shared_I=0, shared_gate=False, norm_topk=False, routed_scale=1.0,
                 zipf_bias=True, w_std=0.02, gate_std=0.02):
        rng = np.random.default_rng(seed)
        self.L, self.E, self.H, self.I, self.k = L, E, H, I, k
        self.shared_I, self.norm_topk, self.routed_scale = shared_I, norm_topk, routed_scale
        self.gate_w = [bf16_weights(rng, (E, H), gate_std) for _ in range(L)]
        self.gate_bias = None
        if zipf_bias:
            self.gate_bias = []
            for _ in range(L):
                p = 1.0 / (rng.permutation(E) + 1.0) ** 1.1
                self.gate_bias.append((0.5 * np.log(p / p.sum())).astype(np.float32))
        self.experts = [[(bf16_weights(rng, (I, H), w_std), bf16_weights(rng, (I, H), w_std),
                          bf16_weights(rng, (H, I), w_std)) for _ in range(E)] for _ in range(L)]
        self.shared = None
        if shared_I:
            self.shared = [(bf16_weights(rng, (shared_I, H), w_std), bf16_weights(rng, (shared_I, H), w_std),
                            bf16_weights(rng, (H, shared_I), w_std)) for _ in range(L)]
        self.shared_gate_w = [bf16_weights(rng, (H,), w_std) for _ in range(L)] if shared_gate else None
        self.rng = rng

    def hidden_stream(self, batch, steps):
        """h_0 ~ N(0,1), h_t = 0.8 h_{t-1} + 0.6 N(0,1), rounded to bf16."""
        h = self.rng.standard_normal((batch, self.H))
        out = []
        for _ in range(steps):
            out.append(om.bf16_round(h.astype(np.float32)))
            h = 0.8 * h + 0.6 * self.rng.standard_normal((batch, self.H))
        return out

    def oracle_forward(self, layer, x, report_experts=None):
        return om.moe_block_forward(
            x, self.gate_w[layer], self.experts[layer], self.k, self.norm_topk, self.routed_scale,
            gate_bias=None if self.gate_bias is None else self.gate_bias[layer],
            shared=None if self.shared is None else self.shared[layer],
            shared_gate_w=None if self.shared_gate_w is None else self.shared_gate_w[layer],
            report_experts=report_experts, round_h_bf16=True)

    def canonical_routing(self, layer, x):
        lg = om.gate_logits_canonical(x, self.gate_w[layer], None if self.gate_bias is None else self.gate_bias[layer])
        return om.route(lg, self.k, self.norm_topk, self.routed_scale)

    def make_cache(self, **config):
        """An ExpertCache holding this model: experts in pinned host records, the rest on the GPU."""
        from promoe_b200.engine import ExpertCache
        cfg = dict(num_expert_per_token=self.k)
        cfg.update(config)
        cache = ExpertCache(self.L, self.E, **cfg)
        cache.set_param_list(["gate_proj.weight", "up_proj.weight", "down_proj.weight"])
        for l in range(self.L):
            for e in range(self.E):
                cache.register_expert(l, e, [om.to_bf16_bits(w) for w in self.experts[l][e]])
        cache.pin_all()
        cache.build_slab()
        for l in range(self.L):
            cache.set_layer_weights(
                l, dev_bf16(self.gate_w[l]), self.I, self.k, self.norm_topk, self.routed_scale,
                gate_bias=None if self.gate_bias is None else dev(self.gate_bias[l]),
                shared=None if self.shared is None else [dev_bf16(w) for w in self.shared[l]],
                shared_gate_w=None if self.shared_gate_w is None else dev_bf16(self.shared_gate_w[l]))
        return cache


class LazyExperts:
    """experts[e] -> (w_gate, w_up, w_down) float32 numpy arrays made on demand from bf16 CPU tensors,
    so that the oracle only ever widens the experts a batch activated."""

    def __init__(self, tensors):
        self.tensors = tensors

    def __len__(self):
        return len(self.tensors)

    def __getitem__(self, e):
        return tuple(t.float().numpy() for t in self.tensors[e])


class ShapeModel(TinyModel):
    """A stack with the dimensions of one of the benchmark configurations. Weights are N(0, 0.02)
    bf16 drawn with torch on the GPU (numpy would need minutes for a 64-expert layer) and kept as
    bf16 CPU tensors; the oracle widens them per expert. Same interface as TinyModel."""

    def __init__(self, seed, L, E, H, I, k, shared_I=0, shared_gate=False, norm_topk=False, routed_scale=1.0,
                 zipf_bias=True, w_std=0.02, gate_std=0.02):
        g = torch.Generator(device="cuda").manual_seed(seed)
        rng = np.random.default_rng(seed)

        def draw(shape, std):
            return (torch.randn(shape, generator=g, device="cuda") * std).to(torch.bfloat16).cpu()

        self.L, self.E, self.H, self.I, self.k = L, E, H, I, k
        self.shared_I, self.norm_topk, self.routed_scale = shared_I, norm_topk, routed_scale
        self.gate_w = [draw((E, H), gate_std).float().numpy() for _ in range(L)]
        self.gate_bias = None
        if zipf_bias:
            self.gate_bias = []
            for _ in range(L):
                p = 1.0 / (rng.permutation(E) + 1.0) ** 1.1
                self.gate_bias.append((0.5 * np.log(p / p.sum())).astype(np.float32))
        self.expert_tensors = [[(draw((I, H), w_std), draw((I, H), w_std), draw((H, I), w_std)) for _ in range(E)]
                               for _ in range(L)]
        self.experts = [LazyExperts(self.expert_tensors[l]) for l in range(L)]
        self.shared = None
        if shared_I:
            self.shared = [tuple(draw(s, w_std).float().numpy() for s in ((shared_I, H), (shared_I, H), (H, shared_I)))
                           for _ in range(L)]
        self.shared_gate_w = [draw((H,), w_std).float().numpy() for _ in range(L)] if shared_gate else None
        self.rng = rng

    def register_experts(self, cache):
        for l in range(self.L):
            for e in range(self.E):
                cache.register_expert(l, e, list(self.expert_tensors[l][e]))

    def make_cache(self, **config):
        from promoe_b200.engine import ExpertCache
        cfg = dict(num_expert_per_token=self.k)
        cfg.update(config)
        cache = ExpertCache(self.L, self.E, **cfg)
        cache.set_param_list(["gate_proj.weight", "up_proj.weight", "down_proj.weight"])
        self.register_experts(cache)
        cache.pin_all()
        cache.build_slab()
        for l in range(self.L):
            cache.set_layer_weights(
                l, dev_bf16(self.gate_w[l]), self.I, self.k, self.norm_topk, self.routed_scale,
                gate_bias=None if self.gate_bias is None else dev(self.gate_bias[l]),
                shared=None if self.shared is None else [dev_bf16(w) for w in self.shared[l]],
                shared_gate_w=None if self.shared_gate_w is None else dev_bf16(self.shared_gate_w[l]))
        return cache
