"""Synthetic MoE stacks with the shapes of the benchmark configurations.

Weights are N(0, 0.02) from a seed per (config, layer, tensor); the gate bias is
0.5*ln(p_e) with p_e proportional to rank^-1.1 over a seeded permutation (Zipf-skewed expert
popularity); hidden states follow h_0 ~ N(0,1), h_t = 0.8 h_{t-1} + 0.6 N(0,1) per sequence
(temporal expert reuse) and every layer of a stack is fed the same h_t. These stand in for
the chat-prompt sets and checkpoints the reference's sweeps use, which need a network.
Tensors are generated on the GPU and the experts copied straight into the cache's pinned
host records.
"""
from __future__ import annotations

import ctypes as C
import hashlib
from dataclasses import dataclass

import numpy as np
import torch

from .engine import ExpertCache

MASTER_SEED = 20240812


@dataclass(frozen=True)
class StackConfig:
    name: str
    num_layer: int
    num_expert: int
    top_k: int
    hidden: int
    inter: int
    shared_inter: int
    shared_gate: bool
    norm_topk: bool
    batch: int
    steps: int
    cache_rate: float
    predictor_width: int = 0   # 0 = no predictor
    model_id: str = ""
    quant4: bool = False       # routed experts stored as uint4 group-128 (scale/zero fp16)


CONFIGS = {
    # BASELINE.json configs[0]: one DeepSeek-MoE-16B-shaped layer
    "c1": StackConfig("deepseek-moe-16b-layer", 1, 64, 6, 2048, 1408, 2816, False, False, 32, 64, 0.375,
                      model_id="deepseek-ai/deepseek-moe-16b-chat"),
    # configs[1]: Qwen1.5-MoE-A2.7B-shaped 24-layer stack with the next-layer predictor
    "c2": StackConfig("qwen1.5-moe-a2.7b-stack", 24, 60, 4, 2048, 1408, 5632, True, False, 8, 128, 0.375,
                      predictor_width=512, model_id="Qwen/Qwen1.5-MoE-A2.7B-Chat"),
    # configs[2]: Mixtral-8x7B-shaped 32-layer stack with uint4 group-128 experts
    "c3": StackConfig("mixtral-8x7b-int4-stack", 32, 8, 2, 4096, 14336, 0, False, True, 16, 128, 0.5,
                      model_id="mistralai/Mixtral-8x7B-Instruct-v0.1", quant4=True),
    # configs[3]: Qwen2-57B-A14B-shaped 28-layer stack (expert parallel over 2/4/8 GPUs)
    "c4": StackConfig("qwen2-57b-a14b-stack", 28, 64, 8, 3584, 2560, 20480, True, False, 64, 64, 0.375,
                      model_id="Qwen/Qwen2-57B-A14B-Instruct"),
    # configs[4]: DeepSeek-V2-Lite-shaped 26 layers
    "c5": StackConfig("deepseek-v2-lite-stack", 26, 64, 6, 2048, 1408, 2816, False, False, 4, 256, 0.375,
                      model_id="deepseek-ai/DeepSeek-V2-Lite-Chat"),
}


def seed_for(*parts) -> int:
    h = hashlib.sha256(("/".join(str(p) for p in (MASTER_SEED,) + parts)).encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 62) - 1)


def _randn(shape, seed, device, std=0.02, dtype=torch.bfloat16):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(dtype)


def zipf_gate_bias(num_expert: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    p = 1.0 / (rng.permutation(num_expert) + 1.0) ** 1.1
    return (0.5 * np.log(p / p.sum())).astype(np.float32)


def hidden_stream(cfg: StackConfig, steps: int, batch: int, device, seed_tag="hidden") -> torch.Tensor:
    """[steps, batch, hidden] bf16: the AR(1) process, one chain per sequence."""
    g = torch.Generator(device=device).manual_seed(seed_for(cfg.name, seed_tag))
    out = torch.empty((steps, batch, cfg.hidden), dtype=torch.bfloat16, device=device)
    h = torch.randn((batch, cfg.hidden), generator=g, device=device)
    for t in range(steps):
        out[t] = h.to(torch.bfloat16)
        h = 0.8 * h + 0.6 * torch.randn((batch, cfg.hidden), generator=g, device=device)
    return out


def _host_tensor(addr: int, nbytes: int) -> torch.Tensor:
    """A CPU int16 tensor aliasing `nbytes` at `addr` (the cache's pinned record)."""
    buf = (C.c_int16 * (nbytes // 2)).from_address(addr)
    return torch.from_numpy(np.ctypeslib.as_array(buf))


def quantize_pack_torch(w: torch.Tensor):
    """Same quantiser and packing as promoe_b200.quant4.quantize_pack, on whatever device `w` lives:
    returns (int32 words [rows, K/8], float16 {scale, zero} [rows, K/128, 2])."""
    rows, K = w.shape
    g = w.float().view(rows, K // 128, 128)
    lo, hi = g.amin(dim=2), g.amax(dim=2)
    scale = ((hi - lo) / 15.0).clamp_min(1e-8).to(torch.float16)
    zero = (-lo / scale.float()).to(torch.float16)
    q = torch.clamp(torch.round(g / scale.float()[..., None] + zero.float()[..., None]), 0, 15).to(torch.int64)
    q8 = q.view(rows, K // 8, 8)
    word = torch.zeros((rows, K // 8), dtype=torch.int64, device=w.device)
    for j in range(4):
        word |= q8[:, :, 2 * j] << (4 * j)
        word |= q8[:, :, 2 * j + 1] << (4 * j + 16)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)  # same bits, signed container
    return word, torch.stack([scale, zero], dim=-1).contiguous()


class SyntheticStack:
    """Builds the cache, the pinned expert records and the resident weights of one config."""

    def __init__(self, cfg: StackConfig, device="cuda", num_layer: int | None = None, expert_range=None,
                 shared_arena: str | None = None, **cache_config):
        self.cfg = cfg
        self.device = torch.device(device)
        L = cfg.num_layer if num_layer is None else num_layer
        self.num_layer = L
        # expert_range = (first, count): this rank's contiguous block of experts (expert parallel)
        self.e0, self.n_local = expert_range if expert_range else (0, cfg.num_expert)
        conf = dict(num_expert_per_token=cfg.top_k, cache_rate=repr(cfg.cache_rate), model_arch_string=cfg.model_id)
        conf.update(cache_config)
        self.cache = ExpertCache(L, self.n_local, **conf)
        H, I = cfg.hidden, cfg.inter
        if cfg.quant4:
            self.cache.set_param_list(["w1.qweight", "w1.scale_zero", "w3.qweight", "w3.scale_zero",
                                       "w2.qweight", "w2.scale_zero"])
            sizes = [I * H // 2, I * H // 128 * 4] * 3
        else:
            self.cache.set_param_list(["gate_proj.weight", "up_proj.weight", "down_proj.weight"])
            sizes = [I * H * 2, I * H * 2, H * I * 2]
        for l in range(L):
            for e in range(self.n_local):
                self.cache.register_expert_sizes(l, e, sizes)
        if shared_arena:  # records in POSIX shared memory, so the other ranks of the node can pull them too
            self.cache.set("shared_arena", shared_arena)
        self.cache.pin_all()
        self.gate_w, self.gate_bias, self.shared, self.shared_gate_w = [], [], [], []
        for l in range(L):
            for e in range(self.n_local):
                if cfg.quant4:
                    self._fill_quant4_expert(l, e)
                    continue
                for p, (name, shape) in enumerate((("gate", (I, H)), ("up", (I, H)), ("down", (H, I)))):
                    w = _randn(shape, seed_for(cfg.name, l, self.e0 + e, name), self.device)
                    addr, n = self.cache.host_record(l, e, p)
                    _host_tensor(addr, n).copy_(w.view(torch.int16).reshape(-1))
            self.gate_w.append(_randn((cfg.num_expert, H), seed_for(cfg.name, l, "router"), self.device))
            self.gate_bias.append(torch.from_numpy(zipf_gate_bias(cfg.num_expert, seed_for(cfg.name, l, "bias"))).to(self.device))
            if cfg.shared_inter:
                Is = cfg.shared_inter
                self.shared.append((_randn((Is, H), seed_for(cfg.name, l, "shared_gate_proj"), self.device),
                                    _randn((Is, H), seed_for(cfg.name, l, "shared_up_proj"), self.device),
                                    _randn((H, Is), seed_for(cfg.name, l, "shared_down_proj"), self.device)))
            self.shared_gate_w.append(_randn((H,), seed_for(cfg.name, l, "shared_expert_gate"), self.device)
                                      if cfg.shared_gate else None)
        self.cache.build_slab()
        self.predictors = {}

    def _fill_quant4_expert(self, l: int, e: int):
        """uint4 experts of the synthetic stack: N(0, 0.02) masters quantised on the GPU and packed in the
        layout of promoe_b200/quant4.py, written straight into the pinned record."""
        cfg = self.cfg
        for m, (name, shape) in enumerate((("gate", (cfg.inter, cfg.hidden)), ("up", (cfg.inter, cfg.hidden)),
                                           ("down", (cfg.hidden, cfg.inter)))):
            w = _randn(shape, seed_for(cfg.name, l, self.e0 + e, name), self.device, dtype=torch.float32)
            word, sz = quantize_pack_torch(w)
            addr, n = self.cache.host_record(l, e, 2 * m)
            _host_tensor(addr, n).copy_(word.view(torch.int16).reshape(-1))
            addr, n = self.cache.host_record(l, e, 2 * m + 1)
            _host_tensor(addr, n).copy_(sz.view(torch.int16).reshape(-1))

    def install_layers(self):
        """Full-width routing on this GPU (single-GPU use: local experts == all experts)."""
        cfg = self.cfg
        for l in range(self.num_layer):
            self.cache.set_layer_weights(l, self.gate_w[l], cfg.inter, cfg.top_k, cfg.norm_topk, 1.0,
                                         gate_bias=self.gate_bias[l],
                                         shared=self.shared[l] if cfg.shared_inter else None,
                                         shared_gate_w=self.shared_gate_w[l], quant4=cfg.quant4)

    def install_routed_only(self):
        """Expert-parallel rank: the cache serves rows routed elsewhere (no router in the context)."""
        cfg = self.cfg
        for l in range(self.num_layer):
            self.cache.set_layer_weights(l, None, cfg.inter, 1, False, 1.0, hidden=cfg.hidden)

    def ep_layers(self):
        """Per-layer resident weights for promoe_b200.ep.CudaBackend (router over ALL experts)."""
        cfg = self.cfg
        return [dict(gate_w=self.gate_w[l], gate_bias=self.gate_bias[l],
                     shared=self.shared[l] if cfg.shared_inter else None, shared_gate_w=self.shared_gate_w[l],
                     top_k=cfg.top_k, norm_topk=cfg.norm_topk, routed_scale=1.0, inter=cfg.inter)
                for l in range(self.num_layer)]

    def make_predictors(self):
        """Random-initialised MLPs hidden -> width -> num_expert (ReLU, over ALL experts) for every
        (source, target) pair of the reference's default prediction window (predictor.cpp:8-46).
        Returns (dict (src, dst) -> (w1, b1, w2, b2), list of (first, last + 1) per source index)."""
        cfg = self.cfg
        if not cfg.predictor_width:
            return {}, []
        L, W, E = self.num_layer, cfg.predictor_width, cfg.num_expert
        mapping = predict_layer_mapping(L, window0=int(self.cache.get("limit_layer_0_window")))
        for src, (a, b) in enumerate(mapping):
            for dst in range(a, b):
                if (src, dst) in self.predictors:
                    continue
                w1 = _randn((W, cfg.hidden), seed_for(cfg.name, "pred", src, dst, "w1"), self.device)
                w2 = _randn((E, W), seed_for(cfg.name, "pred", src, dst, "w2"), self.device)
                b1 = torch.zeros(W, device=self.device)
                b2 = torch.zeros(E, device=self.device)
                self.predictors[(src, dst)] = (w1, b1, w2, b2)
        return self.predictors, mapping

    def install_predictors(self):
        """Single-GPU use: the predictors run inside the context's own forward."""
        for (src, dst), (w1, b1, w2, b2) in self.make_predictors()[0].items():
            self.cache.set_predictor(src, dst, w1, b1, w2, b2)

    def host_expert(self, layer: int, expert: int):
        """The bf16 tensors of one expert as float32 CPU tensors (for the CPU baseline)."""
        cfg = self.cfg
        out = []
        for p, shape in enumerate(((cfg.inter, cfg.hidden), (cfg.inter, cfg.hidden), (cfg.hidden, cfg.inter))):
            addr, n = self.cache.host_record(layer, expert, p)
            out.append(_host_tensor(addr, n).view(torch.bfloat16).reshape(shape).float())
        return out


def predict_layer_mapping(num_layer: int, interval: int = 1, window: int = 3, window0: int = 1):
    """(first, last+1) of the layers each source index predicts (predictor.cpp:8-46)."""
    stops = [0] * (num_layer + 1)
    stop = 0
    for l in range(0, num_layer, interval):
        w = window0 if l == 0 else window
        stops[l] = stop
        stops[l + 1] = min(l + w, num_layer)
        stop = stops[l + 1]
    for l in range(1, num_layer + 1):
        stops[l] = max(stops[l], stops[l - 1])
    return [(stops[l], stops[l + 1]) for l in range(num_layer)]
