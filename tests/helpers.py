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
