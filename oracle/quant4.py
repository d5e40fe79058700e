"""CPU oracle for the uint4 group-128 weight format. TEST INFRASTRUCTURE ONLY.

The reference does not define a 4-bit layout (it defers to HQQ / AutoGPTQ, which are absent:
examples/small-demo-hqq/transformers-app.py:41, tests/batch-generate/transformers-app.py:43-45), so
there is no reference vector to pin against: this file restates the format documented in
promoe_b200/quant4.py independently (unpacking from the packed bytes) and the parity tests feed
the SAME dequantised weights to the float64 MoE oracle (tolerance rtol 3e-2)."""
from __future__ import annotations

import numpy as np


def dequantize(packed: np.ndarray, sz: np.ndarray) -> np.ndarray:
    """packed uint8 [rows, K/2], sz float16 [rows, K/128, 2] -> float32 [rows, K] = (q - zero) * scale."""
    rows = packed.shape[0]
    K = packed.shape[1] * 2
    words = np.ascontiguousarray(packed).view("<u4").reshape(rows, K // 8).astype(np.uint64)
    q = np.empty((rows, K // 8, 8), np.float32)
    for k in range(8):
        shift = 4 * (k // 2) + (16 if k % 2 else 0)   # even k: low half nibble k/2, odd k: high half
        q[:, :, k] = ((words >> shift) & 0xF).astype(np.float32)
    q = q.reshape(rows, K // 128, 128)
    scale = sz[:, :, 0].astype(np.float32)[..., None]
    zero = sz[:, :, 1].astype(np.float32)[..., None]
    return ((q - zero) * scale).reshape(rows, K)
