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


# Independent dequantisers of the two checkpoint layouts the converters in promoe_b200/quant4.py
# accept. They restate the published tensor formats of AutoGPTQ (v1 serialisation) and HQQ
# (4-bit, `pack_4bit_u8`, axis 1); neither library is present, so parity is against these
# restatements, not against the libraries themselves.

def dequantize_gptq(qweight: np.ndarray, qzeros: np.ndarray, scales: np.ndarray, zero_offset: int = 1) -> np.ndarray:
    """-> float32 weight in nn.Linear layout [out, in]: w[n, k] = (q[k, n] - (z[g, n] + off)) * s[g, n]."""
    qw = np.ascontiguousarray(qweight).view(np.uint32).astype(np.uint64)
    qz = np.ascontiguousarray(qzeros).view(np.uint32).astype(np.uint64)
    K, N = qw.shape[0] * 8, qw.shape[1]
    w = np.empty((N, K), np.float32)
    for k in range(K):
        q = ((qw[k // 8] >> (4 * (k % 8))) & 0xF).astype(np.float32)                       # [N]
        g = k // 128
        z = np.array([(int(qz[g, n // 8]) >> (4 * (n % 8))) & 0xF for n in range(N)], np.float32) if k % 128 == 0 else z
        w[:, k] = (q - (z + zero_offset)) * scales[g].astype(np.float32)
    return w


def dequantize_hqq(w_q: np.ndarray, scale: np.ndarray, zero: np.ndarray, shape) -> np.ndarray:
    """-> float32 [out, in]: rows of 128 consecutive weights, first half of the rows in the high nibbles."""
    out_f, in_f = shape
    rows = out_f * in_f // 128
    b = np.ascontiguousarray(w_q, np.uint8).reshape(rows // 2, 128)
    q = np.empty((rows, 128), np.float32)
    q[: rows // 2] = b >> 4
    q[rows // 2:] = b & 0xF
    s = np.asarray(scale, np.float32).reshape(rows, 1).astype(np.float16).astype(np.float32)
    z = np.asarray(zero, np.float32).reshape(rows, 1).astype(np.float16).astype(np.float32)
    return ((q - z) * s).reshape(out_f, in_f)
