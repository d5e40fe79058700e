"""uint4 group-128 expert weights: quantiser and packer for the layout the device kernels read.

Layout (fixed by this library; the reference leaves it to HQQ / AutoGPTQ):
  * a matrix W [rows, K] (K a multiple of 128) becomes `q` uint8 [rows, K/2] plus `sz` float16
    [rows, K/128, 2] holding {scale, zero} per group of 128 consecutive k;
  * w ~= (q_k - zero) * scale, asymmetric, q in 0..15, zero a float (HQQ style);
  * inside every 32-bit little-endian word of `q` (8 weights k0..k7) the even-k nibbles sit in the
    low half and the odd-k nibbles in the high half: nibble j = q[k0 + 2j], nibble j + 4 =
    q[k0 + 2j + 1] for j = 0..3, so one shift and mask yields a bf16 pair of consecutive k.
"""
from __future__ import annotations

import numpy as np

GROUP = 128


def quantize(w: np.ndarray):
    """W float [rows, K] -> (q uint8 values 0..15 [rows, K], scale f16 [rows, K/128], zero f16)."""
    rows, K = w.shape
    assert K % GROUP == 0
    g = w.astype(np.float32).reshape(rows, K // GROUP, GROUP)
    lo, hi = g.min(axis=2), g.max(axis=2)
    scale = np.maximum((hi - lo) / 15.0, 1e-8).astype(np.float16)
    zero = (-lo / scale.astype(np.float32)).astype(np.float16)
    q = np.clip(np.rint(g / scale.astype(np.float32)[..., None] + zero.astype(np.float32)[..., None]), 0, 15)
    return q.astype(np.uint8).reshape(rows, K), scale, zero


def pack(q: np.ndarray, scale: np.ndarray, zero: np.ndarray):
    """-> (packed uint8 [rows, K/2], sz float16 [rows, K/128, 2]) in the device layout."""
    rows, K = q.shape
    w8 = q.reshape(rows, K // 8, 8).astype(np.uint32)
    word = np.zeros((rows, K // 8), np.uint32)
    for j in range(4):
        word |= w8[:, :, 2 * j] << (4 * j)
        word |= w8[:, :, 2 * j + 1] << (4 * j + 16)
    packed = word.astype("<u4").view(np.uint8).reshape(rows, K // 2)
    sz = np.stack([scale, zero], axis=-1).astype(np.float16)
    return np.ascontiguousarray(packed), np.ascontiguousarray(sz)


def quantize_pack(w: np.ndarray):
    q, s, z = quantize(w)
    return pack(q, s, z)
