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


# ----------------------------------------------------------------------------- checkpoint layouts
# Converters from the two 4-bit checkpoint layouts the reference runs (AutoGPTQ and HQQ experts,
# tests/batch-generate/transformers-app.py:43-45, examples/small-demo-hqq/transformers-app.py:41;
# their buffers are the ones the reference moves with an expert: `qweight|zero|scale`,
# src/sparse_llm_cache/utils/__init__.py:39-46) to the layout above. Both produce, for one linear
# layer with weight [out, in], (packed uint8 [out, in/2], sz float16 [out, in/128, 2]).

def from_gptq(qweight: np.ndarray, qzeros: np.ndarray, scales: np.ndarray, g_idx: np.ndarray | None = None,
              group_size: int = GROUP, zero_offset: int = 1):
    """GPTQ (AutoGPTQ v1 tensors) of one linear layer in -> out:
      qweight int32 [in/8, out]      nibble i of word [r, n] = q[k = 8r + i, n]
      qzeros  int32 [in/g, out/8]    nibble n%8 of word [grp, n/8] = stored zero of (grp, n)
      scales  fp16  [in/g, out]
      g_idx   int32 [in]             group of every k; must be k // g (no activation reordering)
    with w[k, n] = (q[k, n] - (stored zero + zero_offset)) * scale[grp, n]; zero_offset is 1 for the
    v1 serialisation (the zero is stored minus one) and 0 for v2."""
    qweight = np.ascontiguousarray(qweight).view(np.uint32)
    qzeros = np.ascontiguousarray(qzeros).view(np.uint32)
    K, N = qweight.shape[0] * 8, qweight.shape[1]
    if group_size != GROUP:
        raise ValueError(f"only group size {GROUP} has a device kernel (checkpoint uses {group_size})")
    if K % GROUP or scales.shape != (K // GROUP, N) or qzeros.shape != (K // GROUP, N // 8):
        raise ValueError("GPTQ tensor shapes do not describe one [in, out] layer with groups of 128")
    if g_idx is not None and not np.array_equal(np.asarray(g_idx).reshape(-1), np.arange(K) // GROUP):
        raise ValueError("activation-reordered GPTQ checkpoints (g_idx != k // group) are not supported")
    q = np.empty((K, N), np.uint8)
    for i in range(8):
        q[i::8, :] = (qweight >> np.uint32(4 * i)) & np.uint32(0xF)
    z = np.empty((K // GROUP, N), np.uint8)
    for i in range(8):
        z[:, i::8] = (qzeros >> np.uint32(4 * i)) & np.uint32(0xF)
    zero = (z.astype(np.float32) + zero_offset).T.astype(np.float16)          # [out, groups]
    scale = np.asarray(scales, np.float16).T
    return pack(np.ascontiguousarray(q.T), np.ascontiguousarray(scale), np.ascontiguousarray(zero))


def from_hqq(w_q: np.ndarray, scale: np.ndarray, zero: np.ndarray, shape, group_size: int = GROUP, axis: int = 1):
    """HQQ 4-bit tensors of one linear layer with weight `shape` = [out, in], grouped along the input
    dimension (axis 1): the weight is viewed as [out * in / g, g] rows of one group each,
      W_q   uint8 [rows/2, g]   high nibble = row r, low nibble = row r + rows/2
      scale, zero  [rows, 1]    w = (q - zero) * scale, zero a float
    (axis 0 groups run down the output dimension, which the device kernel cannot read)."""
    out_f, in_f = int(shape[0]), int(shape[1])
    if axis != 1:
        raise ValueError("HQQ layers quantised with axis=0 group along the output dimension: re-quantise with axis=1")
    if group_size != GROUP or in_f % GROUP:
        raise ValueError(f"only group size {GROUP} has a device kernel")
    rows = out_f * in_f // GROUP
    w_q = np.ascontiguousarray(w_q, np.uint8).reshape(rows // 2, GROUP)
    q = np.concatenate([(w_q >> 4) & 0xF, w_q & 0xF], axis=0).reshape(out_f, in_f)
    s = np.asarray(scale, np.float32).reshape(out_f, in_f // GROUP).astype(np.float16)
    z = np.asarray(zero, np.float32).reshape(out_f, in_f // GROUP).astype(np.float16)
    return pack(q, s, z)


def adapt_quantised_linear(linear, fmt: str):
    """Rewrites the buffers of one quantised linear module (torch.nn.Module with AutoGPTQ's
    `qweight/qzeros/scales[/g_idx]` or HQQ's `W_q` + `meta`) to this library's layout, in place:
    afterwards it has the buffers `qweight` (uint8 [out, in/2]) and `scale_zero` (float16
    [out, in/128, 2]), which is what inject_model registers, moves and hands to the fused layer."""
    import torch
    if fmt == "gptq":
        packed, sz = from_gptq(linear.qweight.cpu().numpy(), linear.qzeros.cpu().numpy(),
                               linear.scales.cpu().numpy(),
                               linear.g_idx.cpu().numpy() if getattr(linear, "g_idx", None) is not None else None,
                               getattr(linear, "group_size", GROUP))
        for name in ("qzeros", "scales", "g_idx"):
            if name in linear._buffers:
                del linear._buffers[name]
    elif fmt == "hqq":
        meta = linear.meta
        packed, sz = from_hqq(linear.W_q.cpu().numpy(), meta["scale"].float().cpu().numpy(),
                              meta["zero"].float().cpu().numpy(), meta["shape"], meta.get("group_size", GROUP),
                              meta.get("axis", 1))
        for name in ("W_q",):
            linear._buffers.pop(name, None)
            linear._parameters.pop(name, None)
    else:
        raise ValueError(f"unknown quantised layout {fmt!r} (gptq or hqq)")
    linear._buffers["qweight"] = torch.from_numpy(packed)
    linear._buffers["scale_zero"] = torch.from_numpy(sz)
    return linear
