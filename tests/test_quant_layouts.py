"""Converters from the GPTQ and HQQ 4-bit tensor layouts to the library's uint4 group-128 layout:
the converted tensors, unpacked by the oracle's own unpacker, must give exactly the weights the
oracle's independent GPTQ / HQQ dequantisers give for the original tensors."""
import numpy as np
import pytest

from oracle import quant4 as oq
from promoe_b200 import quant4 as pq


def gptq_tensors(rng, K, N):
    q = rng.integers(0, 16, size=(K, N), dtype=np.uint32)
    z = rng.integers(0, 15, size=(K // 128, N), dtype=np.uint32)       # stored zero: real zero minus one
    qweight = np.zeros((K // 8, N), np.uint32)
    for i in range(8):
        qweight |= q[i::8] << np.uint32(4 * i)
    qzeros = np.zeros((K // 128, N // 8), np.uint32)
    for i in range(8):
        qzeros |= z[:, i::8] << np.uint32(4 * i)
    scales = (rng.random((K // 128, N)) * 0.01 + 0.001).astype(np.float16)
    return qweight.view(np.int32), qzeros.view(np.int32), scales, q, z


def test_gptq_layout_round_trip():
    rng = np.random.default_rng(0)
    K, N = 256, 16
    qweight, qzeros, scales, q, z = gptq_tensors(rng, K, N)
    packed, sz = pq.from_gptq(qweight, qzeros, scales, np.arange(K) // 128)
    assert packed.shape == (N, K // 2) and sz.shape == (N, K // 128, 2)
    want = oq.dequantize_gptq(qweight, qzeros, scales)
    np.testing.assert_array_equal(oq.dequantize(packed, sz), want)
    # and the definition spelled out for one element
    k, n = 131, 5
    assert want[n, k] == np.float32((float(q[k, n]) - (float(z[1, n]) + 1.0))) * np.float32(scales[1, n])
    with pytest.raises(ValueError):
        pq.from_gptq(qweight, qzeros, scales, np.random.default_rng(1).permutation(K) // 128)   # act-order
    with pytest.raises(ValueError):
        pq.from_gptq(qweight, qzeros, scales, None, group_size=64)


def test_hqq_layout_round_trip():
    rng = np.random.default_rng(1)
    out_f, in_f = 24, 256
    rows = out_f * in_f // 128
    q = rng.integers(0, 16, size=(rows, 128), dtype=np.uint8)
    w_q = (q[: rows // 2] << 4) | q[rows // 2:]
    scale = (rng.random((rows, 1)) * 0.01 + 0.001).astype(np.float16).astype(np.float32)
    zero = (rng.random((rows, 1)) * 15).astype(np.float16).astype(np.float32)
    packed, sz = pq.from_hqq(w_q, scale, zero, (out_f, in_f))
    want = oq.dequantize_hqq(w_q, scale, zero, (out_f, in_f))
    np.testing.assert_array_equal(oq.dequantize(packed, sz), want)
    assert want[3, 130] == (np.float32(q[3 * 2 + 1, 2]) - zero[7, 0]) * scale[7, 0]
    with pytest.raises(ValueError):
        pq.from_hqq(w_q, scale, zero, (out_f, in_f), axis=0)


def test_own_quantiser_round_trip():
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((8, 256)) * 0.02).astype(np.float32)
    packed, sz = pq.quantize_pack(w)
    deq = oq.dequantize(packed, sz)
    assert np.abs(deq - w).max() < 0.02 * 6 / 15 * 0.6
