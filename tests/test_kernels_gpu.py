"""GPU parity of the stateless kernels (K1 route, K2 permute, K3a grouped SwiGLU FFN, K4
combine, K5 predictor) against the numpy oracle, called through the C ABI."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import moe_math as om
from promoe_b200 import _lib
from tests.helpers import bf16_weights, dev, dev_bf16, ptr

pytestmark = pytest.mark.gpu

RTOL_BF16 = 2e-2  # layer outputs vs the float64 oracle on the same bf16 inputs


def run_gate(lib, x, wg, bias, k, norm, scale=1.0, shared_gate=None, slots=None):
    T, H = x.shape
    E = wg.shape[0]
    xd, wd = dev_bf16(x), dev_bf16(wg)
    bd = dev(bias.astype(np.float32)) if bias is not None else None
    sg = dev_bf16(shared_gate) if shared_gate is not None else None
    sl = dev(slots.astype(np.int32)) if slots is not None else None
    ids = torch.empty((T, k), dtype=torch.int32, device="cuda")
    w = torch.empty((T, k), dtype=torch.float32, device="cuda")
    ts = torch.empty((T, k), dtype=torch.int32, device="cuda")
    ss = torch.empty((T,), dtype=torch.float32, device="cuda")
    lg = torch.empty((T, E), dtype=torch.float32, device="cuda")
    _lib.call("pm_k_gate_topk", ptr(xd), ptr(wd), ptr(bd), ptr(sg), T, H, E, k, int(norm), scale,
              ptr(sl), ptr(ids), ptr(w), ptr(ts), ptr(ss), ptr(lg), None)
    torch.cuda.synchronize()
    return ids.cpu().numpy(), w.cpu().numpy(), ts.cpu().numpy(), ss.cpu().numpy(), lg.cpu().numpy()


@pytest.mark.parametrize("T,H,E,k,norm", [(1, 64, 4, 2, True), (8, 2048, 60, 4, False),
                                          (32, 2048, 64, 6, False), (16, 4096, 8, 2, True),
                                          (64, 3584, 64, 8, False), (5, 2048, 256, 8, True)])
def test_gate_topk_bit_exact(lib, T, H, E, k, norm):
    rng = np.random.default_rng(1000 + T + E)
    x = om.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    wg = bf16_weights(rng, (E, H))
    bias = (0.5 * np.log(1.0 / np.arange(1, E + 1) ** 1.1)).astype(np.float32)
    sgw = bf16_weights(rng, (H,))
    slots = rng.permutation(E).astype(np.int32) - 3
    ids, w, ts, ss, lg = run_gate(lib, x, wg, bias, k, norm, 1.0, sgw, slots)
    ref_lg = om.gate_logits_canonical(x, wg, bias)
    assert np.array_equal(lg.view(np.uint32), ref_lg.view(np.uint32)), "logits must be bit-exact"
    ref_ids, ref_w = om.route(ref_lg, k, norm)
    assert np.array_equal(ids, ref_ids.astype(np.int32)), "routing ids must be bit-exact"
    # float64 restatement agrees wherever the k-th/(k+1)-th gap is not a rounding coincidence
    lg64 = om.gate_logits(x, wg, bias)
    ids64, w64 = om.route(lg64, k, norm)
    srt = -np.sort(-lg64, axis=1)
    safe = (srt[:, :-1] - srt[:, 1:])[:, :k].min(axis=1) > 1e-4
    assert safe.mean() > 0.9
    assert np.array_equal(ids[safe], ids64[safe].astype(np.int32))
    np.testing.assert_allclose(w[safe], w64[safe], rtol=1e-4, atol=1e-7)
    assert np.array_equal(ts, slots[ids])
    ref_ss = 1.0 / (1.0 + np.exp(-(x.astype(np.float64) @ sgw.astype(np.float64))))
    np.testing.assert_allclose(ss, ref_ss, rtol=1e-4, atol=1e-6)


def test_gate_topk_ties_pick_lower_id(lib):
    T, H, E, k = 3, 64, 8, 3
    x = np.ones((T, H), np.float32)
    wg = np.zeros((E, H), np.float32)
    wg[5] = 0.5  # one clear winner, the rest tie at zero
    ids, w, *_ = run_gate(lib, x, wg, None, k, True)
    assert np.array_equal(ids, np.tile(np.array([5, 0, 1], np.int32), (T, 1)))


def test_gate_topk_rejects_bad_sizes(lib):
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_gate_topk", None, None, None, None, 4, 60, 8, 2, 0, 1.0, None, None, None, None,
                  None, None, None)
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_gate_topk", None, None, None, None, 4, 64, 300, 2, 0, 1.0, None, None, None, None,
                  None, None, None)
    # T == 0 is a no-op
    _lib.call("pm_k_gate_topk", None, None, None, None, 0, 64, 8, 2, 0, 1.0, None, None, None, None,
              None, None, None)


def run_permute(lib, ids, E):
    T, k = ids.shape
    R = T * k
    idd = dev(ids.astype(np.int32))
    counts = torch.empty(E, dtype=torch.int32, device="cuda")
    offsets = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    row_token = torch.full((max(R, 1),), -1, dtype=torch.int32, device="cuda")
    pos = torch.full((max(R, 1),), -1, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.call("pm_k_permute", ptr(idd), R, k, E, ptr(counts), ptr(offsets), ptr(row_token), ptr(pos),
              ptr(err), None)
    torch.cuda.synchronize()
    return (counts.cpu().numpy(), offsets.cpu().numpy(), row_token.cpu().numpy()[:R],
            pos.cpu().numpy()[:R], int(err.item()))


@pytest.mark.parametrize("T,k,E", [(1, 2, 8), (8, 4, 60), (32, 6, 64), (64, 8, 64), (512, 2, 8),
                                   (2048, 6, 64), (3, 8, 256)])
def test_permute_bit_exact(lib, T, k, E):
    rng = np.random.default_rng(7 + T)
    ids = np.stack([rng.choice(E, size=k, replace=False) for _ in range(T)]).astype(np.int32)
    counts, offsets, row_token, pos, err = run_permute(lib, ids, E)
    rc, ro, rt, rp = om.permute(ids, E)
    assert err == 0
    assert np.array_equal(counts, rc) and np.array_equal(offsets, ro)
    assert np.array_equal(row_token, rt) and np.array_equal(pos, rp)


def test_permute_empty_and_bad_id(lib):
    counts, offsets, *_ = run_permute(lib, np.zeros((0, 4), np.int32), 16)
    assert counts.sum() == 0 and offsets[-1] == 0
    ids = np.array([[0, 99], [1, 2]], np.int32)
    counts, offsets, row_token, pos, err = run_permute(lib, ids, 8)
    assert err == 1 and counts.sum() == 3


def ffn_case(rng, H, inters, rows_per_group, T):
    """Random grouped FFN problem: returns weights, groups, row_token."""
    groups, row_token, start = [], [], 0
    for inter, r in zip(inters, rows_per_group):
        wg, wu = bf16_weights(rng, (inter, H)), bf16_weights(rng, (inter, H))
        wd = bf16_weights(rng, (H, inter))
        groups.append((wg, wu, wd, start, r, inter))
        row_token += list(rng.integers(0, T, size=r))
        start += r
    return groups, np.array(row_token, np.int32)


def run_ffn(lib, x, groups, row_token, H):
    xd = dev_bf16(x)
    keep = []
    arr = (_lib.pm_ffn_group * len(groups))()
    for i, (wg, wu, wd, start, r, inter) in enumerate(groups):
        tg, tu, td = dev_bf16(wg), dev_bf16(wu), dev_bf16(wd)
        keep += [tg, tu, td]
        arr[i] = _lib.pm_ffn_group(ptr(tg), ptr(tu), ptr(td), None, None, None, start, r, inter, 0)
    n_rows = int(row_token.shape[0])
    rt = dev(row_token)
    max_inter = max(g[5] for g in groups)
    nbytes = _lib.call("pm_k_swiglu_ffn_scratch_bytes", len(groups), n_rows, max_inter, H)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    yexp = torch.full((n_rows, H), float("nan"), dtype=torch.float32, device="cuda")
    _lib.call("pm_k_swiglu_ffn", arr, len(groups), 0, ptr(xd), H, ptr(rt), n_rows, ptr(yexp),
              ptr(scratch), nbytes, None)
    torch.cuda.synchronize()
    return yexp.cpu().numpy()


@pytest.mark.parametrize("H,inters,rows", [
    (64, [64], [1]),
    (128, [64, 128, 32], [3, 8, 1]),
    (2048, [1408] * 5 + [2816], [1, 2, 8, 5, 3, 16]),
    (2048, [1408, 1408, 5632], [9, 16, 8]),
    (4096, [1024, 1024], [2, 16]),
    (3584, [2560, 2560, 2560], [33, 64, 70]),
    (2048, [1408], [150]),
])
def test_swiglu_ffn_matches_oracle(lib, H, inters, rows):
    rng = np.random.default_rng(42 + H + len(rows))
    T = 16
    x = om.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    groups, row_token = ffn_case(rng, H, inters, rows, T)
    y = run_ffn(lib, x, groups, row_token, H)
    assert np.isfinite(y).all()
    for wg, wu, wd, start, r, inter in groups:
        xr = x[row_token[start:start + r]]
        ref = om.swiglu_mlp(xr, wg, wu, wd, round_h_bf16=True)
        scale = np.abs(ref).max()
        np.testing.assert_allclose(y[start:start + r], ref, rtol=RTOL_BF16, atol=RTOL_BF16 * scale * 0.05)


def test_swiglu_ffn_rejects_bad_sizes(lib):
    arr = (_lib.pm_ffn_group * 1)()
    arr[0] = _lib.pm_ffn_group(8, 8, 8, None, None, None, 0, 1, 48, 0)
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_swiglu_ffn", arr, 1, 0, 8, 64, 8, 1, 8, 8, 1 << 20, None)  # inter % 32 != 0
    arr[0] = _lib.pm_ffn_group(8, 8, 8, None, None, None, 0, 1, 64, 0)
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_swiglu_ffn", arr, 1, 0, 8, 96, 8, 1, 8, 8, 1 << 20, None)  # hidden % 64 != 0
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_swiglu_ffn", arr, 1, 0, 8, 64, 8, 1, 8, 8, 16, None)  # scratch too small
    _lib.call("pm_k_swiglu_ffn", arr, 0, 0, 8, 64, 8, 0, 8, 8, 0, None)  # empty: no-op


@pytest.mark.parametrize("T,H,k,n_shared,gate", [(1, 64, 2, 0, False), (8, 2048, 4, 1, True),
                                                (32, 2048, 6, 1, False), (64, 3584, 8, 1, True)])
def test_combine_matches_oracle(lib, T, H, k, n_shared, gate):
    rng = np.random.default_rng(5 + T)
    R = T * k
    yexp = rng.standard_normal((R + n_shared * T, H)).astype(np.float32)
    pos = rng.permutation(R).astype(np.int32).reshape(T, k)
    w = rng.random((T, k)).astype(np.float32)
    ss = rng.random(T).astype(np.float32) if gate else None
    y = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    yd, pd, wd = dev(yexp), dev(pos), dev(w)
    sd = dev(ss) if gate else None
    _lib.call("pm_k_combine", ptr(yd), ptr(pd), ptr(wd), T, H, k, R, n_shared, ptr(sd), ptr(y), None)
    torch.cuda.synchronize()
    ref = np.einsum("tk,tkh->th", w.astype(np.float64), yexp[pos].astype(np.float64))
    for s in range(n_shared):
        sh = yexp[R + s * T: R + (s + 1) * T].astype(np.float64)
        ref = ref + (sh * ss[:, None] if gate else sh)
    got = y.float().cpu().numpy()
    np.testing.assert_allclose(got, ref, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("B,H,D,E", [(1, 64, 32, 8), (8, 2048, 512, 60), (64, 2048, 512, 64)])
def test_predictor_mlp_matches_oracle(lib, B, H, D, E):
    rng = np.random.default_rng(99 + B)
    x = om.bf16_round(rng.standard_normal((B, H)).astype(np.float32))
    w1, w2 = bf16_weights(rng, (D, H)), bf16_weights(rng, (E, D), 0.05)
    b1 = (rng.standard_normal(D) * 0.1).astype(np.float32)
    b2 = (rng.standard_normal(E) * 0.1).astype(np.float32)
    xd, w1d, w2d, b1d, b2d = dev_bf16(x), dev_bf16(w1), dev_bf16(w2), dev(b1), dev(b2)
    hid = torch.empty((B, D), dtype=torch.float32, device="cuda")
    sc = torch.empty((E,), dtype=torch.float32, device="cuda")
    _lib.call("pm_k_predictor_mlp", ptr(xd), B, H, ptr(w1d), ptr(b1d), D, ptr(w2d), ptr(b2d), E,
              ptr(hid), ptr(sc), None)
    torch.cuda.synchronize()
    ref = om.predictor_scores(x, w1, b1, w2, b2)
    np.testing.assert_allclose(sc.cpu().numpy(), ref, rtol=1e-3, atol=1e-3)
    assert np.array_equal(om.rank_experts(sc.cpu().numpy().astype(np.float64), 4), om.rank_experts(ref, 4))


@pytest.mark.parametrize("width,n", [(60, 4), (64, 6), (8, 8), (480, 12), (1000, 64)])
def test_rank_topn_matches_a_stable_descending_sort(lib, width, n):
    """Device-side ranking of predictor scores: the n best ids, descending score, equal scores in
    ascending id (the scores below repeat values on purpose)."""
    rng = np.random.default_rng(5 + width)
    scores = np.round(rng.standard_normal(width) * 3).astype(np.float32) / 2     # many exact ties
    sd = dev(scores)
    out = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    _lib.call("pm_k_rank_topn", ptr(sd), width, n, ptr(out), None)
    torch.cuda.synchronize()
    want = np.argsort(-scores.astype(np.float64), kind="stable")[:n]
    assert np.array_equal(out.cpu().numpy(), want.astype(np.int32))
    assert np.array_equal(want, om.rank_experts(scores.astype(np.float64), n))
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_rank_topn", ptr(sd), width, width + 1, ptr(out), None)
