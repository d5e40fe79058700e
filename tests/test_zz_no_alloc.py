"""pm_k_swiglu_ffn_static: the grouped FFN whose scratch is an array built into the library, for
hosts that cannot allocate device memory when they call it (their own pools own the HBM, or an
allocation's device-wide synchronisation is not acceptable there). Checked against the
caller-scratch entry point on two calls in a row, because the built-in array is shared and keeps
the previous call's bytes. The file name sorts last on purpose: a run that stops at the first
failure has then already executed every other test."""
import numpy as np
import pytest
import torch

from oracle import moe_math as om
from promoe_b200 import _lib
from tests.helpers import bf16_weights, dev, dev_bf16, ptr

pytestmark = pytest.mark.gpu


def build_case(seed, H, inters, rows, T=16):
    rng = np.random.default_rng(seed)
    x = dev_bf16(om.bf16_round(rng.standard_normal((T, H)).astype(np.float32)))
    keep, specs, start, row_token = [x], [], 0, []
    for inter, r in zip(inters, rows):
        w = [dev_bf16(bf16_weights(rng, s)) for s in ((inter, H), (inter, H), (H, inter))]
        keep += w
        specs.append((ptr(w[0]), ptr(w[1]), ptr(w[2]), start, r, inter))
        row_token += list(rng.integers(0, T, size=r))
        start += r
    arr = (_lib.pm_ffn_group * len(specs))()
    for i, (a, b, c, s0, r, inter) in enumerate(specs):
        arr[i] = _lib.pm_ffn_group(a, b, c, None, None, None, s0, r, inter, 0)
    rt = dev(np.array(row_token, np.int32))
    keep.append(rt)
    return x, arr, len(specs), rt, start, max(inters), keep


def run_both(case, H):
    x, arr, n_groups, rt, n_rows, max_inter, _ = case
    nbytes = _lib.call("pm_k_swiglu_ffn_scratch_bytes", n_groups, n_rows, max_inter, H)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    want = torch.full((n_rows, H), float("nan"), dtype=torch.float32, device="cuda")
    got = torch.full((n_rows, H), float("nan"), dtype=torch.float32, device="cuda")
    _lib.call("pm_k_swiglu_ffn", arr, n_groups, 0, ptr(x), H, ptr(rt), n_rows, ptr(want), ptr(scratch), nbytes, None)
    _lib.call("pm_k_swiglu_ffn_static", arr, n_groups, ptr(x), H, ptr(rt), n_rows, ptr(got), None)
    torch.cuda.synchronize()
    return got.cpu().numpy(), want.cpu().numpy()


def test_static_scratch_matches_caller_scratch_twice_in_a_row(lib):
    first = build_case(1, 256, [128, 128, 256], [3, 8, 5])
    second = build_case(2, 128, [64, 192], [16, 40])      # other sizes: stale bytes would show
    for case, H in ((first, 256), (second, 128), (first, 256)):
        got, want = run_both(case, H)
        assert np.isfinite(got).all()
        # same kernels, same inputs: the two entry points agree to the last bit
        np.testing.assert_array_equal(got, want)


def test_static_scratch_rejects_oversize_and_bad_input(lib):
    cap = _lib.call("pm_k_swiglu_ffn_static_capacity")
    assert cap == 8 << 20
    arr = (_lib.pm_ffn_group * 1)()
    # 4096 rows x inter 2048 x 2 bytes = 16 MiB of intermediate rows: more than the array holds
    arr[0] = _lib.pm_ffn_group(8, 8, 8, None, None, None, 0, 4096, 2048, 0)
    with pytest.raises(_lib.PromoeError) as e:
        _lib.call("pm_k_swiglu_ffn_static", arr, 1, 8, 128, 8, 4096, 8, None)
    assert "scratch" in str(e.value)
    arr[0] = _lib.pm_ffn_group(8, 8, 8, None, None, None, 0, 1, 48, 0)
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_swiglu_ffn_static", arr, 1, 8, 128, 8, 1, 8, None)   # inter % 32 != 0
    _lib.call("pm_k_swiglu_ffn_static", arr, 0, 8, 128, 8, 0, 8, None)       # empty launch: no-op


def test_static_scratch_matches_the_oracle_on_a_side_stream(lib):
    """Stands on its own: the built-in-scratch entry point against the float64 oracle, two calls in a
    row on a stream that is not the default one."""
    H, inters, rows, T = 256, [128, 256], [7, 12], 16
    rng = np.random.default_rng(5)
    x = om.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    xd = dev_bf16(x)
    ws, keep, row_token, start = [], [], [], 0
    arr = (_lib.pm_ffn_group * len(inters))()
    for i, (inter, r) in enumerate(zip(inters, rows)):
        w = [bf16_weights(rng, s) for s in ((inter, H), (inter, H), (H, inter))]
        d = [dev_bf16(m) for m in w]
        ws.append(w)
        keep += d
        arr[i] = _lib.pm_ffn_group(ptr(d[0]), ptr(d[1]), ptr(d[2]), None, None, None, start, r, inter, 0)
        row_token += list(rng.integers(0, T, size=r))
        start += r
    rt = dev(np.array(row_token, np.int32))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    for _ in range(2):
        got = torch.full((start, H), float("nan"), dtype=torch.float32, device="cuda")
        with torch.cuda.stream(side):
            _lib.call("pm_k_swiglu_ffn_static", arr, len(inters), ptr(xd), H, ptr(rt), start, ptr(got), side.cuda_stream)
        side.synchronize()
        y, s0 = got.cpu().numpy(), 0
        for w, r in zip(ws, rows):
            ref = om.swiglu_mlp(x[row_token[s0:s0 + r]], *w, round_h_bf16=True)
            np.testing.assert_allclose(y[s0:s0 + r], ref, rtol=2e-2, atol=2e-2 * np.abs(ref).max() * 0.1)
            s0 += r


def test_static_scratch_refuses_a_capturing_stream_and_quantised_groups(lib):
    """Both FFN entry points upload their plan from temporary host memory, which a graph would read
    after it is gone: on a capturing stream they return an error and enqueue nothing."""
    case = build_case(3, 128, [64], [4])
    x, arr, n_groups, rt, n_rows, max_inter, _ = case
    out = torch.zeros((n_rows, 128), dtype=torch.float32, device="cuda")
    nbytes = _lib.call("pm_k_swiglu_ffn_scratch_bytes", n_groups, n_rows, max_inter, 128)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        graph.capture_begin(capture_error_mode="thread_local")
        try:
            with pytest.raises(_lib.PromoeError) as e1:
                _lib.call("pm_k_swiglu_ffn_static", arr, n_groups, ptr(x), 128, ptr(rt), n_rows, ptr(out), side.cuda_stream)
            with pytest.raises(_lib.PromoeError) as e2:
                _lib.call("pm_k_swiglu_ffn", arr, n_groups, 0, ptr(x), 128, ptr(rt), n_rows, ptr(out), ptr(scratch), nbytes,
                          side.cuda_stream)
        finally:
            graph.capture_end()
    assert "capturing" in str(e1.value) and "capturing" in str(e2.value)
    torch.cuda.synchronize()
    # outside the capture the same call works
    _lib.call("pm_k_swiglu_ffn_static", arr, n_groups, ptr(x), 128, ptr(rt), n_rows, ptr(out), None)
    torch.cuda.synchronize()
    assert np.isfinite(out.cpu().numpy()).all()
    q = (_lib.pm_ffn_group * 1)()
    q[0] = _lib.pm_ffn_group(8, 8, 8, 8, 8, 8, 0, 1, 128, 0)
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_swiglu_ffn_static", q, 1, 8, 128, 8, 1, 8, None)
    with pytest.raises(_lib.PromoeError):
        _lib.call("pm_k_swiglu_ffn_static", arr, n_groups, ptr(x), 0, ptr(rt), n_rows, ptr(out), None)
