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
