"""Times the grouped SwiGLU FFN kernels alone (pm_k_swiglu_ffn): G experts with distinct weights,
`rows` token rows each, so that one launch pair streams G * 3 * inter * hidden * 2 bytes.

    python -m promoe_b200.microbench --groups 60 --rows 4 [--hidden 2048 --inter 1408 --iters 20]

Prints one line with the mean time of a launch pair (CUDA events on the launching stream, after
warm-up) and the achieved weight bandwidth. Weights above 126 MB do not fit in L2, so repeated
launches read them from HBM every time.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import _lib


def run_rotating(groups: int, rows: int, hidden: int, inter: int, iters: int, sets: int, shared_inter: int = 0,
                 slices: int = 1, tokens: int = 8) -> dict:
    """Like run(), but cycles through `sets` disjoint weight sets (as a layer stack does), so that no
    launch finds its weights, or their page translations, warm from the previous launch. With
    shared_inter > 0 every launch also carries a shared expert over all `tokens` rows, whole
    (slices = 1) or cut into `slices` groups along its intermediate dimension, the way a decode
    layer call launches it."""
    _lib.load()
    dev = torch.device("cuda")
    mat = inter * hidden
    x = torch.randn((64, hidden), device=dev).to(torch.bfloat16)
    n_routed = groups * rows
    n_rows = n_routed + (slices * tokens if shared_inter else 0)
    row_token = torch.randint(0, 64, (n_rows,), dtype=torch.int32, device=dev)
    n_groups = groups + (slices if shared_inter else 0)
    nbytes = _lib.call("pm_k_swiglu_ffn_scratch_bytes", n_groups, n_rows, max(inter, shared_inter), hidden)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    yexp = torch.empty((n_rows, hidden), dtype=torch.float32, device=dev)
    plans, keep = [], []
    for _ in range(sets):
        arr = (_lib.pm_ffn_group * n_groups)()
        g0 = 0
        if shared_inter:
            sw = torch.empty(3 * shared_inter * hidden, dtype=torch.bfloat16, device=dev).normal_(0, 0.02)
            keep.append(sw)
            p, smat, width = sw.data_ptr(), shared_inter * hidden, shared_inter // slices
            for j in range(slices):
                arr[j] = _lib.pm_ffn_group(p + j * width * hidden * 2, p + smat * 2 + j * width * hidden * 2,
                                           p + 2 * smat * 2 + j * width * 2, None, None, None,
                                           n_routed + j * tokens, tokens, width, shared_inter)
            g0 = slices
        for i in range(groups):
            w = torch.empty(3 * mat, dtype=torch.bfloat16, device=dev).normal_(0, 0.02)
            keep.append(w)
            p = w.data_ptr()
            arr[g0 + i] = _lib.pm_ffn_group(p, p + mat * 2, p + 2 * mat * 2, None, None, None, i * rows, rows, inter, 0)
        plans.append(arr)
    groups_total = n_groups

    def once(arr):
        _lib.call("pm_k_swiglu_ffn", arr, groups_total, 0, x.data_ptr(), hidden, row_token.data_ptr(), n_rows,
                  yexp.data_ptr(), scratch.data_ptr(), nbytes, None)

    for arr in plans:
        once(arr)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for it in range(iters):
        once(plans[it % sets])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    weight_bytes = (groups * 3 * mat + 3 * shared_inter * hidden) * 2
    return {"groups": groups, "rows": rows, "shared_inter": shared_inter, "slices": slices, "sets": sets,
            "total_gb": sets * weight_bytes / 1e9, "mb_per_launch": weight_bytes / 1e6,
            "us_per_launch": ms * 1e3, "gb_per_s": weight_bytes / ms / 1e6}


def run(groups: int, rows: int, hidden: int, inter: int, iters: int, warmup: int = 3, quant4: bool = False) -> dict:
    _lib.load()
    dev = torch.device("cuda")
    tokens = 64
    x = torch.randn((tokens, hidden), device=dev).to(torch.bfloat16)
    arr = (_lib.pm_ffn_group * groups)()
    mat = inter * hidden
    if quant4:
        # random nibbles and {scale, zero} pairs: timing does not depend on the values
        weights = [torch.randint(0, 256, (3 * mat // 2,), dtype=torch.uint8, device=dev) for _ in range(groups)]
        meta = [torch.full((3 * mat // 128, 2), 0.01, dtype=torch.float16, device=dev) for _ in range(groups)]
        for i, (w, m) in enumerate(zip(weights, meta)):
            p, z = w.data_ptr(), m.data_ptr()
            arr[i] = _lib.pm_ffn_group(p, p + mat // 2, p + mat, z, z + mat // 128 * 4, z + 2 * (mat // 128) * 4,
                                       i * rows, rows, inter, 0)
        weight_bytes = groups * 3 * (mat // 2 + mat // 128 * 4)
    else:
        weights = [(torch.randn(3 * mat, device=dev) * 0.02).to(torch.bfloat16) for _ in range(groups)]
        for i, w in enumerate(weights):
            p = w.data_ptr()
            arr[i] = _lib.pm_ffn_group(p, p + mat * 2, p + 2 * mat * 2, None, None, None, i * rows, rows, inter, 0)
        weight_bytes = groups * 3 * mat * 2
    n_rows = groups * rows
    row_token = torch.randint(0, tokens, (n_rows,), dtype=torch.int32, device=dev)
    nbytes = _lib.call("pm_k_swiglu_ffn_scratch_bytes", groups, n_rows, inter, hidden)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    yexp = torch.empty((n_rows, hidden), dtype=torch.float32, device=dev)

    def once():
        _lib.call("pm_k_swiglu_ffn", arr, groups, int(quant4), x.data_ptr(), hidden, row_token.data_ptr(), n_rows,
                  yexp.data_ptr(), scratch.data_ptr(), nbytes, None)

    for _ in range(warmup):
        once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        once()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    return {"quant4": quant4, "groups": groups, "rows": rows, "hidden": hidden, "inter": inter, "us_per_launch_pair": ms * 1e3,
            "weight_mb": weight_bytes / 1e6, "gb_per_s": weight_bytes / ms / 1e6}


def run_prefill(config: str, tokens: int, iters: int, tc: bool) -> dict:
    """Times one fused layer call of a prefill-size batch (all experts resident) and reports the
    FFN rate: flop = tokens * (k * 6 * H * I + 6 * H * I_shared)."""
    from . import synth
    cfg = synth.CONFIGS[config]
    stack = synth.SyntheticStack(cfg, "cuda", num_layer=1, cache_rate="1.0", num_predict_expert_per_layer=0)
    stack.install_layers()
    cache = stack.cache
    cache.set("tc_prefill", int(tc))
    cache.set("seq_len", tokens)
    x = torch.randn((tokens, cfg.hidden), device="cuda").to(torch.bfloat16)
    y = torch.empty_like(x)
    for _ in range(2):
        cache.forward(0, x, out=y)
    torch.cuda.synchronize()
    cache.set("profile_ffn", 1)
    cache.profile(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        cache.forward(0, x, out=y)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    prof = cache.profile(reset=True)
    flop = tokens * 6.0 * cfg.hidden * (cfg.top_k * cfg.inter + cfg.shared_inter)
    ffn_ms = (prof["gateup_ms"] + prof["down_ms"] + prof["fused_ms"]) / iters
    out = {"config": config, "tokens": tokens, "tensor_core_path": tc, "tc_launches": int(cache.get("tc_launches")),
           "tc_error": cache.get("tc_error"), "layer_ms": ms, "ffn_ms": ffn_ms, "ffn_tflops": flop / ffn_ms / 1e9,
           "layer_tflops": flop / ms / 1e9, "gateup_ms": prof["gateup_ms"] / iters, "down_ms": prof["down_ms"] / iters}
    cache.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--groups", type=int, default=60)
    ap.add_argument("--rows", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=1408)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--quant4", action="store_true", help="uint4 group-128 experts")
    ap.add_argument("--prefill-tokens", type=int, default=0, help="time one prefill-size layer call instead")
    ap.add_argument("--config", default="c5")
    ap.add_argument("--no-tc", action="store_true", help="prefill through the staged mma.sync kernel")
    ap.add_argument("--rotate", type=int, default=0, help="cycle through this many disjoint weight sets")
    ap.add_argument("--shared-inter", type=int, default=0, help="with --rotate: add a shared expert of this width")
    ap.add_argument("--slices", type=int, default=1, help="cut the shared expert into this many groups")
    ap.add_argument("--tokens", type=int, default=8, help="rows of the shared expert")
    a = ap.parse_args()
    if a.prefill_tokens:
        print(json.dumps(run_prefill(a.config, a.prefill_tokens, a.iters, not a.no_tc)))
        return
    if a.rotate > 1:
        print(json.dumps(run_rotating(a.groups, a.rows, a.hidden, a.inter, a.iters, a.rotate, a.shared_inter, a.slices,
                                      a.tokens)))
        return
    print(json.dumps(run(a.groups, a.rows, a.hidden, a.inter, a.iters, a.warmup, a.quant4)))


if __name__ == "__main__":
    main()
