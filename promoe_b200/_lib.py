"""ctypes binding of libpromoe_b200.so (the C ABI declared in include/promoe_b200.h).

There is no fallback: if the library is missing, loading raises. Calls that fail raise
PromoeError carrying pm_last_error().
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libpromoe_b200.so"

PM_OK = 0


class PromoeError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"promoe_b200 error {code}: {msg}")
        self.code = code


class pm_event(C.Structure):
    _fields_ = [("kind", C.c_int32), ("layer", C.c_int32), ("expert", C.c_int32),
                ("slot", C.c_int32), ("evicted", C.c_int32), ("evicted_layer", C.c_int32)]


class pm_stats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "precise_hit", "precise_miss", "prefetch_hit", "prefetch_miss", "ready", "unready",
        "activated_experts", "layer_calls", "h2d_bytes", "h2d_copies", "kernel_launches")]


class pm_profile(C.Structure):
    _fields_ = [("ffn_launches", C.c_int64), ("gateup_ms", C.c_double), ("down_ms", C.c_double),
                ("gateup_bytes", C.c_int64), ("down_bytes", C.c_int64), ("fused_launches", C.c_int64),
                ("fused_ms", C.c_double), ("fused_bytes", C.c_int64), ("resident_launches", C.c_int64),
                ("resident_ms", C.c_double), ("resident_bytes", C.c_int64)]


class pm_layer_weights(C.Structure):
    _fields_ = [("gate_w", C.c_void_p), ("gate_bias", C.c_void_p), ("shared_gate_w", C.c_void_p),
                ("shared_w_gate", C.c_void_p), ("shared_w_up", C.c_void_p), ("shared_w_down", C.c_void_p),
                ("hidden", C.c_int32), ("inter", C.c_int32), ("shared_inter", C.c_int32),
                ("top_k", C.c_int32), ("norm_topk", C.c_int32), ("routed_scale", C.c_float),
                ("quant4", C.c_int32)]


class pm_ffn_group(C.Structure):
    _fields_ = [("w_gate", C.c_void_p), ("w_up", C.c_void_p), ("w_down", C.c_void_p),
                ("q_gate", C.c_void_p), ("q_up", C.c_void_p), ("q_down", C.c_void_p),
                ("row_start", C.c_int32), ("row_count", C.c_int32), ("inter", C.c_int32),
                ("ld_down", C.c_int32)]


_vp, _i, _i64, _u64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_float, C.c_size_t
_cp = C.c_char_p

# name -> (restype, argtypes). Functions returning int are status codes unless listed in _RAW.
SIGNATURES = {
    "pm_version": (_i, []),
    "pm_last_error": (_cp, []),
    "pm_ctx_create": (_i, [C.POINTER(_vp), _i, _i, _cp]),
    "pm_ctx_destroy": (_i, [_vp]),
    "pm_ctx_get": (_i, [_vp, _cp, C.c_char_p, _sz]),
    "pm_ctx_set": (_i, [_vp, _cp, _cp]),
    "pm_ctx_set_param_list": (_i, [_vp, _cp]),
    "pm_register_expert_param": (_i, [_vp, _i, _i, _i, _vp, _sz]),
    "pm_pin_all": (_i, [_vp]),
    "pm_expert_host_ptr": (_i, [_vp, _i, _i, _i, C.POINTER(_vp), C.POINTER(_sz)]),
    "pm_plan_slots": (_i, [_vp, C.POINTER(C.c_int32), _i, C.POINTER(_i)]),
    "pm_build_slab": (_i, [_vp]),
    "pm_build_policy_only": (_i, [_vp]),
    "pm_param_device_ptr": (_i, [_vp, _i, _i, _i, C.POINTER(_vp)]),
    "pm_expert_slot": (_i, [_vp, _i, _i, C.POINTER(C.c_int32)]),
    "pm_report_layer": (_i, [_vp, _i, C.POINTER(_i64), _i64]),
    "pm_prefetch_layer": (_i, [_vp, _i, C.POINTER(_i64), _i64]),
    "pm_report_expert": (_i, [_vp, _i, _i]),
    "pm_expert_done": (_i, [_vp, _i, _i]),
    "pm_layer_done": (_i, [_vp, _i]),
    "pm_expert_acquire": (_i, [_vp, _i, _i, _vp, C.POINTER(_vp)]),
    "pm_expert_release": (_i, [_vp, _i, _i, _vp]),
    "pm_param_offset": (_i, [_vp, _i, C.POINTER(_sz)]),
    "pm_temp_move_expert_to_gpu": (_i, [_vp, _i, _i, _vp, C.POINTER(_vp)]),
    "pm_temp_move_expert_back_to_host": (_i, [_vp, _i, _i, _vp]),
    "pm_set_cur_seq": (_i, [_vp, _u64]),
    "pm_oracle_add_use_times": (_i, [_vp, _u64, _i, _i, C.POINTER(_i64), _i64]),
    "pm_update_priority": (_i, [_vp, C.POINTER(_f), _i, _i]),
    "pm_history_input": (_i, [_vp, C.POINTER(_f), _sz]),
    "pm_event_log_enable": (_i, [_vp, _i]),
    "pm_event_log_read": (_i, [_vp, C.POINTER(pm_event), _sz, C.POINTER(_sz)]),
    "pm_event_log_clear": (_i, [_vp]),
    "pm_stats_read": (_i, [_vp, C.POINTER(pm_stats)]),
    "pm_iter_marks_read": (_i, [_vp, C.POINTER(pm_stats), _sz, C.POINTER(_sz)]),
    "pm_profile_read": (_i, [_vp, C.POINTER(pm_profile), _i]),
    "pm_layer_set_weights": (_i, [_vp, _i, C.POINTER(pm_layer_weights)]),
    "pm_moe_forward": (_i, [_vp, _i, _vp, _i, _vp, _vp]),
    "pm_moe_forward_routed": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "pm_moe_forward_routed_begin": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp,
                                         C.POINTER(C.c_int32), _i, C.POINTER(_i)]),
    "pm_moe_forward_routed_end": (_i, [_vp]),
    "pm_pool_init": (_i, [_vp, _i, _i, _cp]),
    "pm_pool_open_peer": (_i, [_vp, _i, _cp, _i]),
    "pm_pool_exchange": (_i, [_vp, _i64, C.POINTER(C.c_int32), _i, C.POINTER(C.c_int32), C.c_double]),
    "pm_pool_stage": (_i, [_vp, _i, C.POINTER(C.c_int32), _vp, _sz, _sz, C.POINTER(_i64), C.POINTER(_i64), _vp]),
    "pm_pool_scatter": (_i, [_vp, _vp, _vp]),
    "pm_pool_fetch_locally": (_i, [_vp]),
    "pm_moe_forward_host": (_i, [_vp, _i, _vp, _i, _vp, _vp]),
    "pm_last_routing": (_i, [_vp, _i, C.POINTER(C.c_int32), C.POINTER(_f), _i]),
    "pm_predictor_set": (_i, [_vp, _i, _i, _vp, _vp, _i, _vp, _vp]),
    "pm_report_hidden": (_i, [_vp, _i, _vp, _i, _i, _vp]),
    "pm_k_gate_topk": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "pm_k_permute": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "pm_k_gather_rows": (_i, [_vp, _vp, _i, _sz, _vp, _vp]),
    "pm_k_swiglu_ffn_scratch_bytes": (_sz, [_i, _i, _i, _i]),
    "pm_k_swiglu_ffn": (_i, [C.POINTER(pm_ffn_group), _i, _i, _vp, _i, _vp, _i, _vp, _vp, _sz, _vp]),
    "pm_k_swiglu_ffn_static_capacity": (_sz, []),
    "pm_k_swiglu_ffn_static": (_i, [C.POINTER(pm_ffn_group), _i, _vp, _i, _vp, _i, _vp, _vp]),
    "pm_k_ep_pack": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp]),
    "pm_k_ep_unpack": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "pm_k_combine": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "pm_k_predictor_mlp": (_i, [_vp, _i, _i, _vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp]),
    "pm_k_rank_topn": (_i, [_vp, _i, _i, _vp, _vp]),
}
_RAW = {"pm_version", "pm_last_error", "pm_k_swiglu_ffn_scratch_bytes", "pm_k_swiglu_ffn_static_capacity"}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library and attaches signatures; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m promoe_b200.build` "
            "(there is no CPU or PyTorch fallback for this library)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the header and the build disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().pm_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code != PM_OK:
        raise PromoeError(code, last_error())


def call(name: str, *args):
    """Calls a status-returning entry point and raises PromoeError on failure."""
    fn = getattr(load(), name)
    rc = fn(*args)
    if name in _RAW:
        return rc
    check(rc)
    return rc
