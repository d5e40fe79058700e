"""Python handle on one pm_ctx: the expert cache plus the fused MoE layer forward.

This is plumbing over the C ABI (include/promoe_b200.h): torch is used for device memory and
streams only. `promoe_b200.cpp_worker` re-exposes the same context under the reference's
class names for `sparse_llm_cache`-style callers.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np
import torch

from . import _lib

EVENT_KINDS = ("precise_hit", "precise_miss", "prefetch_hit", "prefetch_miss")


def _config_text(cfg: dict) -> bytes:
    return "\n".join(f"{k}={v}" for k, v in cfg.items()).encode()


def _host_view(t) -> tuple[int, int, object]:
    """(address, nbytes, keep-alive) of a host tensor / array."""
    if isinstance(t, torch.Tensor):
        if t.device.type != "cpu":
            raise ValueError("expert tensors are registered from host memory")
        t = t.contiguous()
        return t.data_ptr(), t.numel() * t.element_size(), t
    a = np.ascontiguousarray(t)
    return a.ctypes.data, a.nbytes, a


class ExpertCache:
    """Owns a pm_ctx. Every failing call raises promoe_b200._lib.PromoeError."""

    def __init__(self, num_layer: int, num_expert: int, **config):
        _lib.load()
        self.num_layer, self.num_expert = num_layer, num_expert
        self._ctx = C.c_void_p()
        _lib.call("pm_ctx_create", C.byref(self._ctx), num_layer, num_expert, _config_text(config))
        self._keep: list = []          # device tensors whose addresses the context holds
        self._hidden = 0
        self._n_params = 0
        self.pinned = False

    # ------------------------------------------------------------------ lifecycle
    def close(self):
        if self._ctx:
            _lib.call("pm_ctx_destroy", self._ctx)
            self._ctx = C.c_void_p()
            self._keep.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self) -> C.c_void_p:
        return self._ctx

    # ------------------------------------------------------------------ configuration
    def get(self, key: str) -> str:
        buf = C.create_string_buffer(256)
        _lib.call("pm_ctx_get", self._ctx, key.encode(), buf, 256)
        return buf.value.decode()

    def set(self, key: str, value) -> None:
        _lib.call("pm_ctx_set", self._ctx, key.encode(), str(value).encode())

    def set_param_list(self, names: Sequence[str]) -> None:
        self._n_params = len(names)
        _lib.call("pm_ctx_set_param_list", self._ctx, "\n".join(names).encode())

    # ------------------------------------------------------------------ experts and slab
    def register_expert(self, layer: int, expert: int, tensors: Sequence) -> None:
        """Registers the host tensors of one expert, in set_param_list order."""
        for pid, t in enumerate(tensors):
            addr, nbytes, keep = _host_view(t)
            self._keep.append(keep)
            _lib.call("pm_register_expert_param", self._ctx, layer, expert, pid, addr, nbytes)

    def register_expert_sizes(self, layer: int, expert: int, nbytes: Sequence[int]) -> None:
        """Declares tensor sizes only; the caller fills the pinned record through host_record()."""
        for pid, n in enumerate(nbytes):
            _lib.call("pm_register_expert_param", self._ctx, layer, expert, pid, None, int(n))

    def pin_all(self) -> None:
        _lib.call("pm_pin_all", self._ctx)
        self.pinned = True
        self._keep = [k for k in self._keep if isinstance(k, torch.Tensor) and k.is_cuda]

    def host_record(self, layer: int, expert: int, param: int) -> tuple[int, int]:
        p, n = C.c_void_p(), C.c_size_t()
        _lib.call("pm_expert_host_ptr", self._ctx, layer, expert, param, C.byref(p), C.byref(n))
        return p.value, n.value

    def plan_slots(self) -> list[int]:
        n = C.c_int()
        _lib.call("pm_plan_slots", self._ctx, None, 0, C.byref(n))
        lens = (C.c_int32 * n.value)()
        _lib.call("pm_plan_slots", self._ctx, lens, n.value, C.byref(n))
        return list(lens)

    def build_slab(self) -> None:
        _lib.call("pm_build_slab", self._ctx)

    def build_policy_only(self) -> None:
        _lib.call("pm_build_policy_only", self._ctx)

    def expert_slot(self, layer: int, expert: int) -> int:
        s = C.c_int32()
        _lib.call("pm_expert_slot", self._ctx, layer, expert, C.byref(s))
        return s.value

    def expert_acquire(self, layer: int, expert: int, stream: int) -> int:
        """report_one_expert + wait_expert for a caller that runs the expert itself on `stream`:
        returns the device address of the expert's cache line (tensor i at + param_offset(i))."""
        p = C.c_void_p()
        _lib.call("pm_expert_acquire", self._ctx, layer, expert, stream, C.byref(p))
        return p.value

    def expert_release(self, layer: int, expert: int, stream: int) -> None:
        _lib.call("pm_expert_release", self._ctx, layer, expert, stream)

    def param_offset(self, param: int) -> int:
        n = C.c_size_t()
        _lib.call("pm_param_offset", self._ctx, param, C.byref(n))
        return n.value

    def temp_move_expert_to_gpu(self, layer: int, expert: int, stream: int) -> int:
        p = C.c_void_p()
        _lib.call("pm_temp_move_expert_to_gpu", self._ctx, layer, expert, stream, C.byref(p))
        return p.value

    def temp_move_expert_back_to_host(self, layer: int, expert: int, stream: int) -> None:
        _lib.call("pm_temp_move_expert_back_to_host", self._ctx, layer, expert, stream)

    def expert_range_tensor(self) -> torch.Tensor:
        """stable_va=1: the experts' own address ranges ([L * E] x line_stride bytes) as one uint8 CUDA
        tensor. Only the ranges of resident experts are mapped; touching another part faults."""
        base = int(self.get("expert_va_base"))
        nbytes = int(self.get("line_stride")) * self.num_layer * self.num_expert

        class _Raw:
            __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (base, False), "version": 3}
        return torch.as_tensor(_Raw(), device=torch.device("cuda", torch.cuda.current_device()))

    def slab_tensor(self) -> torch.Tensor:
        """The whole slab (policy lines + the spare line) as one uint8 CUDA tensor that aliases it."""
        base, nbytes = int(self.get("slab_base")), int(self.get("slab_bytes"))

        class _Raw:
            __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (base, False), "version": 3}
        return torch.as_tensor(_Raw(), device=torch.device("cuda", torch.cuda.current_device()))

    def param_device_ptr(self, layer: int, expert: int, param: int) -> int | None:
        p = C.c_void_p()
        _lib.call("pm_param_device_ptr", self._ctx, layer, expert, param, C.byref(p))
        return p.value

    # ------------------------------------------------------------------ policy requests
    def report_layer(self, layer: int, ids: Sequence[int]) -> list[int]:
        arr = (C.c_int64 * len(ids))(*[int(i) for i in ids])
        _lib.call("pm_report_layer", self._ctx, layer, arr, len(ids))
        return list(arr)

    def prefetch_layer(self, layer: int, ids: Sequence[int]) -> None:
        arr = (C.c_int64 * len(ids))(*[int(i) for i in ids])
        _lib.call("pm_prefetch_layer", self._ctx, layer, arr, len(ids))

    def report_expert(self, layer: int, expert: int) -> None:
        _lib.call("pm_report_expert", self._ctx, layer, expert)

    def expert_done(self, layer: int, expert: int) -> None:
        _lib.call("pm_expert_done", self._ctx, layer, expert)

    def layer_done(self, layer: int) -> None:
        _lib.call("pm_layer_done", self._ctx, layer)

    def set_cur_seq(self, seq: int) -> None:
        _lib.call("pm_set_cur_seq", self._ctx, seq)

    def add_use_times(self, seq: int, layer: int, expert: int, times: Sequence[int]) -> None:
        arr = (C.c_int64 * len(times))(*[int(t) for t in times])
        _lib.call("pm_oracle_add_use_times", self._ctx, seq, layer, expert, arr, len(times))

    def update_priority(self, prob: np.ndarray, start_layer: int) -> None:
        p = np.ascontiguousarray(prob, np.float32).reshape(-1, self.num_expert)
        _lib.call("pm_update_priority", self._ctx, p.ctypes.data_as(C.POINTER(C.c_float)), p.shape[0], start_layer)

    def history_input(self) -> np.ndarray:
        """[num_layer, num_expert] float32: the history-based predictor input (see pm_history_input)."""
        out = np.zeros((self.num_layer, self.num_expert), np.float32)
        _lib.call("pm_history_input", self._ctx, out.ctypes.data_as(C.POINTER(C.c_float)), out.size)
        return out

    def enable_event_log(self, on: bool = True) -> None:
        _lib.call("pm_event_log_enable", self._ctx, int(on))

    def events(self, clear: bool = False) -> list[tuple]:
        n = C.c_size_t()
        _lib.call("pm_event_log_read", self._ctx, None, 0, C.byref(n))
        evs = (_lib.pm_event * max(1, n.value))()
        _lib.call("pm_event_log_read", self._ctx, evs, n.value, C.byref(n))
        out = [(e.kind, e.layer, e.expert, e.slot, e.evicted, e.evicted_layer) for e in evs[: n.value]]
        if clear:
            _lib.call("pm_event_log_clear", self._ctx)
        return out

    def stats(self) -> dict:
        s = _lib.pm_stats()
        _lib.call("pm_stats_read", self._ctx, C.byref(s))
        return {name: getattr(s, name) for name, _ in s._fields_}

    def iter_marks(self) -> list[dict]:
        """Counters at the end of every model iteration (see pm_iter_marks_read)."""
        n = C.c_size_t()
        _lib.call("pm_iter_marks_read", self._ctx, None, 0, C.byref(n))
        arr = (_lib.pm_stats * max(1, n.value))()
        _lib.call("pm_iter_marks_read", self._ctx, arr, n.value, C.byref(n))
        return [{name: getattr(s, name) for name, _ in s._fields_} for s in arr[: n.value]]

    def profile(self, reset: bool = False) -> dict:
        """Accumulated device time / weight bytes of the grouped FFN launches (profile_ffn=1)."""
        p = _lib.pm_profile()
        _lib.call("pm_profile_read", self._ctx, C.byref(p), int(reset))
        return {name: getattr(p, name) for name, _ in p._fields_}

    # ------------------------------------------------------------------ fused layer
    def set_layer_weights(self, layer: int, gate_w: torch.Tensor | None, inter: int, top_k: int, norm_topk: bool,
                          routed_scale: float = 1.0, gate_bias: torch.Tensor | None = None,
                          shared: Sequence[torch.Tensor] | None = None,
                          shared_gate_w: torch.Tensor | None = None, quant4: bool = False,
                          hidden: int | None = None) -> None:
        """gate_w [E, H] bf16 on the device; shared = (w_gate [Is, H], w_up [Is, H], w_down [H, Is]).
        gate_w may be None (then pass `hidden`) for a context that only serves pm_moe_forward_routed."""
        def dev(t, dtype):
            if t is None:
                return None
            if not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
                raise ValueError(f"layer weights must be contiguous CUDA tensors of {dtype}")
            self._keep.append(t)
            return t.data_ptr()
        w = _lib.pm_layer_weights()
        w.gate_w = dev(gate_w, torch.bfloat16)
        w.gate_bias = dev(gate_bias, torch.float32)
        w.shared_gate_w = dev(shared_gate_w, torch.bfloat16)
        w.hidden = gate_w.shape[1] if gate_w is not None else int(hidden)
        w.inter = inter
        w.shared_inter = 0
        if shared is not None:
            w.shared_w_gate, w.shared_w_up, w.shared_w_down = (dev(t, torch.bfloat16) for t in shared)
            w.shared_inter = shared[0].shape[0]
        w.top_k, w.norm_topk, w.routed_scale, w.quant4 = top_k, int(norm_topk), routed_scale, int(quant4)
        self._hidden = w.hidden
        _lib.call("pm_layer_set_weights", self._ctx, layer, C.byref(w))

    def set_predictor(self, src: int, dst: int, w1: torch.Tensor, b1: torch.Tensor | None, w2: torch.Tensor,
                      b2: torch.Tensor | None) -> None:
        for t in (w1, b1, w2, b2):
            if t is not None:
                if not t.is_cuda or not t.is_contiguous():
                    raise ValueError("predictor weights must be contiguous CUDA tensors")
                self._keep.append(t)
        _lib.call("pm_predictor_set", self._ctx, src, dst, w1.data_ptr(), None if b1 is None else b1.data_ptr(),
                  w1.shape[0], w2.data_ptr(), None if b2 is None else b2.data_ptr())

    def forward(self, layer: int, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x [T, H] bf16 on the device -> y [T, H] bf16, on torch's current stream."""
        if not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("x must be a contiguous CUDA bf16 tensor")
        x2 = x.view(-1, x.shape[-1])
        y = torch.empty_like(x2) if out is None else out
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.call("pm_moe_forward", self._ctx, layer, x2.data_ptr(), x2.shape[0], y.data_ptr(), stream)
        return y.view(x.shape)

    def forward_host(self, layer: int, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Host-to-host call: x [T, H] bf16 in (pinned) host memory -> y in host memory."""
        if x.device.type != "cpu" or x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("x must be a contiguous CPU bf16 tensor")
        x2 = x.view(-1, x.shape[-1])
        y = torch.empty_like(x2) if out is None else out
        stream = torch.cuda.current_stream().cuda_stream
        _lib.call("pm_moe_forward_host", self._ctx, layer, x2.data_ptr(), x2.shape[0], y.data_ptr(), stream)
        return y.view(x.shape)

    def report_hidden(self, index: int, hidden: torch.Tensor) -> None:
        """hidden [B, seq, H] bf16 entering layer `index` (MoeLayerHook's report_moe_layer_logits)."""
        B, seq = hidden.shape[0], hidden.shape[1]
        stream = torch.cuda.current_stream(hidden.device).cuda_stream
        _lib.call("pm_report_hidden", self._ctx, index, hidden.data_ptr(), B, seq, stream)

    def last_routing(self, layer: int, T: int, k: int):
        ids = np.empty((T, k), np.int32)
        w = np.empty((T, k), np.float32)
        _lib.call("pm_last_routing", self._ctx, layer, ids.ctypes.data_as(C.POINTER(C.c_int32)),
                  w.ctypes.data_as(C.POINTER(C.c_float)), T * k)
        return ids, w
