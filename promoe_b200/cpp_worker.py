"""The reference's `sparse_llm_cache.cpp_worker` module surface over the promoe_b200 C ABI.

Same class, method and enum names as the pybind11 module of the reference
(src/cpp_worker/adapter.cpp:13-158), so `sparse_llm_cache.utils`-style code runs unchanged:
ModuleMeta, ModelLoader, PredictorBase / LegacyPredictor, PrefetchMngr, CacheMngr,
CacheOracle, CacheStatistics, TimerGuard, TraceEventGuard and the free functions.

Differences that a caller can observe, all documented where they occur:
  * no worker threads exist: `launch_thread()` only marks the manager as launched, and every
    cache decision is taken synchronously inside the call that requests it;
  * errors raise `promoe_b200._lib.PromoeError` instead of aborting the process;
  * `ref_one_expert_param` returns a placeholder: the fused MoE block reads expert weights by
    cache slot, module parameters are not re-pointed on every fetch.
"""
from __future__ import annotations

import ctypes as C
import enum
import json
import time

import torch

from . import _lib
from .engine import ExpertCache


# ----------------------------------------------------------------------------- enums (adapter.cpp:129-157)
class ThreadType(enum.IntEnum):
    kPythonMain = 0
    kHook = 1
    kFetchScheduler = 2
    kFetcher = 3
    kUnlocker = 4
    kCache = 5
    kPredictor = 6
    kGPU = 7


class PredictInputMode(enum.IntEnum):
    kNoPredict = 0
    kOneToken = 1
    kDecodeCumsum = 2
    kLastUseDistance = 3
    kWeighedDecodeCumsum = 4
    kFirstMoeAttnInputLogits = 5
    kMoeAttnInputLogits = 6
    kMoeLayerLogits = 7


class PredictorType(enum.IntEnum):
    kLegacyPredictor = 0
    kSepPredictor = 1


class TimeType(enum.IntEnum):
    kModelForward = 0


# pybind's export_values(): the enum members are also module attributes
for _enum in (ThreadType, PredictInputMode, PredictorType, TimeType):
    globals().update(_enum.__members__)

_INPUT_MODES = ["no_predict", "one_token", "decode_cumsum", "last_use_distance", "weighted_decode_cumsum",
                "first_moe_attn_input_logits", "moe_attn_input_logits", "moe_layer_logits"]


# ----------------------------------------------------------------------------- ModuleMeta
class ModuleMeta:
    """Configuration object (src/cpp_worker/utils.hpp:127-192). Fields set before
    `init_from_map` are merged into the map; afterwards every field reads and writes the
    library context, which is created by `init_from_map`."""

    _FIELDS = ("model_arch_string", "num_layer", "num_expert", "num_per_expert_param",
               "num_predict_expert_per_layer", "num_expert_per_token", "max_prefetch_layer_distance",
               "per_layer_cache", "cache_policy", "reorder_experts", "promote_hit_in_prefetch", "early_preempt",
               "chunk_prefetch", "predict_input_mode", "predictor_type", "layer_predict_interval",
               "layer_predict_max_window", "layer_predict_replace_first_input_with_last_output",
               "limit_layer_0_window", "limit_layer_0_num_predict", "cache_only")
    _BOOL = {"per_layer_cache", "reorder_experts", "promote_hit_in_prefetch", "early_preempt", "chunk_prefetch",
             "layer_predict_replace_first_input_with_last_output", "cache_only"}
    _STR = {"model_arch_string", "cache_policy"}

    def __init__(self, num_layer: int, num_expert: int):
        object.__setattr__(self, "_pending", {})
        object.__setattr__(self, "_param_names", [])
        object.__setattr__(self, "_cache", None)
        object.__setattr__(self, "_shape", (int(num_layer), int(num_expert)))

    # -- field access
    def __getattr__(self, name):
        if name not in ModuleMeta._FIELDS:
            raise AttributeError(name)
        if name == "num_layer":
            return self._shape[0]
        if name == "num_expert":
            return self._shape[1]
        if self._cache is None:
            if name in self._pending:
                return self._pending[name]
            raise AttributeError(f"{name} is not resolved before init_from_map")
        raw = self._cache.get(name)
        if name == "predict_input_mode":
            return PredictInputMode(_INPUT_MODES.index(raw))
        if name == "predictor_type":
            return PredictorType.kSepPredictor if raw == "sep" else PredictorType.kLegacyPredictor
        if name in ModuleMeta._BOOL:
            return raw == "true"
        return raw if name in ModuleMeta._STR else int(raw)

    def __setattr__(self, name, value):
        if name not in ModuleMeta._FIELDS:
            raise AttributeError(f"ModuleMeta has no field {name}")
        if name in ("num_layer", "num_expert", "num_per_expert_param"):
            raise AttributeError(f"{name} is fixed at construction")
        if self._cache is None:
            self._pending[name] = value
        else:
            self._cache.set(name, value)

    # -- reference methods
    def init_param_list(self, params):
        object.__setattr__(self, "_param_names", list(params))
        if self._cache is not None:
            self._cache.set_param_list(self._param_names)

    def init_from_map(self, config_map: dict):
        cfg = {k: str(v) for k, v in config_map.items()}
        for k, v in self._pending.items():
            cfg.setdefault(k, str(v))
        cache = ExpertCache(self._shape[0], self._shape[1], **cfg)
        object.__setattr__(self, "_cache", cache)
        if self._param_names:
            cache.set_param_list(self._param_names)

    def handle_uninited_configs(self):
        """Defaults and environment overrides are resolved when the context is created."""
        if self._cache is None:
            raise RuntimeError("handle_uninited_configs before init_from_map")

    @property
    def cache(self) -> ExpertCache:
        if self._cache is None:
            raise RuntimeError("ModuleMeta.init_from_map has not been called")
        return self._cache


# ----------------------------------------------------------------------------- predictor
class PredictorBase:
    """Predictor handle (src/cpp_worker/predictor.hpp:40-67). The MLPs run on the GPU inside the
    library; `load_model` reads a directory of `<src>-<dst>.pt` files holding either a
    TorchScript module or a state dict of one MLP hidden -> d -> num_expert
    (first and last 2-D tensors = the two matrices, 1-D tensors = biases)."""

    def __init__(self, meta: ModuleMeta):
        self.metas = meta
        self.loaded = {}

    @staticmethod
    def create(meta: ModuleMeta) -> "PredictorBase":
        return LegacyPredictor(meta) if meta.predictor_type == PredictorType.kLegacyPredictor else PredictorBase(meta)

    def load_model(self, path: str | None = None):
        import os
        cache = self.metas.cache
        path = path if path is not None else cache.get("predictor_model_path")
        if not path:
            return  # no predictor configured: prediction stays off
        if not os.path.isdir(path):
            raise FileNotFoundError(f"Model file is not a directory: {path}")
        from .synth import predict_layer_mapping
        L = self.metas.num_layer
        mapping = predict_layer_mapping(L, int(cache.get("layer_predict_interval")),
                                        int(cache.get("layer_predict_max_window")),
                                        int(cache.get("limit_layer_0_window")))
        for src, (a, b) in enumerate(mapping):
            for dst in range(a, b):
                f = os.path.join(path, f"{src}-{dst}.pt")
                obj = torch.load(f, map_location="cpu", weights_only=False) if not _is_torchscript(f) \
                    else torch.jit.load(f, map_location="cpu")
                self.set_mlp(src, dst, *_mlp_tensors(obj))

    def set_mlp(self, src: int, dst: int, w1, b1, w2, b2):
        dev = torch.device("cuda", torch.cuda.current_device())
        t = [None if v is None else v.detach().to(dev) for v in (w1, b1, w2, b2)]
        w1d, w2d = t[0].to(torch.bfloat16).contiguous(), t[2].to(torch.bfloat16).contiguous()
        b1d = None if t[1] is None else t[1].float().contiguous()
        b2d = None if t[3] is None else t[3].float().contiguous()
        self.loaded[(src, dst)] = (w1d, b1d, w2d, b2d)
        self.metas.cache.set_predictor(src, dst, w1d, b1d, w2d, b2d)


class LegacyPredictor(PredictorBase):
    """Kept for name compatibility (src/cpp_worker/predictor.hpp:69-136); same device path."""


def _is_torchscript(path: str) -> bool:
    import zipfile
    try:
        with zipfile.ZipFile(path) as z:
            return any(n.endswith("constants.pkl") for n in z.namelist())
    except zipfile.BadZipFile:
        return False


def _mlp_tensors(obj):
    sd = obj.state_dict() if hasattr(obj, "state_dict") else dict(obj)
    mats = [v for v in sd.values() if v.dim() == 2]
    vecs = [v for v in sd.values() if v.dim() == 1]
    if len(mats) != 2:
        raise ValueError("predictor file must hold exactly two weight matrices (hidden -> d -> num_expert)")
    b1 = next((v for v in vecs if v.shape[0] == mats[0].shape[0]), None)
    b2 = next((v for v in vecs if v.shape[0] == mats[1].shape[0] and v is not b1), None)
    return mats[0], b1, mats[1], b2


# ----------------------------------------------------------------------------- ModelLoader
class ModelLoader:
    """Expert registry (src/cpp_worker/model_loader.hpp:276-319)."""

    def __init__(self, meta: ModuleMeta):
        self.metas = meta
        self._names = {n: i for i, n in enumerate(meta._param_names)}
        self._dtype = {}

    def add_one_expert_param(self, param: torch.Tensor, layer_id: int, expert_id: int, param_name: str):
        pid = self._names[param_name]
        t = param.detach()
        if t.device.type != "cpu":
            t = t.cpu()
        if t.is_floating_point() and t.dtype != torch.bfloat16 and t.dim() == 2:
            t = t.to(torch.bfloat16)  # the device kernels compute on bf16 weight matrices
        self._dtype[pid] = t.dtype
        _register_one(self.metas.cache, layer_id, expert_id, pid, t)

    def build_logical_expert_param(self):
        """Nothing to build: weights are addressed by cache slot, not through re-pointed tensors."""

    def ref_one_expert_param(self, layer_id: int, expert_id: int, param) -> torch.Tensor:
        pid = self._names[param] if isinstance(param, str) else int(param)
        return torch.empty(0, dtype=self._dtype.get(pid, torch.bfloat16), device="cuda")

    def pin_memory(self):
        if not self.metas.cache.pinned:  # init_gpu_mem_buffer may have pinned already
            self.metas.cache.pin_all()


def _register_one(cache: ExpertCache, layer, expert, pid, t: torch.Tensor):
    t = t.contiguous()
    cache._keep.append(t)
    _lib.call("pm_register_expert_param", cache.handle, layer, expert, pid, t.data_ptr(), t.numel() * t.element_size())


# ----------------------------------------------------------------------------- cache handles
class CacheOracle:
    """Trace loader of the Belady policy (src/cpp_worker/cache.cpp:431-489,592-644)."""

    def __init__(self, cache: ExpertCache, num_layer: int, num_expert: int):
        self._cache, self._L, self._E = cache, num_layer, num_expert

    def load_from_tensor(self, entry_metas, prefill_expert_len, prefill_expert_selection, decode_expert_selection):
        num_seq = prefill_expert_len.shape[0]
        reply_len = torch.bincount(entry_metas[:, 0].long(), minlength=num_seq)
        begin = 0
        for seq in range(num_seq):
            use = {}
            time_ = 0
            for l in range(self._L):
                for off in range(int(prefill_expert_len[seq][l])):
                    use.setdefault((l, int(prefill_expert_selection[seq][l][off])), []).append(time_)
                time_ += 1
            for r in range(int(reply_len[seq])):
                for l in range(self._L):
                    for e in decode_expert_selection[begin + r][l].tolist():
                        use.setdefault((l, int(e)), []).append(time_)
                    time_ += 1
            begin += int(reply_len[seq])
            for l in range(self._L):
                for e in range(self._E):
                    self._cache.add_use_times(seq, l, e, use.get((l, e), []))

    def load_from_file(self, file_path: str):
        with open(file_path) as f:
            traces = json.load(f)
        for key, tr in traces.items():
            seq, prompt_len = int(key), int(tr["prompt_len"])
            reply = len(tr["0"]) - prompt_len
            use, time_ = {}, 0
            for l in range(self._L):
                ids = sorted({int(e) for t in range(prompt_len) for e in tr[str(l)][str(t)]})
                for e in ids:
                    use.setdefault((l, e), []).append(time_)
                time_ += 1
            for r in range(reply):
                for l in range(self._L):
                    for e in tr[str(l)][str(r + prompt_len)]:
                        use.setdefault((l, int(e)), []).append(time_)
                    time_ += 1
            for l in range(self._L):
                for e in range(self._E):
                    self._cache.add_use_times(seq, l, e, use.get((l, e), []))


class CacheMngr:
    def __init__(self, cache: ExpertCache, num_layer: int, num_expert: int):
        self._cache = cache
        self.cache_oracle = CacheOracle(cache, num_layer, num_expert)

    def set_cur_seq(self, seq_id: int):
        self._cache.set_cur_seq(int(seq_id))


class CacheStatistics:
    """Per layer-call ready / unready counts (src/cpp_worker/profiler.hpp:201-251)."""

    def __init__(self):
        self.rows = []

    def forward(self):
        self.rows.append([0, 0])

    def to_tensor(self) -> torch.Tensor:
        return torch.tensor(self.rows, dtype=torch.float32).reshape(-1, 2)

    def dump_average(self, prefill_cnt_threshold: int) -> torch.Tensor:
        t = self.to_tensor()
        return t[t.sum(1) <= prefill_cnt_threshold].mean(0)

    def dump_average_per_layer(self, num_layer: int, prefill_cnt_threshold: int) -> torch.Tensor:
        t = self.to_tensor()
        t = t[t.sum(1) <= prefill_cnt_threshold]
        return t.reshape(-1, num_layer, 2).mean(0)


class TimeProfiler:
    def __init__(self):
        self.series = {TimeType.kModelForward: []}

    def push(self, kind, dur_us):
        self.series.setdefault(kind, []).append(int(dur_us))


class TimerGuard:
    """Times one span into the profiler (src/cpp_worker/profiler.hpp:321-346)."""

    def __init__(self, profiler: TimeProfiler):
        self._profiler, self._start, self._kind = profiler, None, None

    def init(self, kind):
        self._kind, self._start = kind, time.perf_counter()

    def release(self):
        if self._start is not None:
            self._profiler.push(self._kind, (time.perf_counter() - self._start) * 1e6)
            self._start = None


_TRACE_EVENTS: list[dict] = []


class TraceEventGuard:
    """Chrome-trace span (src/cpp_worker/profiler.hpp:134-178); recorded only while
    SPARSE_CACHE_ENABLE_TRACE is on."""

    def __init__(self):
        self._ev = None

    def init(self, tid, name, phase="X"):
        import os
        if os.environ.get("SPARSE_CACHE_ENABLE_TRACE", "").lower() in ("1", "on", "true"):
            self._ev = {"name": name, "ph": phase, "tid": int(tid), "pid": 0, "ts": time.perf_counter() * 1e6}

    def release(self):
        if self._ev is not None:
            self._ev["dur"] = time.perf_counter() * 1e6 - self._ev["ts"]
            _TRACE_EVENTS.append(self._ev)
            self._ev = None


def dump_trace_event_collector_singleton() -> str:
    return json.dumps({"traceEvents": _TRACE_EVENTS})


# ----------------------------------------------------------------------------- PrefetchMngr
class PrefetchMngr:
    """The manager the hooks talk to (src/cpp_worker/prefetcher.hpp:134-196)."""

    def __init__(self, meta: ModuleMeta, model_loader: ModelLoader, predictor: PredictorBase):
        self.metas, self.model_loader, self.predictor = meta, model_loader, predictor
        self._cache = meta.cache
        self.cache = CacheMngr(self._cache, meta.num_layer, meta.num_expert)
        self.cache_stats = CacheStatistics()
        self.profiler = TimeProfiler()
        # The reference creates a private non-blocking compute stream and makes torch use it
        # (prefetcher.cpp:406-418); this keeps that contract for the caller's set_stream().
        self._stream = torch.cuda.Stream()
        self.compute_stream = self._stream.cuda_stream
        self.copy_stream = 0  # owned by the library, created with the slab
        self.launched = False

    def launch_thread(self):
        self.launched = True  # no worker threads: decisions are taken inside the requesting call

    def reload_env(self):
        pass

    def init_gpu_mem_buffer(self):
        # The reference pins after building the lines (utils/__init__.py:331-334); here the pinned
        # records fix the line size and are the copy source, so they are built first.
        if not self._cache.pinned:
            self._cache.pin_all()
        self._cache.build_slab()

    def report_one_layer(self, layer_id: int, experts: torch.Tensor):
        if experts.dtype != torch.int64 or experts.device.type != "cpu" or not experts.is_contiguous():
            raise ValueError("experts must be a contiguous CPU int64 tensor (it is reordered in place)")
        self.cache_stats.forward()
        _lib.call("pm_report_layer", self._cache.handle, layer_id,
                  C.cast(experts.data_ptr(), C.POINTER(C.c_int64)), experts.numel())

    def report_one_expert(self, layer_id: int, expert_id: int):
        self._cache.report_expert(layer_id, expert_id)

    def one_expert_done(self, layer_id: int, expert_id: int):
        self._cache.expert_done(layer_id, expert_id)

    def one_moe_layer_done(self, layer_id: int):
        self._cache.layer_done(layer_id)

    def report_moe_attn_logits(self, layer_id: int, attn_logits: torch.Tensor):
        pass  # only the moe_layer_logits input mode has a device predictor

    def report_moe_layer_logits(self, layer_id: int, layer_logits: torch.Tensor):
        if self._cache.get("predict_input_mode") != "moe_layer_logits":
            return  # the other input modes ignore hidden states (predictor.cpp:641-648)
        if layer_logits.dim() != 3:
            raise ValueError(f"input logits must be [batch, seq_len, hidden], found {tuple(layer_logits.shape)}")
        if layer_logits.shape[1] != 1 or not layer_logits.is_cuda:
            return
        h = layer_logits if layer_logits.dtype == torch.bfloat16 else layer_logits.to(torch.bfloat16)
        self._cache.report_hidden(layer_id, h.contiguous())

    def build_timer(self) -> TimerGuard:
        return TimerGuard(self.profiler)

    def temp_move_expert_to_gpu(self, layer_id: int, expert_id: int):
        raise _lib.PromoeError(4, "temp_move_expert_to_gpu serves exllama post_init, which this library does not run")

    def temp_move_expert_back_to_host(self, layer_id: int, expert_id: int):
        raise _lib.PromoeError(4, "temp_move_expert_back_to_host serves exllama post_init, which this library does not run")

    def __reduce__(self):
        raise TypeError("PrefetchMngr cannot be pickled across processes")


# ----------------------------------------------------------------------------- free functions
def to_um(t: torch.Tensor) -> torch.Tensor:
    """The reference's managed-memory baseline (model_loader.cpp:166-173) is not part of the
    MoE hot path; the nearest equivalent here keeps the tensor in pinned host memory."""
    return t.detach().cpu().pin_memory()


def log_gpu_mem_info(tag: str = ""):
    free, total = torch.cuda.mem_get_info()
    print(f"{tag} gpu memory free {free / 2**20:.0f} MiB / total {total / 2**20:.0f} MiB")


_EATEN = []


def eat_cuda_memory(nbytes: int):
    _EATEN.append(torch.empty(int(nbytes), dtype=torch.uint8, device="cuda"))


def auto_eat_cuda_memory():
    import os
    mib = os.environ.get("SPARSE_EVAL_EAT_CUDA_MEMORY_MiB")
    if mib:
        eat_cuda_memory(int(mib) << 20)
