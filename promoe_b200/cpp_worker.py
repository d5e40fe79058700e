"""The reference's `sparse_llm_cache.cpp_worker` module surface over the promoe_b200 C ABI.

Same class, method and enum names as the pybind11 module of the reference
(src/cpp_worker/adapter.cpp:13-158), so `sparse_llm_cache.utils`-style code runs unchanged:
ModuleMeta, ModelLoader, PredictorBase / LegacyPredictor, PrefetchMngr, CacheMngr,
CacheOracle, CacheStatistics, TimerGuard, TraceEventGuard and the free functions.

Differences that a caller can observe, all documented where they occur:
  * no worker threads exist: `launch_thread()` only marks the manager as launched, and every
    cache decision is taken synchronously inside the call that requests it;
  * errors raise `promoe_b200._lib.PromoeError` instead of aborting the process;
  * `ref_one_expert_param` returns a tensor that aliases the expert's current cache line; it is
    re-pointed inside `report_one_expert` (the reference does it on the fetch thread). The fused
    MoE block does not need it: it reads expert weights by cache slot.
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

    HISTORY_MODES = ("one_token", "decode_cumsum", "last_use_distance", "weighted_decode_cumsum")

    def __init__(self, meta: ModuleMeta):
        self.metas = meta
        self.loaded = {}
        self.history_model = None   # optional module for the history-based input modes

    def history_scores(self, hist: torch.Tensor):
        """Scores from the history-based predictor input `hist` [num_layer, num_expert]
        (LegacyPredictor::predict, src/cpp_worker/predictor.cpp:143-175,240-250): the model is applied
        to the rows, its output reshaped to [rows, -1, num_expert] and summed over the rows. Without
        a model file the history itself is the score of every layer (frequency / recency ranking).
        Returns (scores [n_layers, num_expert] float32, first predicted layer)."""
        E = hist.shape[1]
        if self.history_model is None:
            return hist.float().contiguous(), 0
        with torch.no_grad():
            out = self.history_model(hist.float().flatten(1, -1))
        return out.reshape(hist.shape[0], -1, E).sum(0).float().contiguous(), 0

    @staticmethod
    def create(meta: ModuleMeta) -> "PredictorBase":
        return LegacyPredictor(meta) if meta.predictor_type == PredictorType.kLegacyPredictor else PredictorBase(meta)

    def load_model(self, path: str | None = None):
        import os
        cache = self.metas.cache
        path = path if path is not None else cache.get("predictor_model_path")
        if not path or path == "None":
            return  # no predictor configured: prediction stays off
        if cache.get("predict_input_mode") in self.HISTORY_MODES:
            # one model file for the whole stack (LegacyPredictor::load_model, predictor.cpp:262-281)
            self.history_model = torch.jit.load(path, map_location="cpu") if _is_torchscript(path) \
                else torch.load(path, map_location="cpu", weights_only=False)
            self.history_model.eval()
            return
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
        self._shape = {}     # (layer, expert, pid) -> tensor shape
        self._logical = {}   # (layer, expert, pid) -> the tensor handed to the model
        self._line = {}      # (layer, expert) -> line address the logical tensors point at
        self._slab = None

    def add_one_expert_param(self, param: torch.Tensor, layer_id: int, expert_id: int, param_name: str):
        pid = self._names[param_name]
        t = param.detach()
        if t.device.type != "cpu":
            t = t.cpu()
        if t.is_floating_point() and t.dtype != torch.bfloat16 and t.dim() == 2:
            t = t.to(torch.bfloat16)  # the device kernels compute on bf16 weight matrices
        self._dtype[pid] = t.dtype
        self._shape[(layer_id, expert_id, pid)] = tuple(t.shape)
        _register_one(self.metas.cache, layer_id, expert_id, pid, t)

    def build_logical_expert_param(self):
        """Logical tensors are created on demand by ref_one_expert_param."""

    def ref_one_expert_param(self, layer_id: int, expert_id: int, param) -> torch.Tensor:
        """The tensor a module uses for one expert tensor (ModelLoader::ref_one_expert_param,
        src/cpp_worker/model_loader.hpp:290-313): it has the registered shape and dtype once the
        expert has been fetched and aliases the cache line that holds the expert; before the
        first fetch it is empty. `PrefetchMngr.report_one_expert` re-points it."""
        pid = self._names[param] if isinstance(param, str) else int(param)
        key = (layer_id, expert_id, pid)
        if key not in self._logical:
            self._logical[key] = torch.empty(0, dtype=self._dtype.get(pid, torch.bfloat16), device="cuda")
        return self._logical[key]

    def repoint(self, layer_id: int, expert_id: int, line_addr: int):
        """Points the logical tensors of one expert at the cache line at `line_addr`."""
        if self._line.get((layer_id, expert_id)) == line_addr:
            return
        cache = self.metas.cache
        if self._slab is None:
            self._slab = cache.slab_tensor()
            self._slab_base = int(cache.get("slab_base"))
            self._offsets = [cache.param_offset(p) for p in range(len(self._names))]
            self._ranges, self._ranges_base = None, 0
            if cache.get("stable_va") == "true":  # addresses then lie in the experts' own ranges
                self._ranges, self._ranges_base = cache.expert_range_tensor(), int(cache.get("expert_va_base"))
        raw, base = self._slab, self._slab_base
        if self._ranges is not None and not (base <= line_addr < base + raw.numel()):
            raw, base = self._ranges, self._ranges_base
        for pid in range(len(self._names)):
            key = (layer_id, expert_id, pid)
            t = self._logical.get(key)
            if t is None:
                continue
            shape, dtype = self._shape[key], self._dtype[pid]
            n = 1
            for d in shape:
                n *= d
            off = line_addr - base + self._offsets[pid]
            view = raw[off:off + n * torch.empty(0, dtype=dtype).element_size()].view(dtype).view(shape)
            with torch.no_grad():
                t.set_(view)
        self._line[(layer_id, expert_id)] = line_addr

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
                row = entry_metas[begin + r]
                if int(row[0]) != seq or int(row[1]) != r:  # the reference CHECKs the same (cache.cpp:624-625)
                    raise ValueError(f"trace entry {begin + r} is (seq {int(row[0])}, token {int(row[1])}), "
                                     f"expected (seq {seq}, token {r})")
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
    """Per layer-call ready / unready counts (src/cpp_worker/profiler.hpp:201-251): one row per
    `report_one_layer`, filled from the library's counters. "Ready" is an activated expert that was
    completely resident when it was demanded, "unready" one whose copy the demand had to issue or
    finish (the reference counts whether the main thread had to spin in wait_expert,
    src/cpp_worker/prefetcher.cpp:243-258; here the host never waits, the device does)."""

    def __init__(self, cache: ExpertCache | None = None):
        self._cache = cache
        self.rows = []
        self._last = (0, 0)

    def _settle(self):
        if self._cache is None or not self.rows:
            return
        st = self._cache.stats()
        now = (st["ready"], st["unready"])
        self.rows[-1][0] += now[0] - self._last[0]
        self.rows[-1][1] += now[1] - self._last[1]
        self._last = now

    def forward(self):
        self._settle()
        self.rows.append([0, 0])

    def to_tensor(self) -> torch.Tensor:
        self._settle()
        return torch.tensor(self.rows, dtype=torch.float32).reshape(-1, 2)

    def dump_average(self, prefill_cnt_threshold: int) -> torch.Tensor:
        t = self.to_tensor()
        return t[t.sum(1) <= prefill_cnt_threshold].mean(0)

    def dump_average_per_layer(self, num_layer: int, prefill_cnt_threshold: int) -> torch.Tensor:
        t = self.to_tensor()
        t = t[t.sum(1) <= prefill_cnt_threshold]
        return t.reshape(-1, num_layer, 2).mean(0)


class TimeProfiler:
    """The per-forward series of the reference's TimeProfiler (src/cpp_worker/profiler.hpp:262-319).
    The counter series come from the library (differences of its end-of-iteration snapshots); the
    forward times and sequence lengths are pushed on the Python side, where the reference's hooks
    produce them (TimingHook, MoeLayerHook at layer 0)."""

    COUNTER_KINDS = {"activated": "activated_experts", "hit": "precise_hit", "miss": "precise_miss",
                     "ready": "ready", "unready": "unready", "prefetch_hit": "prefetch_hit",
                     "prefetch_miss": "prefetch_miss"}

    def __init__(self, cache: ExpertCache | None = None):
        self._cache = cache
        self.series = {TimeType.kModelForward: [], "seq_len": [], "predict_time": []}

    def push(self, kind, value):
        self.series.setdefault(kind, []).append(int(value))

    def to_tensor(self, kind) -> torch.Tensor:
        """One value per completed model iteration for the counter kinds ("hit", "miss", "ready",
        "unready", "prefetch_hit", "prefetch_miss", "activated", "wait_time"), one per push for
        TimeType.kModelForward, "seq_len" and "predict_time"."""
        if kind in self.COUNTER_KINDS:
            field, prev, out = self.COUNTER_KINDS[kind], 0, []
            for m in (self._cache.iter_marks() if self._cache is not None else []):
                out.append(m[field] - prev)
                prev = m[field]
            return torch.tensor(out, dtype=torch.int64)
        if kind == "wait_time":  # the host never waits for a copy: the device stream does
            n = len(self._cache.iter_marks()) if self._cache is not None else 0
            return torch.zeros(n, dtype=torch.int64)
        return torch.tensor(self.series.get(kind, []), dtype=torch.int64)

    def report_lines(self) -> list[str]:
        """The `key:value` lines the reference prints when its profiler is destroyed
        (src/cpp_worker/prefetcher.cpp:327-402), which its sweep scripts parse: means over the decode
        and the prefill iterations after the warm-up prompts (the first four prefill iterations and
        everything before them are skipped, five when the run starts llama.cpp style with prefill
        iterations at positions 0, 1, 2)."""
        seq = self.to_tensor("seq_len")
        n = min(len(seq), len(self.to_tensor("hit")))
        seq = seq[:n]
        is_prefill, is_decode = seq > 1, seq <= 1
        prefill_idx = torch.nonzero(is_prefill).flatten().tolist()
        skip = 5 if len(prefill_idx) > 2 and prefill_idx[1] == 1 and prefill_idx[2] == 2 else 4
        start = n if len(prefill_idx) <= skip else prefill_idx[skip]
        is_prefill[:start] = False
        is_decode[:start] = False

        def mean(kind, idx, scale=1.0):
            t = self.to_tensor(kind)[:n][idx].float()
            return float("nan") if t.numel() == 0 else t.mean().item() / scale

        lines = []
        for on, off, name in (("ready", "unready", "ready"), ("hit", "miss", "hit"),
                              ("prefetch_hit", "prefetch_miss", "prefetch_hit")):
            for stage, idx in (("decode", is_decode), ("prefill", is_prefill)):
                a, b = mean(on, idx), mean(off, idx)
                off_name = name.replace("hit", "miss") if "hit" in name else "unready"
                lines += [f"{stage}_stage_{name}_cnt:{a:g}", f"{stage}_stage_{off_name}_cnt:{b:g}",
                          f"{stage}_stage_{name}_rate:{(a / (a + b) if a + b else float('nan')):g}"]
        fwd = self.to_tensor(TimeType.kModelForward)[:n]
        for stage, idx in (("decode", is_decode), ("prefill", is_prefill)):
            lines.append(f"{stage}_stage_wait_time:{mean('wait_time', idx, 1000.0):g}")
        for stage, idx in (("decode", is_decode), ("prefill", is_prefill)):
            t = fwd[idx[:len(fwd)]].float() if len(fwd) else fwd.float()
            lines.append(f"{stage}_stage_forward_time:{(t.mean().item() / 1000.0 if t.numel() else float('nan')):g}")
        lines += [f"num_prefill_iter:{int(is_prefill.sum())}", f"num_decode_iter:{int(is_decode.sum())}"]
        pt = self.to_tensor("predict_time")[10:].float()
        lines.append(f"predict_time:{(pt.mean().item() / 1000.0 if pt.numel() else float('nan')):g}")
        return lines


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
        self.cache_stats = CacheStatistics(self._cache)
        self.profiler = TimeProfiler(self._cache)
        # The reference creates a private non-blocking compute stream and makes torch use it
        # (prefetcher.cpp:406-418); this keeps that contract for the caller's set_stream().
        self._stream = torch.cuda.Stream() if torch.cuda.is_available() else None  # policy-only use needs no GPU
        self.compute_stream = self._stream.cuda_stream if self._stream is not None else 0
        self.copy_stream = 0  # owned by the library, created with the slab
        self.launched = False

    def launch_thread(self):
        """No worker threads exist: decisions are taken inside the requesting call. What remains of
        the reference's launch is the end-of-run report, printed at interpreter exit like the
        reference's profiler destructor does."""
        if not self.launched:
            import atexit
            atexit.register(self._report_at_exit)
        self.launched = True

    def _report_at_exit(self):
        try:
            lines = self.profiler.report_lines()
            kept = sum(int(ln.split(":")[1]) for ln in lines if ln.startswith(("num_prefill_iter", "num_decode_iter")))
            if kept > 0:  # a run shorter than the reference's warm-up (four prompts) has nothing to report
                print("\n".join(lines), flush=True)
        except Exception:
            pass  # the context may already be closed

    def reload_env(self):
        """Re-reads the environment switches of the reference's logging and tracing
        (src/cpp_worker/prefetcher.cpp:659-662). Tracing is read from the environment on every span
        here, so there is nothing to cache."""

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
        """report_one_expert + wait_expert (src/cpp_worker/prefetcher.cpp:225-258). With a slab, torch's
        current stream is made to wait for the expert's copy (the host does not wait) and the expert's
        logical parameters are pointed at its cache line."""
        if self._cache.get("slab_impl") == "none":
            self._cache.report_expert(layer_id, expert_id)
            return
        line = self._cache.expert_acquire(layer_id, expert_id, torch.cuda.current_stream().cuda_stream)
        self.model_loader.repoint(layer_id, expert_id, line)

    def one_expert_done(self, layer_id: int, expert_id: int):
        if self._cache.get("slab_impl") == "none":
            self._cache.expert_done(layer_id, expert_id)
            return
        self._cache.expert_release(layer_id, expert_id, torch.cuda.current_stream().cuda_stream)

    def one_moe_layer_done(self, layer_id: int):
        self._cache.layer_done(layer_id)
        if layer_id == self.metas.num_layer - 1:
            self._predict_from_history()

    def _predict_from_history(self):
        """End of a model iteration in a history-based input mode (PredictWorker::on_one_iter_done ->
        do_one_task_impl, src/cpp_worker/worker.cpp:6-77): score every layer from the access history,
        hand the scores to the NN policy and prefetch the top experts of every layer in layer order."""
        mode = self._cache.get("predict_input_mode")
        if mode not in PredictorBase.HISTORY_MODES:
            return
        n = int(self._cache.get("num_predict_expert_per_layer"))
        nn = self._cache.get("cache_policy") == "nn"
        if n <= 0 and not nn:
            return
        t0 = time.perf_counter()
        scores, start = self.predictor.history_scores(torch.from_numpy(self._cache.history_input()))
        self.profiler.push("predict_time", (time.perf_counter() - t0) * 1e6)
        if nn:
            self._cache.update_priority(scores.numpy(), start)
        if n > 0:
            order = torch.argsort(scores, dim=1, descending=True, stable=True)[:, :n]
            for i in range(scores.shape[0]):
                self._cache.prefetch_layer(start + i, order[i].tolist())

    def report_moe_attn_logits(self, layer_id: int, attn_logits: torch.Tensor):
        # The separate-model predictor ignores attention logits, as the reference's does (the base
        # class method is empty, src/cpp_worker/predictor.hpp:53); only the legacy predictor's input
        # modes consume them, and those have no device path here.
        return None

    def report_moe_layer_logits(self, layer_id: int, layer_logits: torch.Tensor):
        if layer_id == 0 and layer_logits.dim() == 3:
            self.profiler.push("seq_len", layer_logits.shape[1])  # prefetcher.cpp:453-456
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
        """Copies the expert into the spare cache line and points its logical parameters there, so
        that a quantised layer's post_init can work on device tensors
        (src/cpp_worker/prefetcher.cpp:664-680; used by AutoGPTQFirstPostInitHook)."""
        line = self._cache.temp_move_expert_to_gpu(layer_id, expert_id, torch.cuda.current_stream().cuda_stream)
        self.model_loader.repoint(layer_id, expert_id, line)

    def temp_move_expert_back_to_host(self, layer_id: int, expert_id: int):
        """Copies the spare line back into the expert's pinned host record (prefetcher.cpp:681-697)."""
        self._cache.temp_move_expert_back_to_host(layer_id, expert_id, torch.cuda.current_stream().cuda_stream)

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
