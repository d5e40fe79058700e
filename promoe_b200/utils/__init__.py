"""The injection API of `sparse_llm_cache.utils`, over the B200 library: `inject_model`,
`launch`, `hack_transformers`, `inject_model_um`, `hack_transformers_um` and the helper
functions the reference exports next to them (src/sparse_llm_cache/utils/__init__.py).

`inject_model(model, **config)` takes the same keyword arguments as the reference's
(utils/__init__.py:147-191) and performs the same steps in the same order: metadata lookup by
model id, configuration, registration of every expert tensor, cache lines, re-pointing of the
expert parameters, the `report_experts` closure on every MoE block, predictor loading, hooks,
pinning, launch. One step is added: with `fused=True` (default) the forward of every MoE block
is replaced by the fused device path, which is what the reference's patched transformers fork
provides on its side.
"""
from __future__ import annotations

import functools
import os

import torch

from .. import cpp_worker
from . import hooks
from .common_metas import ModelMetas, auto_infer_model_metas, predefined_metas  # noqa: F401
from .filter import Filter, RegexFilter  # noqa: F401
from .hooks import *  # noqa: F401,F403


# ----------------------------------------------------------------------------- tree walks
def recursive_traverse_childrens(module, func, filter=Filter(), prefix="", reverse_filter=False):
    """Calls func(module, name) on every module of the tree whose dotted name passes `filter`."""
    if filter(prefix):
        func(module, prefix)
    for name, child in module.named_children():
        recursive_traverse_childrens(child, func, filter, f"{prefix}.{name}" if prefix else name, reverse_filter)


def recursive_traverse_childrens_leaf_only(module, func, filter=Filter(), prefix="", reverse_filter=False):
    """Same, but only modules without children are visited."""
    children = list(module.named_children())
    for name, child in children:
        recursive_traverse_childrens_leaf_only(child, func, filter, f"{prefix}.{name}" if prefix else name, reverse_filter)
    if not children and filter(prefix):
        func(module, prefix)


def add_metadata_to_submodules(model, parse_expert_meta_from_name):
    def tag(module, name):
        module._prefix = name
        layer, expert = parse_expert_meta_from_name(name)
        if layer is not None and expert is not None:
            module._layer_id, module._expert_id = int(layer), int(expert)
        elif layer is not None:
            module._layer_id = int(layer)
    recursive_traverse_childrens(model, tag)


def add_prefix_to_submodules(model):
    recursive_traverse_childrens(model, lambda m, n: setattr(m, "_prefix", n))


def param_buffer_name_to_prefetch(name: str) -> bool:
    """Buffers of quantised layers that travel with the expert (utils/__init__.py:39-46)."""
    return any(k in name for k in ("qweight", "zero", "scale"))


_EXPERT = RegexFilter(r".*layers\.(\d+)\.mlp\.experts\.(\d+)$")


def _expert_tensors(module):
    for k, v in module.named_parameters():
        yield k, v
    for k, v in module.named_buffers():
        if param_buffer_name_to_prefetch(k):
            yield k, v


def register_expert_params(model, model_loader, filter=_EXPERT):
    def reg(module, name):
        for k, v in _expert_tensors(module):
            model_loader.add_one_expert_param(v, module._layer_id, module._expert_id, k)
    recursive_traverse_childrens(model, reg, filter)


def replace_expert_param_reference(model, model_loader, filter=_EXPERT):
    """Points every expert parameter at the loader's logical tensor, which releases the original
    host copy once it has been pinned into the cache's records. The logical tensor object itself
    goes into the module (as in the reference, utils/__init__.py:58-69): the loader re-points it in
    place whenever the expert moves to another cache line."""
    model_loader.build_logical_expert_param()

    def per_expert(module, name):
        def per_leaf(leaf, leaf_name):
            for n, _ in list(leaf.named_parameters(recurse=False)):
                leaf._parameters[n] = model_loader.ref_one_expert_param(module._layer_id, module._expert_id,
                                                                        f"{leaf_name}.{n}")
            for n, _ in list(leaf.named_buffers(recurse=False)):
                if param_buffer_name_to_prefetch(n):
                    leaf._buffers[n] = model_loader.ref_one_expert_param(module._layer_id, module._expert_id, f"{leaf_name}.{n}")
        recursive_traverse_childrens_leaf_only(module, per_leaf)
    recursive_traverse_childrens(model, per_expert, filter)


def attach_prefetch_mngr_to_all_module(model, prefetch_mngr):
    recursive_traverse_childrens(model, lambda m, n: setattr(m, "_prefetch_mngr", prefetch_mngr), RegexFilter(r".*"))


def move_non_moe_to_gpu(model, device="cuda", filter=RegexFilter(r".*layers\.(\d+)\.mlp\.experts\.(\d+)").reverse()):
    recursive_traverse_childrens_leaf_only(model, lambda m, n: m.to(device), filter)


def replace_mlp_report_experts(model, prefetch_mngr, predictor, num_moe_layer, num_expert, num_predict_expert,
                               filter=RegexFilter(r".*layers\.([1-9]\d*)\.mlp$")):
    def install(module, name):
        def report_experts(experts):
            prefetch_mngr.report_one_layer(module._layer_id, experts)
            return experts
        module.report_experts = report_experts
    recursive_traverse_childrens(model, install, filter)


def add_hook_to_experts(model, prefetch_mngr, filter=_EXPERT):
    hook = hooks.ExpertHook(prefetch_mngr)
    recursive_traverse_childrens(model, lambda m, n: hooks.add_hook_to_module(m, hook), filter)


def add_hook_to_moe_attns(model, prefetch_mngr, filter):
    hook = hooks.MoEAttnHook(prefetch_mngr)
    recursive_traverse_childrens(model, lambda m, n: hooks.add_hook_to_module(m, hook), filter)


def add_hook_to_moe_layers(model, prefetch_mngr, filter):
    hook = hooks.MoeLayerHook(prefetch_mngr)
    recursive_traverse_childrens(model, lambda m, n: hooks.add_hook_to_module(m, hook), filter)


def add_hook_to_some_modules(model, hook, filter=RegexFilter(r".*"), append=False):
    recursive_traverse_childrens(model, lambda m, n: hooks.add_hook_to_module(m, hook, append), filter)


def install_fused_moe_forward(model, prefetch_mngr, filter, device="cuda"):
    """Replaces the forward of every MoE block that `filter` selects by the fused device path."""
    from ..moe_block import install_fused_forward
    cache = prefetch_mngr.metas.cache
    config = getattr(model, "config", None)

    def install(module, name):
        if not (hasattr(module, "experts") and hasattr(module, "gate")):
            raise ValueError(f"{name} matches the MoE block filter but has no `experts` and `gate`: it cannot be "
                             "given the fused forward (pass fused=False to keep the model's own expert loop)")
        install_fused_forward(module, cache, module._layer_id, device, config)
    recursive_traverse_childrens(model, install, filter)


def repo_folder_name(repo_id: str, repo_type: str = "model") -> str:
    """huggingface_hub's cache folder name of a repo, e.g. models--org--name."""
    return "--".join([f"{repo_type}s", *repo_id.split("/")])


# ----------------------------------------------------------------------------- inject_model
def inject_model(model: torch.nn.Module, model_id=None, num_moe_layer: int = None, num_expert_per_layer: int = None,
                 num_expert_per_token: int = None, cache_rate: float = None, num_predict_expert_per_layer: int = None,
                 reorder_experts: bool = None, early_preempt: bool = None, chunk_prefetch: bool = None,
                 predict_input_mode=None, predictor_type: str = None, predictor_model_path: str = None,
                 layer_predict_interval=None, layer_predict_max_window=None,
                 layer_predict_replace_first_input_with_last_output=False, limit_layer_0_window=None,
                 limit_layer_0_num_predict=None, max_prefetch_layer_distance=None, cache_only=False,
                 per_layer_cache: bool = None, promote_hit_in_prefetch: bool = None, cache_policy: str = None,
                 cache_device="cuda", pin_memory: bool = True, module_trace_event: bool = False,
                 enable_model_timer: bool = True, trace_event: bool = False, cache_trace_path: str = None,
                 launch_now=True, fused: bool = True, expert_meta_parser=None, expert_name_filter=None,
                 moe_mlp_name_filter=None, moe_layer_name_filter=None, **kwargs):
    """Attaches the expert cache to `model` (see the module docstring). Returns the PrefetchMngr."""
    if kwargs:
        print("warning, unused kwargs", kwargs)
    model_id = model.config._name_or_path if model_id is None else model_id
    if num_moe_layer is None or expert_name_filter is None:
        m = auto_infer_model_metas(model_id, return_dict=False)
        num_moe_layer = m.num_moe_layer if num_moe_layer is None else num_moe_layer
        num_expert_per_layer = m.num_expert_per_layer if num_expert_per_layer is None else num_expert_per_layer
        num_expert_per_token = m.num_expert_per_token if num_expert_per_token is None else num_expert_per_token
        expert_meta_parser = expert_meta_parser or m.expert_meta_parser
        expert_name_filter = expert_name_filter or m.expert_name_filter
        moe_mlp_name_filter = moe_mlp_name_filter or m.moe_mlp_name_filter
        moe_layer_name_filter = moe_layer_name_filter or m.moe_layer_name_filter

    meta = cpp_worker.ModuleMeta(num_moe_layer, num_expert_per_layer)
    meta.model_arch_string = model_id
    meta.num_expert_per_token = num_expert_per_token

    found = []
    recursive_traverse_childrens(model, lambda mod, n: found.append(mod), expert_name_filter)
    if not found:
        raise ValueError("no expert module matches the expert name filter")
    meta.init_param_list([k for k, _ in _expert_tensors(found[0])])

    meta.init_from_map({
        "model_arch_string": str(model_id), "num_expert_per_token": str(num_expert_per_token),
        "cache_rate": str(cache_rate), "num_predict_expert_per_layer": str(num_predict_expert_per_layer),
        "reorder_experts": str(reorder_experts), "early_preempt": str(early_preempt),
        "chunk_prefetch": str(chunk_prefetch), "predict_input_mode": str(predict_input_mode),
        "predictor_type": str(predictor_type), "predictor_model_path": str(predictor_model_path),
        "layer_predict_interval": str(layer_predict_interval), "layer_predict_max_window": str(layer_predict_max_window),
        "cross_token_pred": str(layer_predict_replace_first_input_with_last_output),
        "limit_layer_0_window": str(limit_layer_0_window), "limit_layer_0_num_predict": str(limit_layer_0_num_predict),
        "max_prefetch_layer_distance": str(max_prefetch_layer_distance), "cache_only": str(cache_only),
        "per_layer_cache": str(per_layer_cache), "promote_hit_in_prefetch": str(promote_hit_in_prefetch),
        "cache_policy": str(cache_policy)})
    meta.handle_uninited_configs()

    if isinstance(cache_device, str) and ":" in cache_device:
        torch.cuda.set_device(torch.device(cache_device))
    elif isinstance(cache_device, int):
        torch.cuda.set_device(cache_device)
    model_loader = cpp_worker.ModelLoader(meta)
    predictor = cpp_worker.PredictorBase.create(meta)
    prefetch_mngr = cpp_worker.PrefetchMngr(meta, model_loader, predictor)
    torch.cuda.set_stream(torch.cuda.ExternalStream(prefetch_mngr.compute_stream))

    add_metadata_to_submodules(model, expert_meta_parser)
    register_expert_params(model, model_loader, expert_name_filter)
    prefetch_mngr.init_gpu_mem_buffer()
    if fused:
        install_fused_moe_forward(model, prefetch_mngr, moe_mlp_name_filter, "cuda")
    replace_expert_param_reference(model, model_loader, expert_name_filter)
    replace_mlp_report_experts(model, prefetch_mngr, predictor, num_moe_layer, num_expert_per_layer,
                               num_predict_expert_per_layer, moe_mlp_name_filter)
    predictor.load_model()

    if meta.cache_policy == "min":
        load = lambda f: torch.load(os.path.join(cache_trace_path, f))  # noqa: E731
        prefetch_mngr.cache.cache_oracle.load_from_tensor(
            load("entry_to_metas.pt"), load("prefill_expert_len.pt"), load("prefill_expert_selection.pt"),
            load("decode_expert_selection.pt"))

    if not fused:
        add_hook_to_experts(model, prefetch_mngr, expert_name_filter)
    add_hook_to_moe_layers(model, prefetch_mngr, moe_layer_name_filter)
    attach_prefetch_mngr_to_all_module(model, prefetch_mngr)

    if trace_event:
        os.environ["SPARSE_CACHE_ENABLE_TRACE"] = "1"
        prefetch_mngr.reload_env()
        if module_trace_event:
            add_hook_to_some_modules(model, hooks.TraceEventHook(), append=True)
    if enable_model_timer:
        add_hook_to_some_modules(model, hooks.TimingHook(prefetch_mngr), filter=RegexFilter("^$"), append=True)
    if pin_memory:
        model_loader.pin_memory()
    model._prefetch_mngr = prefetch_mngr
    if launch_now:
        launch(model)
    return prefetch_mngr


def launch(model: torch.nn.Module):
    prefetch_mngr = model._prefetch_mngr
    prefetch_mngr.launch_thread()
    torch.set_num_threads(8)
    return prefetch_mngr


# ----------------------------------------------------------------------------- transformers loaders
def _loader_is_static(cls) -> bool:
    """transformers 5.x: `_load_pretrained_model(model, state_dict, checkpoint_files, load_config, ...)`
    is a staticmethod and the device map travels inside `load_config`; 4.x: a classmethod
    `(cls, model, ..., device_map=...)` that returns the model first."""
    import inspect
    return isinstance(inspect.getattr_static(cls, "_load_pretrained_model"), staticmethod)


def _single_device(device_map):
    if isinstance(device_map, (str, int, torch.device)):
        device_map = {"": device_map}
    assert device_map is not None and len(device_map) == 1 and "" in device_map, "only support single device"
    return device_map[""]


def _wrap_loader(PreTrainedModel, after_load):
    """Replaces `_load_pretrained_model` by one that loads every tensor on the CPU and then calls
    `after_load(model, device)`. Works for both loader generations."""
    import dataclasses
    old = PreTrainedModel._old_load_pretrained_model
    if _loader_is_static(PreTrainedModel):
        @staticmethod
        @functools.wraps(old)
        def load_pretrained_model(model, state_dict, checkpoint_files, load_config, *args, **kwargs):
            device = "cpu"
            if load_config.device_map is not None:     # without one the static loader stays on the CPU anyway
                device = _single_device(load_config.device_map)
                load_config = dataclasses.replace(load_config, device_map={"": "cpu"})
            ret = old(model, state_dict, checkpoint_files, load_config, *args, **kwargs)
            model._promoe_target_device = device
            after_load(model, device)
            return ret
    else:
        @classmethod
        @functools.wraps(old.__func__)
        def load_pretrained_model(cls, *args, **kwargs):
            device = _single_device(kwargs.get("device_map"))
            kwargs["device_map"] = {"": "cpu"}
            ret = old.__func__(cls, *args, **kwargs)
            model = ret[0] if isinstance(ret, tuple) else ret
            model._promoe_target_device = device
            after_load(model, device)
            return ret
    PreTrainedModel._load_pretrained_model = load_pretrained_model


def _inject_loaded(model, device="cuda", **sparse_cache_kwargs):
    """Per-expert modules (the reference's fork layout): inject_model. Fused expert tensors (stock
    transformers 5.x): the adapter for that layout, which takes the subset of the options it knows."""
    from ..hf_fused import find_moe_blocks, inject_hf_fused_model
    if find_moe_blocks(model):
        known = ("cache_rate", "cache_policy", "num_predict_expert_per_layer", "reorder_experts", "early_preempt",
                 "chunk_prefetch", "per_layer_cache", "promote_hit_in_prefetch")
        opts = {k: v for k, v in sparse_cache_kwargs.items() if k in known and v is not None}
        inject_hf_fused_model(model, device=device, **opts)
        model._promoe_fused_layout = True
    else:
        inject_model(model, **sparse_cache_kwargs, launch_now=False)


def hack_transformers(**sparse_cache_kwargs):
    """Makes `from_pretrained` load the checkpoint on the CPU, inject the cache, then launch
    (utils/__init__.py:369-392). The injection runs once the model is complete: inside the loader for
    the 4.x classmethod (as the reference does), after `from_pretrained` has finalised the weights
    (tied weights, missing-key initialisation) for the 5.x static loader. There the caller's
    single-device `device_map` is taken out of the call (5.x loads on the CPU without one, and needs
    no accelerate for that) and the rest of the model is moved to that device after the injection."""
    from transformers.modeling_utils import PreTrainedModel
    if hasattr(PreTrainedModel, "_old_load_pretrained_model"):
        return
    static = _loader_is_static(PreTrainedModel)
    PreTrainedModel._old_load_pretrained_model = inspect_static(PreTrainedModel, "_load_pretrained_model")
    PreTrainedModel._old_from_pretrained = inspect_static(PreTrainedModel, "from_pretrained")
    if not static:
        _wrap_loader(PreTrainedModel, lambda model, device: _inject_loaded(model, device, **sparse_cache_kwargs))
    old_from = PreTrainedModel._old_from_pretrained.__func__

    @classmethod
    @functools.wraps(old_from)
    def from_pretrained(cls, *args, **kwargs):
        if static:
            device = _single_device(kwargs.pop("device_map", None))
        out = old_from(cls, *args, **kwargs)
        model = out[0] if isinstance(out, tuple) else out
        if static:
            _inject_loaded(model, device, **sparse_cache_kwargs)
            model.to(device)
        if not getattr(model, "_promoe_fused_layout", False):
            launch(model)
        return out

    PreTrainedModel.from_pretrained = from_pretrained


def unhack_transformers():
    """Restores the loaders that hack_transformers / hack_transformers_um replaced."""
    from transformers.modeling_utils import PreTrainedModel
    if hasattr(PreTrainedModel, "_old_load_pretrained_model"):
        PreTrainedModel._load_pretrained_model = inspect_static(PreTrainedModel, "_old_load_pretrained_model")
        del PreTrainedModel._old_load_pretrained_model
    if hasattr(PreTrainedModel, "_old_from_pretrained"):
        PreTrainedModel.from_pretrained = inspect_static(PreTrainedModel, "_old_from_pretrained")
        del PreTrainedModel._old_from_pretrained


def inspect_static(cls, name):
    """The attribute as stored on the class (keeps staticmethod / classmethod wrappers)."""
    import inspect
    return inspect.getattr_static(cls, name)


def inject_model_um(model, model_id=None):
    """The reference's unified-memory baseline; here experts are kept in pinned host memory
    (see cpp_worker.to_um)."""
    model_id = model.config._name_or_path if model_id is None else model_id
    m = auto_infer_model_metas(model_id, return_dict=False)
    add_metadata_to_submodules(model, m.expert_meta_parser)

    def per_expert(module, name):
        def per_leaf(leaf, leaf_name):
            for n, v in list(leaf.named_parameters(recurse=False)):
                leaf._parameters[n] = torch.nn.Parameter(cpp_worker.to_um(v), requires_grad=False)
            for n, v in list(leaf.named_buffers(recurse=False)):
                if param_buffer_name_to_prefetch(n):
                    leaf._buffers[n] = cpp_worker.to_um(v)
        recursive_traverse_childrens_leaf_only(module, per_leaf)
    recursive_traverse_childrens(model, per_expert, m.expert_name_filter)


def hack_transformers_um():
    from transformers.modeling_utils import PreTrainedModel
    if hasattr(PreTrainedModel, "_old_load_pretrained_model"):
        return
    PreTrainedModel._old_load_pretrained_model = inspect_static(PreTrainedModel, "_load_pretrained_model")
    _wrap_loader(PreTrainedModel, lambda model, device: inject_model_um(model))
