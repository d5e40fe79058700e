"""Forward-wrapping hooks (counterpart of the reference's src/sparse_llm_cache/utils/hooks.py).

`add_hook_to_module` replaces a module's `forward` with a wrapper that calls
`hook.pre_forward(module, *args, **kwargs)` before and `hook.post_forward(module, output)`
after the original forward (the accelerate-style protocol the reference uses, hooks.py:8-170).
The concrete hooks make the same manager calls as the reference's:
  ExpertHook    -> report_one_expert / one_expert_done          (hooks.py:187-198)
  MoeLayerHook  -> report_moe_layer_logits / one_moe_layer_done (hooks.py:202-223)
  MoEAttnHook   -> report_moe_attn_logits                       (hooks.py:173-185)
  TimingHook, TraceEventHook                                    (hooks.py:227-253)
Modules whose forward is the fused block (promoe_b200.moe_block) do not need ExpertHook: the
library performs those steps inside one call.
"""
from __future__ import annotations

import functools

import torch

from .. import cpp_worker


class ModelHook:
    """Callbacks around a module's forward. `no_grad` runs the forward without autograd."""
    no_grad = True

    def init_hook(self, module):
        return module

    def pre_forward(self, module, *args, **kwargs):
        return args, kwargs

    def post_forward(self, module, output):
        return output

    def detach_hook(self, module):
        return module


class SequentialHook(ModelHook):
    """Several hooks as one: pre in order, post in reverse order."""

    def __init__(self, *hooks):
        self.hooks = hooks

    def init_hook(self, module):
        for h in self.hooks:
            module = h.init_hook(module)
        return module

    def pre_forward(self, module, *args, **kwargs):
        for h in self.hooks:
            args, kwargs = h.pre_forward(module, *args, **kwargs)
        return args, kwargs

    def post_forward(self, module, output):
        for h in reversed(self.hooks):
            output = h.post_forward(module, output)
        return output

    def detach_hook(self, module):
        for h in self.hooks:
            module = h.detach_hook(module)
        return module


def _wrap(module, method_name, hook_attr, old_attr, hook, append):
    existing = getattr(module, hook_attr, None)
    if append and existing is not None:
        hook = SequentialHook(existing, hook)
    if not hasattr(module, old_attr):
        setattr(module, old_attr, getattr(module, method_name))
    original = getattr(module, old_attr)
    module = hook.init_hook(module)
    setattr(module, hook_attr, hook)

    @functools.wraps(original)
    def wrapped(*args, **kwargs):
        h = getattr(module, hook_attr)
        args, kwargs = h.pre_forward(module, *args, **kwargs)
        if h.no_grad:
            with torch.no_grad():
                out = original(*args, **kwargs)
        else:
            out = original(*args, **kwargs)
        return h.post_forward(module, out)

    setattr(module, method_name, wrapped)
    return module


def add_hook_to_module(module: torch.nn.Module, hook: ModelHook, append: bool = False):
    """Wraps `module.forward`; a second call replaces the hook unless append=True chains it."""
    return _wrap(module, "forward", "_hf_hook", "_old_forward", hook, append)


def add_hook_to_module_custom_method(module, hook: ModelHook, method_name: str, hook_attr_name: str, append=False):
    """Same for another method (the reference wraps quantised layers' post_init this way)."""
    return _wrap(module, method_name, hook_attr_name, f"_old_{method_name}", hook, append)


def remove_hook_from_module(module: torch.nn.Module, recurse: bool = False):
    if hasattr(module, "_hf_hook"):
        module._hf_hook.detach_hook(module)
        del module._hf_hook
    if hasattr(module, "_old_forward"):
        module.forward = module._old_forward
        del module._old_forward
    if recurse:
        for child in module.children():
            remove_hook_from_module(child, True)
    return module


class ExpertHook(ModelHook):
    def __init__(self, prefetch_mngr):
        self.prefetch_mngr = prefetch_mngr

    def pre_forward(self, module, *args, **kwargs):
        self.prefetch_mngr.report_one_expert(module._layer_id, module._expert_id)
        return args, kwargs

    def post_forward(self, module, output):
        self.prefetch_mngr.one_expert_done(module._layer_id, module._expert_id)
        return output


class MoeLayerHook(ModelHook):
    """Reports the hidden states entering a decoder layer (index l) and leaving it (index l+1)."""

    def __init__(self, prefetch_mngr, extract_logits_from_input=None, extract_logits_from_output=None):
        self.prefetch_mngr = prefetch_mngr
        self.extract_logits_from_input = extract_logits_from_input or (lambda *a, **k: a[0] if a else k["hidden_states"])
        self.extract_logits_from_output = extract_logits_from_output or (
            lambda out: out[0] if isinstance(out, (tuple, list)) else out)

    def pre_forward(self, module, *args, **kwargs):
        if module._layer_id == 0:
            self.prefetch_mngr.report_moe_layer_logits(0, self.extract_logits_from_input(*args, **kwargs))
        return args, kwargs

    def post_forward(self, module, output):
        self.prefetch_mngr.report_moe_layer_logits(module._layer_id + 1, self.extract_logits_from_output(output))
        self.prefetch_mngr.one_moe_layer_done(module._layer_id)
        return output


class MoEAttnHook(ModelHook):
    def __init__(self, prefetch_mngr):
        self.prefetch_mngr = prefetch_mngr

    def pre_forward(self, module, *args, **kwargs):
        self.prefetch_mngr.report_moe_attn_logits(module._layer_id, kwargs["hidden_states"])
        return args, kwargs


class TraceEventHook(ModelHook):
    def __init__(self):
        self.open_spans = []

    def pre_forward(self, module, *args, **kwargs):
        span = cpp_worker.TraceEventGuard()
        span.init(cpp_worker.kPythonMain, getattr(module, "_prefix", type(module).__name__))
        self.open_spans.append(span)
        return args, kwargs

    def post_forward(self, module, output):
        self.open_spans.pop().release()
        return output


class TimingHook(ModelHook):
    def __init__(self, prefetch_mngr):
        self.timing_guard = prefetch_mngr.build_timer()

    def pre_forward(self, module, *args, **kwargs):
        self.timing_guard.init(cpp_worker.kModelForward)
        return args, kwargs

    def post_forward(self, module, output):
        self.timing_guard.release()
        return output
