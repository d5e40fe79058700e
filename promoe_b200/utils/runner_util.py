"""Command-line flags for the cache configuration (counterpart of the reference's
src/sparse_llm_cache/utils/runner_util.py:18-55: the same flag names, so sweep scripts written
for the reference parse unchanged). parse_args() returns a dict ready for inject_model(**cfg)."""
from __future__ import annotations

import argparse


def _flag(v: str) -> bool:
    return str(v).lower() in ("1", "true", "on", "yes")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_id", type=str, default=None)
    ap.add_argument("--cache_rate", "--moe_cache_rate", dest="cache_rate", type=float, default=None)
    ap.add_argument("--cache_policy", "--moe_cache_policy", dest="cache_policy", type=str, default=None)
    ap.add_argument("--num_predict_expert_per_layer", "--num_predict", dest="num_predict_expert_per_layer",
                    type=int, default=None)
    ap.add_argument("--reorder_experts", type=_flag, default=None)
    ap.add_argument("--early_preempt", type=_flag, default=None)
    ap.add_argument("--chunk_prefetch", type=_flag, default=None)
    ap.add_argument("--predict_input_mode", type=str, default=None)
    ap.add_argument("--predictor_type", type=str, default=None)
    ap.add_argument("--predictor_model_path", "--pred_model_path", dest="predictor_model_path", type=str, default=None)
    ap.add_argument("--layer_predict_interval", "--predict_interval", dest="layer_predict_interval", type=int, default=None)
    ap.add_argument("--layer_predict_max_window", "--predict_window", dest="layer_predict_max_window", type=int, default=None)
    ap.add_argument("--layer_predict_replace_first_input_with_last_output", "--cross_token_pred",
                    dest="layer_predict_replace_first_input_with_last_output", type=_flag, default=False)
    ap.add_argument("--limit_layer_0_window", type=int, default=None)
    ap.add_argument("--limit_layer_0_num_predict", type=int, default=None)
    ap.add_argument("--max_prefetch_layer_distance", type=int, default=None)
    ap.add_argument("--cache_only", type=_flag, default=False)
    ap.add_argument("--per_layer_cache", type=_flag, default=None)
    ap.add_argument("--promote_hit_in_prefetch", type=_flag, default=None)
    ap.add_argument("--cache_trace_path", type=str, default=None)
    ap.add_argument("--trace_event", type=_flag, default=False)
    ap.add_argument("--dataset", type=str, default="chatgpt-prompts-small")
    return ap


def parse_args(argv=None) -> dict:
    ns, _ = build_parser().parse_known_args(argv)
    cfg = vars(ns)
    cfg.pop("dataset", None)
    if cfg.get("model_id") is None:
        cfg.pop("model_id")
    return cfg
