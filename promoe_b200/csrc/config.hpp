// Runtime configuration of the expert cache: the same keys, aliases, defaults and
// environment overrides as the reference's ModuleMeta (src/cpp_worker/utils.hpp:127-192,
// src/cpp_worker/utils.cpp:54-273), held as plain data with string get/set access.
#pragma once
#include <map>
#include <string>
#include <vector>

namespace pm {

struct Config {
  int num_layer = 0;
  int num_expert = 0;
  std::string model_arch_string;
  int num_expert_per_token = 0;

  float cache_rate = 0.5f;
  int num_predict_expert_per_layer = -1;
  bool reorder_experts = false;
  bool early_preempt = false;
  bool chunk_prefetch = false;

  std::string predict_input_mode = "moe_layer_logits";
  std::string predictor_type = "sep";
  std::string predictor_model_path;
  int layer_predict_interval = 1;
  int layer_predict_max_window = 3;
  bool cross_token_pred = false;  // layer_predict_replace_first_input_with_last_output

  int limit_layer_0_window = -1;
  int limit_layer_0_num_predict = -1;

  int max_prefetch_layer_distance = -1;
  bool cache_only = false;
  bool per_layer_cache = true;
  bool promote_hit_in_prefetch = true;
  std::string cache_policy = "lru";
  int predict_input_reuse_distance_max = 10;
  int predict_input_decay = 2;

  // Not reference keys: how this library behaves around the policy.
  bool predict_from_moe_input = false;  // run the predictor inside pm_moe_forward on its input

  std::vector<std::string> param_names;
  int num_per_expert_param() const { return (int)param_names.size(); }

  // Parses "key=value" lines. Returns "" on success, else the error text.
  std::string init_from_text(const std::string& kv);
  // Fills values the map left open (and applies the environment overrides).
  void resolve_defaults();
  // String access to one resolved value; false if the key is unknown.
  bool get(const std::string& key, std::string* out) const;
  std::string set(const std::string& key, const std::string& value);

  // For every source index 0..num_layer the half-open range of layers it predicts
  // (src/cpp_worker/predictor.cpp:8-46).
  std::vector<std::pair<int, int>> predict_layer_mapping() const;
};

}  // namespace pm
