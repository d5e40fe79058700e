#include "config.hpp"

#include <algorithm>
#include <cstdlib>
#include <sstream>

namespace pm {
namespace {

std::string lower(std::string s) {
  std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return (char)std::tolower(c); });
  return s;
}

// "on", "true" or "1" in any case (src/cpp_worker/utils.hpp:448-451).
bool is_on(const std::string& s) {
  std::string l = lower(s);
  return l == "on" || l == "true" || l == "1";
}

bool unset(const std::string& v) { return v == "None" || v.empty(); }

const std::map<std::string, std::string>& aliases() {
  // src/cpp_worker/utils.cpp:147-172
  static const std::map<std::string, std::string> a = {
      {"cross_token_pred", "layer_predict_replace_first_input_with_last_output"},
      {"predict_using_last_token_output", "layer_predict_replace_first_input_with_last_output"},
      {"num_predict", "num_predict_expert_per_layer"},
      {"predict_interval", "layer_predict_interval"},
      {"predict_window", "layer_predict_max_window"},
      {"moe_cache_policy", "cache_policy"},
      {"moe_cache_rate", "cache_rate"},
      {"pred_model_path", "predictor_model_path"},
  };
  return a;
}

const char* kPolicies[] = {"lru", "fifo", "static-1", "static-2", "nn", "min"};
const char* kInputModes[] = {"no_predict", "one_token", "decode_cumsum", "last_use_distance",
                             "weighted_decode_cumsum", "first_moe_attn_input_logits",
                             "moe_attn_input_logits", "moe_layer_logits"};

bool parse_int(const std::string& s, int* out) {
  try {
    size_t used = 0;
    *out = std::stoi(s, &used);
    return used > 0;
  } catch (...) {
    return false;
  }
}

bool parse_float(const std::string& s, float* out) {
  try {
    *out = std::stof(s);
    return true;
  } catch (...) {
    return false;
  }
}

}  // namespace

std::string Config::init_from_text(const std::string& kv) {
  std::map<std::string, std::string> m;
  std::istringstream in(kv);
  std::string line;
  while (std::getline(in, line)) {
    if (line.empty()) continue;
    size_t eq = line.find('=');
    if (eq == std::string::npos) return "config line without '=': " + line;
    std::string key = line.substr(0, eq), val = line.substr(eq + 1);
    std::replace(key.begin(), key.end(), '-', '_');
    auto al = aliases().find(key);
    if (al != aliases().end()) key = al->second;
    if (m.count(key)) return "duplicate config key " + key;
    m[key] = val;
  }
  std::string err;
  auto take = [&](const char* key, std::string* v) -> bool {  // true if a usable value was present
    auto it = m.find(key);
    if (it == m.end()) return false;
    std::string val = it->second;
    m.erase(it);
    if (unset(val)) return false;
    *v = val;
    return true;
  };
  auto take_int = [&](const char* key, int* dst) {
    std::string v;
    if (take(key, &v) && !parse_int(v, dst)) err = std::string("invalid key ") + key + " with value " + v;
  };
  auto take_float = [&](const char* key, float* dst) {
    std::string v;
    if (take(key, &v) && !parse_float(v, dst)) err = std::string("invalid key ") + key + " with value " + v;
  };
  auto take_bool = [&](const char* key, bool* dst) {
    std::string v;
    if (take(key, &v)) *dst = is_on(v);
  };
  auto take_str = [&](const char* key, std::string* dst) {
    std::string v;
    if (take(key, &v)) *dst = v;
  };

  take_str("model_arch_string", &model_arch_string);
  {
    std::string v;
    if (!take("num_expert_per_token", &v)) return "required key num_expert_per_token not found";
    if (!parse_int(v, &num_expert_per_token)) return "invalid key num_expert_per_token with value " + v;
  }
  take_float("cache_rate", &cache_rate);
  take_int("num_predict_expert_per_layer", &num_predict_expert_per_layer);
  if (num_predict_expert_per_layer == -1) num_predict_expert_per_layer = num_expert_per_token;
  reorder_experts = early_preempt = chunk_prefetch = (num_predict_expert_per_layer > 0);
  take_bool("reorder_experts", &reorder_experts);
  take_bool("early_preempt", &early_preempt);
  take_bool("chunk_prefetch", &chunk_prefetch);

  take_str("predict_input_mode", &predict_input_mode);
  if (std::find(std::begin(kInputModes), std::end(kInputModes), predict_input_mode) == std::end(kInputModes))
    predict_input_mode = "no_predict";  // the reference's map lookup yields its zero value
  take_str("predictor_type", &predictor_type);
  if (predictor_type != "sep" && predictor_type != "legacy") predictor_type = "legacy";
  take_str("predictor_model_path", &predictor_model_path);
  take_int("layer_predict_interval", &layer_predict_interval);
  take_int("layer_predict_max_window", &layer_predict_max_window);
  take_bool("layer_predict_replace_first_input_with_last_output", &cross_token_pred);
  take_int("limit_layer_0_window", &limit_layer_0_window);
  take_int("limit_layer_0_num_predict", &limit_layer_0_num_predict);
  take_int("max_prefetch_layer_distance", &max_prefetch_layer_distance);
  take_bool("cache_only", &cache_only);
  take_bool("per_layer_cache", &per_layer_cache);
  take_bool("promote_hit_in_prefetch", &promote_hit_in_prefetch);
  take_str("cache_policy", &cache_policy);
  take_int("predict_input_reuse_distance_max", &predict_input_reuse_distance_max);
  take_int("predict_input_decay", &predict_input_decay);
  take_bool("predict_from_moe_input", &predict_from_moe_input);
  if (!err.empty()) return err;
  if (std::find_if(std::begin(kPolicies), std::end(kPolicies),
                   [&](const char* p) { return cache_policy == p; }) == std::end(kPolicies))
    return "unknown cache_policy " + cache_policy;
  if (layer_predict_interval <= 0) return "layer_predict_interval must be positive";
  if (!m.empty()) {
    std::string msg = "unrecognized configs:";
    for (auto& p : m) msg += " " + p.first + "=" + p.second;
    return msg;
  }
  return "";
}

void Config::resolve_defaults() {
  if (max_prefetch_layer_distance == -1) max_prefetch_layer_distance = num_layer - 1;
  model_arch_string = lower(model_arch_string);
  if (limit_layer_0_window == -1)
    limit_layer_0_window = (model_arch_string.find("deepseek") != std::string::npos) ? layer_predict_max_window : 1;
}

std::vector<std::pair<int, int>> Config::predict_layer_mapping() const {
  const int L = num_layer;
  std::vector<int> stop_of(L + 1, 0);
  int stop = 0;
  for (int l = 0; l < L; l += layer_predict_interval) {
    int window = (l == 0 && limit_layer_0_window != -1) ? limit_layer_0_window : layer_predict_max_window;
    stop_of[l] = stop;
    stop_of[l + 1] = std::min((l % L) + window, L);
    stop = stop_of[l + 1];
  }
  for (int l = 1; l <= L; ++l) stop_of[l] = std::max(stop_of[l], stop_of[l - 1]);
  std::vector<std::pair<int, int>> out(L + 1, {0, 0});
  for (int l = 0; l < L; ++l) out[l] = {stop_of[l], stop_of[l + 1]};
  if (cross_token_pred) {
    out[L] = out[0];
    out[0] = {0, 0};
  }
  return out;
}

bool Config::get(const std::string& key, std::string* out) const {
  auto b = [](bool v) { return std::string(v ? "true" : "false"); };
  std::ostringstream os;
  if (key == "num_layer") os << num_layer;
  else if (key == "num_expert") os << num_expert;
  else if (key == "model_arch_string") os << model_arch_string;
  else if (key == "num_expert_per_token") os << num_expert_per_token;
  else if (key == "cache_rate") os << cache_rate;
  else if (key == "num_predict_expert_per_layer") os << num_predict_expert_per_layer;
  else if (key == "reorder_experts") os << b(reorder_experts);
  else if (key == "early_preempt") os << b(early_preempt);
  else if (key == "chunk_prefetch") os << b(chunk_prefetch);
  else if (key == "predict_input_mode") os << predict_input_mode;
  else if (key == "predictor_type") os << predictor_type;
  else if (key == "predictor_model_path") os << predictor_model_path;
  else if (key == "layer_predict_interval") os << layer_predict_interval;
  else if (key == "layer_predict_max_window") os << layer_predict_max_window;
  else if (key == "layer_predict_replace_first_input_with_last_output" || key == "cross_token_pred") os << b(cross_token_pred);
  else if (key == "limit_layer_0_window") os << limit_layer_0_window;
  else if (key == "limit_layer_0_num_predict") os << limit_layer_0_num_predict;
  else if (key == "max_prefetch_layer_distance") os << max_prefetch_layer_distance;
  else if (key == "cache_only") os << b(cache_only);
  else if (key == "per_layer_cache") os << b(per_layer_cache);
  else if (key == "promote_hit_in_prefetch") os << b(promote_hit_in_prefetch);
  else if (key == "cache_policy") os << cache_policy;
  else if (key == "predict_input_reuse_distance_max") os << predict_input_reuse_distance_max;
  else if (key == "predict_input_decay") os << predict_input_decay;
  else if (key == "predict_from_moe_input") os << b(predict_from_moe_input);
  else if (key == "num_per_expert_param") os << num_per_expert_param();
  else return false;
  *out = os.str();
  return true;
}

std::string Config::set(const std::string& key, const std::string& value) {
  auto as_int = [&](int* dst) -> std::string {
    return parse_int(value, dst) ? "" : "invalid value " + value + " for " + key;
  };
  if (key == "num_predict_expert_per_layer") return as_int(&num_predict_expert_per_layer);
  if (key == "num_expert_per_token") return as_int(&num_expert_per_token);
  if (key == "max_prefetch_layer_distance") return as_int(&max_prefetch_layer_distance);
  if (key == "layer_predict_interval") return as_int(&layer_predict_interval);
  if (key == "layer_predict_max_window") return as_int(&layer_predict_max_window);
  if (key == "limit_layer_0_window") return as_int(&limit_layer_0_window);
  if (key == "limit_layer_0_num_predict") return as_int(&limit_layer_0_num_predict);
  if (key == "reorder_experts") { reorder_experts = is_on(value); return ""; }
  if (key == "early_preempt") { early_preempt = is_on(value); return ""; }
  if (key == "chunk_prefetch") { chunk_prefetch = is_on(value); return ""; }
  if (key == "per_layer_cache") { per_layer_cache = is_on(value); return ""; }
  if (key == "promote_hit_in_prefetch") { promote_hit_in_prefetch = is_on(value); return ""; }
  if (key == "cache_only") { cache_only = is_on(value); return ""; }
  if (key == "predict_from_moe_input") { predict_from_moe_input = is_on(value); return ""; }
  if (key == "layer_predict_replace_first_input_with_last_output" || key == "cross_token_pred") {
    cross_token_pred = is_on(value);
    return "";
  }
  if (key == "model_arch_string") { model_arch_string = value; return ""; }
  if (key == "cache_policy") { cache_policy = value; return ""; }
  if (key == "cache_rate") return parse_float(value, &cache_rate) ? "" : "invalid value " + value + " for cache_rate";
  return "unknown or read-only config key " + key;
}

}  // namespace pm
