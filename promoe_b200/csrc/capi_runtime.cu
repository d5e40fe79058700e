// C-ABI entry points of the stateful part: configuration, expert registry, slab, cache policy,
// fused layer forward.
#include <cstring>
#include <sstream>

#include "runtime.hpp"

using namespace pm;

namespace {

int need(pm_ctx* c) { return c == nullptr ? fail(PM_ERR_INVALID, "null context") : PM_OK; }

int from(const std::string& err, int code = PM_ERR_STATE) { return err.empty() ? PM_OK : fail(code, err); }

// Which registered tensor is the gate / up / down matrix (and, for uint4 experts, which hold the
// scale/zero pairs), judged from the tensor names the reference collects from the first expert
// module (src/sparse_llm_cache/utils/__init__.py:250-261).
void assign_roles(pm_ctx* c) {
  const std::vector<std::string>& names = c->cfg.param_names;
  auto find = [&](std::initializer_list<const char*> keys, bool quant_meta) {
    for (size_t i = 0; i < names.size(); ++i) {
      const std::string& n = names[i];
      bool is_meta = n.find("scale") != std::string::npos || n.find("zero") != std::string::npos;
      if (is_meta != quant_meta) continue;
      for (const char* k : keys)
        if (n.find(k) != std::string::npos) return (int)i;
    }
    return -1;
  };
  int g = find({"gate_proj", "w1"}, false), u = find({"up_proj", "w3"}, false), d = find({"down_proj", "w2"}, false);
  if (g >= 0 && u >= 0 && d >= 0) {
    c->role_gate = g;
    c->role_up = u;
    c->role_down = d;
  }
  c->role_qgate = find({"gate_proj", "w1"}, true);
  c->role_qup = find({"up_proj", "w3"}, true);
  c->role_qdown = find({"down_proj", "w2"}, true);
}

}  // namespace

extern "C" {

int pm_ctx_create(pm_ctx** out, int num_layer, int num_expert, const char* config_kv) {
  if (out == nullptr) return fail(PM_ERR_INVALID, "null output pointer");
  *out = nullptr;
  if (num_layer <= 0 || num_expert <= 0 || num_expert > 256)
    return fail(PM_ERR_INVALID, "num_layer must be positive and num_expert in [1, 256]");
  std::unique_ptr<pm_ctx> c(new pm_ctx());
  c->cfg.num_layer = num_layer;
  c->cfg.num_expert = num_expert;
  std::string err = c->cfg.init_from_text(config_kv ? config_kv : "");
  if (!err.empty()) return fail(PM_ERR_INVALID, err);
  c->cfg.resolve_defaults();
  c->eng.reset(new CacheEngine(c->cfg));
  c->layers.resize(num_layer);
  c->predictors.resize((size_t)(num_layer + 1) * num_layer);
  c->last_ids.resize(num_layer);
  c->last_w.resize(num_layer);
  *out = c.release();
  return PM_OK;
}

int pm_ctx_destroy(pm_ctx* ctx) {
  delete ctx;
  return PM_OK;
}

int pm_ctx_get(pm_ctx* ctx, const char* key, char* buf, size_t cap) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!key || !buf || cap == 0) return fail(PM_ERR_INVALID, "null argument");
  std::string v;
  std::string k(key);
  if (k == "keep_routing") v = ctx->keep_routing ? "true" : "false";
  else if (k == "seq_len") v = std::to_string(ctx->seq_len);
  else if (k == "tc_launches") v = std::to_string(ctx->tc_launches);
  else if (k == "q4_expanded") v = std::to_string(ctx->q4_expanded);
  else if (k == "topn_launches") v = std::to_string(ctx->topn_launches);
  else if (k == "device_topn") v = ctx->device_topn ? "1" : "0";
  else if (k == "tc_error") {
    int32_t code = 0;
    if (ctx->have_last_stream) cudaStreamSynchronize(ctx->last_stream);
    if (ctx->d_tc_err) cudaMemcpy(&code, ctx->d_tc_err, 4, cudaMemcpyDeviceToHost);
    v = std::to_string(code);
  }
  else if (k == "slab_impl") v = !ctx->slab_built ? "none" : (ctx->slab_vmm ? "vmm" : "cudamalloc");
  else if (k == "line_stride") v = std::to_string(ctx->line_stride);
  else if (k == "stable_va") v = ctx->stable_va ? "true" : "false";
  else if (k == "shared_arena") v = ctx->shared_prefix;
  else if (k == "pool_slice") v = std::to_string(ctx->pool_slice);
  else if (k == "pool_bytes_pulled") v = std::to_string(ctx->pool_bytes_pulled);
  else if (k == "expert_va_base") v = std::to_string((unsigned long long)(uintptr_t)ctx->expert_va);
  else if (k == "slab_base") v = std::to_string((unsigned long long)(uintptr_t)ctx->slab);
  else if (k == "slab_bytes") v = std::to_string((unsigned long long)ctx->line_stride * (ctx->n_lines + 1));
  else if (k == "num_lines") v = std::to_string(ctx->n_lines);
  else if (k == "record_bytes") v = std::to_string(ctx->param_offset.empty() ? 0 : ctx->param_offset.back());
  else if (!ctx->cfg.get(k, &v)) return fail(PM_ERR_INVALID, "unknown config key " + k);
  if (v.size() + 1 > cap) return fail(PM_ERR_INVALID, "buffer too small");
  std::memcpy(buf, v.c_str(), v.size() + 1);
  return PM_OK;
}

int pm_ctx_set(pm_ctx* ctx, const char* key, const char* value) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!key || !value) return fail(PM_ERR_INVALID, "null argument");
  std::string k(key), v(value);
  if (k == "keep_routing") {
    ctx->keep_routing = (v == "1" || v == "true" || v == "True" || v == "on");
    return PM_OK;
  }
  if (k == "seq_len") {
    ctx->seq_len = std::atoi(value);
    return PM_OK;
  }
  if (k == "tc_prefill") {
    ctx->tc_prefill = (v == "1" || v == "true" || v == "True" || v == "on");
    return PM_OK;
  }
  if (k == "device_topn") {  // rank the predictor scores on the device (default) or on the host
    ctx->device_topn = (v == "1" || v == "true" || v == "True" || v == "on");
    return PM_OK;
  }
  if (k == "shared_arena") {
    if (ctx->pinned) return fail(PM_ERR_STATE, "shared_arena must be set before pin_all");
    ctx->shared_prefix = v;
    return PM_OK;
  }
  if (k == "stable_va") {
    if (ctx->slab_built) return fail(PM_ERR_STATE, "stable_va must be set before build_slab");
    ctx->stable_va = (v == "1" || v == "true" || v == "True" || v == "on");
    return PM_OK;
  }
  if (k == "device_plan") {
    ctx->device_plan = (v == "1" || v == "true" || v == "True" || v == "on");
    return PM_OK;
  }
  if (k == "profile_ffn") {
    ctx->profile_ffn = (v == "1" || v == "true" || v == "True" || v == "on");
    return PM_OK;
  }
  return from(ctx->cfg.set(k, v), PM_ERR_INVALID);
}

int pm_ctx_set_param_list(pm_ctx* ctx, const char* names) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (ctx->pinned) return fail(PM_ERR_STATE, "set_param_list after pin_all");
  std::vector<std::string> v;
  std::istringstream in(names ? names : "");
  std::string line;
  while (std::getline(in, line))
    if (!line.empty()) v.push_back(line);
  if (v.empty()) return fail(PM_ERR_INVALID, "empty tensor name list");
  ctx->cfg.param_names = v;
  ctx->params.assign((size_t)ctx->cfg.num_layer * ctx->cfg.num_expert * v.size(), pm_ctx::Param());
  assign_roles(ctx);
  return PM_OK;
}

int pm_register_expert_param(pm_ctx* ctx, int layer, int expert, int param_id, const void* host_ptr,
                             size_t nbytes) {
  if (need(ctx)) return PM_ERR_INVALID;
  const int N = ctx->cfg.num_per_expert_param();
  if (N == 0) return fail(PM_ERR_STATE, "register_expert_param before set_param_list");
  if (ctx->pinned) return fail(PM_ERR_STATE, "register_expert_param after pin_all");
  if (layer < 0 || layer >= ctx->cfg.num_layer || expert < 0 || expert >= ctx->cfg.num_expert || param_id < 0 ||
      param_id >= N)
    return fail(PM_ERR_INVALID, "layer, expert or tensor index out of range");
  pm_ctx::Param& p = ctx->params[((size_t)layer * ctx->cfg.num_expert + expert) * N + param_id];
  p.src = host_ptr;
  p.nbytes = nbytes;
  return PM_OK;
}

int pm_pin_all(pm_ctx* ctx) {
  if (need(ctx)) return PM_ERR_INVALID;
  return rt_pin_all(ctx);
}

int pm_expert_host_ptr(pm_ctx* ctx, int layer, int expert, int param_id, void** out, size_t* nbytes) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!ctx->pinned) return fail(PM_ERR_STATE, "expert_host_ptr before pin_all");
  const int N = ctx->cfg.num_per_expert_param();
  if (layer < 0 || layer >= ctx->cfg.num_layer || expert < 0 || expert >= ctx->cfg.num_expert || param_id < 0 ||
      param_id >= N || !out)
    return fail(PM_ERR_INVALID, "layer, expert or tensor index out of range");
  const size_t f = (size_t)layer * ctx->cfg.num_expert + expert;
  *out = ctx->host_rec[f] + ctx->param_offset[param_id];
  if (nbytes) *nbytes = ctx->params[f * N + param_id].nbytes;
  return PM_OK;
}

int pm_plan_slots(pm_ctx* ctx, int32_t* per_pool_len, int cap, int* n_pools) {
  if (need(ctx)) return PM_ERR_INVALID;
  const int n = ctx->cfg.per_layer_cache ? ctx->cfg.num_layer : 1;
  if (n_pools) *n_pools = n;
  if (per_pool_len == nullptr) return PM_OK;
  if (cap < n) return fail(PM_ERR_INVALID, "buffer too small");
  std::vector<int32_t> lens = CacheEngine::plan_lines(n, ctx->eng->total_lines());
  std::memcpy(per_pool_len, lens.data(), (size_t)n * 4);
  return PM_OK;
}

int pm_build_slab(pm_ctx* ctx) {
  if (need(ctx)) return PM_ERR_INVALID;
  return rt_build_slab(ctx);
}

int pm_build_policy_only(pm_ctx* ctx) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (ctx->cfg.num_per_expert_param() == 0) ctx->cfg.param_names = {"w"};
  return from(ctx->eng->build());
}

int pm_param_device_ptr(pm_ctx* ctx, int layer, int expert, int param_id, void** out) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!out) return fail(PM_ERR_INVALID, "null output pointer");
  *out = nullptr;
  if (!ctx->slab_built) return fail(PM_ERR_STATE, "param_device_ptr before build_slab");
  if (layer < 0 || layer >= ctx->cfg.num_layer || expert < 0 || expert >= ctx->cfg.num_expert || param_id < 0 ||
      param_id >= ctx->cfg.num_per_expert_param())
    return fail(PM_ERR_INVALID, "layer, expert or tensor index out of range");
  if (ctx->stable_va) {  // the expert's own range: the same address for the life of the context
    *out = ctx->expert_va + ((size_t)layer * ctx->cfg.num_expert + expert) * ctx->line_stride + ctx->param_offset[param_id];
    return PM_OK;
  }
  int line = ctx->eng->expert(layer, expert).line;
  if (line >= 0) *out = ctx->slab + (size_t)line * ctx->line_stride + ctx->param_offset[param_id];
  return PM_OK;
}

int pm_expert_slot(pm_ctx* ctx, int layer, int expert, int32_t* slot) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!slot || layer < 0 || layer >= ctx->cfg.num_layer || expert < 0 || expert >= ctx->cfg.num_expert)
    return fail(PM_ERR_INVALID, "layer or expert out of range");
  if (!ctx->eng->built()) return fail(PM_ERR_STATE, "expert_slot before the cache was built");
  *slot = ctx->eng->slot_of(layer, expert);
  return PM_OK;
}

int pm_report_layer(pm_ctx* ctx, int layer, int64_t* ids, int64_t n) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (n < 0 || (n > 0 && !ids)) return fail(PM_ERR_INVALID, "bad id list");
  std::vector<Action> acts;
  int rc = from(ctx->eng->report_layer(layer, ids, n, &acts));
  if (rc != PM_OK) return rc;
  rt_mark_dirty(ctx, acts);
  return rt_execute_copies(ctx, acts);
}

int pm_prefetch_layer(pm_ctx* ctx, int layer, const int64_t* ids, int64_t n) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (n < 0 || (n > 0 && !ids)) return fail(PM_ERR_INVALID, "bad id list");
  std::vector<Action> acts;
  int rc = from(ctx->eng->prefetch_layer(layer, ids, n, &acts));
  if (rc != PM_OK) return rc;
  rt_mark_dirty(ctx, acts);
  return rt_execute_copies(ctx, acts);
}

int pm_report_expert(pm_ctx* ctx, int layer, int expert) {
  if (need(ctx)) return PM_ERR_INVALID;
  std::vector<Action> acts;
  int rc = from(ctx->eng->report_expert(layer, expert, &acts));
  if (rc != PM_OK) return rc;
  rt_mark_dirty(ctx, acts);
  return rt_execute_copies(ctx, acts);
}

int pm_expert_done(pm_ctx* ctx, int layer, int expert) {
  if (need(ctx)) return PM_ERR_INVALID;
  return from(ctx->eng->expert_done(layer, expert), PM_ERR_INVALID);
}

int pm_expert_acquire(pm_ctx* ctx, int layer, int expert, void* stream, void** line) {
  if (need(ctx)) return PM_ERR_INVALID;
  return rt_expert_acquire(ctx, layer, expert, (cudaStream_t)stream, line);
}

int pm_expert_release(pm_ctx* ctx, int layer, int expert, void* stream) {
  if (need(ctx)) return PM_ERR_INVALID;
  return rt_expert_release(ctx, layer, expert, (cudaStream_t)stream);
}

int pm_param_offset(pm_ctx* ctx, int param_id, size_t* offset) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!ctx->pinned) return fail(PM_ERR_STATE, "param_offset before pin_all");
  if (!offset || param_id < 0 || param_id >= ctx->cfg.num_per_expert_param())
    return fail(PM_ERR_INVALID, "tensor index out of range");
  *offset = ctx->param_offset[param_id];
  return PM_OK;
}

int pm_temp_move_expert_to_gpu(pm_ctx* ctx, int layer, int expert, void* stream, void** line) {
  if (need(ctx)) return PM_ERR_INVALID;
  return rt_temp_move(ctx, layer, expert, true, (cudaStream_t)stream, line);
}

int pm_temp_move_expert_back_to_host(pm_ctx* ctx, int layer, int expert, void* stream) {
  if (need(ctx)) return PM_ERR_INVALID;
  return rt_temp_move(ctx, layer, expert, false, (cudaStream_t)stream, nullptr);
}

int pm_layer_done(pm_ctx* ctx, int layer) {
  if (need(ctx)) return PM_ERR_INVALID;
  return from(ctx->eng->layer_done(layer), PM_ERR_INVALID);
}

int pm_set_cur_seq(pm_ctx* ctx, uint64_t seq_id) {
  if (need(ctx)) return PM_ERR_INVALID;
  return from(ctx->eng->set_cur_seq(seq_id));
}

int pm_oracle_add_use_times(pm_ctx* ctx, uint64_t seq_id, int layer, int expert, const int64_t* times,
                            int64_t n) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (n < 0 || (n > 0 && !times)) return fail(PM_ERR_INVALID, "bad time list");
  return from(ctx->eng->add_use_times(seq_id, layer, expert, times, n), PM_ERR_INVALID);
}

int pm_update_priority(pm_ctx* ctx, const float* prob, int n_layers, int start_layer) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!prob) return fail(PM_ERR_INVALID, "null scores");
  return from(ctx->eng->update_priority(prob, n_layers, start_layer));
}

int pm_history_input(pm_ctx* ctx, float* out, size_t cap) {
  if (need(ctx)) return PM_ERR_INVALID;
  const size_t LE = (size_t)ctx->cfg.num_layer * ctx->cfg.num_expert;
  if (!out || cap < LE) return fail(PM_ERR_INVALID, "history_input: buffer of num_layer * num_expert floats needed");
  std::vector<float> h = ctx->eng->history_input();
  std::memcpy(out, h.data(), LE * sizeof(float));
  return PM_OK;
}

int pm_event_log_enable(pm_ctx* ctx, int on) {
  if (need(ctx)) return PM_ERR_INVALID;
  ctx->eng->log_enabled = on != 0;
  return PM_OK;
}

int pm_event_log_read(pm_ctx* ctx, pm_event* out, size_t cap, size_t* n) {
  if (need(ctx)) return PM_ERR_INVALID;
  const std::vector<CacheEvent>& log = ctx->eng->log;
  if (n) *n = log.size();
  if (out == nullptr) return PM_OK;
  static_assert(sizeof(pm_event) == sizeof(CacheEvent), "event layouts must agree");
  std::memcpy(out, log.data(), std::min(cap, log.size()) * sizeof(pm_event));
  return PM_OK;
}

int pm_event_log_clear(pm_ctx* ctx) {
  if (need(ctx)) return PM_ERR_INVALID;
  ctx->eng->log.clear();
  return PM_OK;
}

int pm_stats_read(pm_ctx* ctx, pm_stats* out) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!out) return fail(PM_ERR_INVALID, "null output pointer");
  const Counters& k = ctx->eng->counters;
  out->precise_hit = k.precise_hit;
  out->precise_miss = k.precise_miss;
  out->prefetch_hit = k.prefetch_hit;
  out->prefetch_miss = k.prefetch_miss;
  out->ready = k.ready;
  out->unready = k.unready;
  out->activated_experts = k.activated_experts;
  out->layer_calls = k.layer_calls;
  out->h2d_bytes = ctx->h2d_bytes;
  out->h2d_copies = ctx->h2d_copies;
  out->kernel_launches = ctx->kernel_launches;
  return PM_OK;
}

int pm_iter_marks_read(pm_ctx* ctx, pm_stats* out, size_t cap, size_t* n) {
  if (need(ctx)) return PM_ERR_INVALID;
  const std::vector<Counters>& marks = ctx->eng->iter_marks;
  if (n) *n = marks.size();
  if (out == nullptr) return PM_OK;
  for (size_t i = 0; i < std::min(cap, marks.size()); ++i) {
    const Counters& k = marks[i];
    pm_stats s{};
    s.precise_hit = k.precise_hit;
    s.precise_miss = k.precise_miss;
    s.prefetch_hit = k.prefetch_hit;
    s.prefetch_miss = k.prefetch_miss;
    s.ready = k.ready;
    s.unready = k.unready;
    s.activated_experts = k.activated_experts;
    s.layer_calls = k.layer_calls;
    out[i] = s;
  }
  return PM_OK;
}

int pm_profile_read(pm_ctx* ctx, pm_profile* out, int reset) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!out) return fail(PM_ERR_INVALID, "null output pointer");
  int rc = rt_profile_collect(ctx);
  if (rc != PM_OK) return rc;
  out->ffn_launches = ctx->ffn_launches;
  out->gateup_ms = ctx->ffn_ms_gu;
  out->down_ms = ctx->ffn_ms_dn;
  out->gateup_bytes = ctx->ffn_bytes_gu;
  out->down_bytes = ctx->ffn_bytes_dn;
  out->fused_launches = ctx->ffn_fused_launches;
  out->fused_ms = ctx->ffn_ms_fused;
  out->fused_bytes = ctx->ffn_bytes_fused;
  out->resident_launches = ctx->ffn_resident_launches;
  out->resident_ms = ctx->ffn_ms_resident;
  out->resident_bytes = ctx->ffn_bytes_resident;
  if (reset) {
    ctx->ffn_fused_launches = 0;
    ctx->ffn_ms_fused = 0;
    ctx->ffn_bytes_fused = 0;
    ctx->ffn_resident_launches = 0;
    ctx->ffn_ms_resident = 0;
    ctx->ffn_bytes_resident = 0;
    ctx->ffn_launches = 0;
    ctx->ffn_ms_gu = ctx->ffn_ms_dn = 0;
    ctx->ffn_bytes_gu = ctx->ffn_bytes_dn = 0;
  }
  return PM_OK;
}

int pm_layer_set_weights(pm_ctx* ctx, int layer, const pm_layer_weights* w) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!w || layer < 0 || layer >= ctx->cfg.num_layer) return fail(PM_ERR_INVALID, "layer out of range");
  if (w->hidden <= 0 || w->hidden % 64 != 0) return fail(PM_ERR_INVALID, "hidden must be a positive multiple of 64");
  if (w->inter <= 0 || w->inter % 32 != 0) return fail(PM_ERR_INVALID, "inter must be a positive multiple of 32");
  if (w->shared_inter < 0 || w->shared_inter % 32 != 0) return fail(PM_ERR_INVALID, "shared_inter must be a multiple of 32");
  if (w->shared_inter > 0 && (!w->shared_w_gate || !w->shared_w_up || !w->shared_w_down))
    return fail(PM_ERR_INVALID, "shared expert weights missing");
  if (w->top_k <= 0 || w->top_k > 16 || w->top_k > ctx->cfg.num_expert) return fail(PM_ERR_INVALID, "top_k out of range");
  if (w->quant4 && (ctx->role_qgate < 0 || ctx->role_qup < 0 || ctx->role_qdown < 0))
    return fail(PM_ERR_INVALID, "quant4 layer needs scale/zero tensors in the tensor list");
  if (w->quant4 && (w->hidden % 128 != 0 || w->inter % 128 != 0))
    return fail(PM_ERR_INVALID, "quant4 layer needs hidden and inter to be multiples of 128");
  ctx->layers[layer].w = *w;
  ctx->layers[layer].set = true;
  return PM_OK;
}

int pm_moe_forward(pm_ctx* ctx, int layer, const void* x_dev, int T, void* y_dev, void* stream) {
  if (need(ctx)) return PM_ERR_INVALID;
  return rt_forward(ctx, layer, x_dev, T, y_dev, (cudaStream_t)stream);
}

namespace {
int fill_routed(pm_ctx* ctx, RoutedRows* r, const int32_t* row_expert, float* rows_out, int max_rows_per_expert,
                const float* pred_scores, const int32_t* pred_layers, int n_pred, int pred_width, int pred_first,
                int pred_top) {
  if (n_pred < 0 || (n_pred > 0 && (!pred_scores || !pred_layers))) return fail(PM_ERR_INVALID, "bad prediction arguments");
  if (n_pred > 0 && (pred_width < ctx->cfg.num_expert || pred_width > 4096 || pred_first < 0 ||
                     pred_first + ctx->cfg.num_expert > pred_width || pred_top < 0))
    return fail(PM_ERR_INVALID, "the prediction's expert range does not contain this context's experts");
  r->row_expert = row_expert;
  r->rows_out = rows_out;
  r->max_rows_per_expert = max_rows_per_expert;
  r->pred_scores = pred_scores;
  r->pred_layers = pred_layers;
  r->n_pred = n_pred;
  r->pred_width = pred_width;
  r->pred_first = pred_first;
  r->pred_top = pred_top;
  return PM_OK;
}
}  // namespace

int pm_moe_forward_routed(pm_ctx* ctx, int layer, const void* x_rows, int n_rows, const int32_t* row_expert,
                          float* rows_out, int max_rows_per_expert, const float* pred_scores,
                          const int32_t* pred_layers, int n_pred, int pred_width, int pred_first, int pred_top,
                          void* stream) {
  if (need(ctx)) return PM_ERR_INVALID;
  RoutedRows r;
  int rc0 = fill_routed(ctx, &r, row_expert, rows_out, max_rows_per_expert, pred_scores, pred_layers, n_pred, pred_width,
                        pred_first, pred_top);
  if (rc0 != PM_OK) return rc0;
  return rt_forward(ctx, layer, x_rows, n_rows, nullptr, (cudaStream_t)stream, &r);
}

int pm_moe_forward_routed_begin(pm_ctx* ctx, int layer, const void* x_rows, int n_rows, const int32_t* row_expert,
                                float* rows_out, int max_rows_per_expert, const float* pred_scores,
                                const int32_t* pred_layers, int n_pred, int pred_width, int pred_first, int pred_top,
                                void* stream, int32_t* miss_experts, int miss_cap, int* n_miss) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!n_miss || (miss_cap > 0 && !miss_experts)) return fail(PM_ERR_INVALID, "null miss list");
  *n_miss = 0;
  RoutedRows r;
  int rc0 = fill_routed(ctx, &r, row_expert, rows_out, max_rows_per_expert, pred_scores, pred_layers, n_pred, pred_width,
                        pred_first, pred_top);
  if (rc0 != PM_OK) return rc0;
  r.collect_demand_copies = true;
  int rc = rt_forward(ctx, layer, x_rows, n_rows, nullptr, (cudaStream_t)stream, &r);
  if (rc != PM_OK) return rc;
  const std::vector<Action>& pooled = rt_pending_pooled(ctx);
  if ((int)pooled.size() > miss_cap || pooled.size() > (size_t)kPoolMaxMiss) {
    rc = rt_pool_fetch_locally(ctx);  // more than the exchange can carry: this rank copies them itself
    return rc;
  }
  for (size_t i = 0; i < pooled.size(); ++i) miss_experts[i] = pooled[i].expert;
  *n_miss = (int)pooled.size();
  return PM_OK;
}

int pm_moe_forward_routed_end(pm_ctx* ctx) {
  if (need(ctx)) return PM_ERR_INVALID;
  return rt_forward_end(ctx);
}

int pm_pool_init(pm_ctx* ctx, int rank, int world, const char* mailbox_name) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!mailbox_name) return fail(PM_ERR_INVALID, "null mailbox name");
  return rt_pool_init(ctx, rank, world, mailbox_name);
}

int pm_pool_open_peer(pm_ctx* ctx, int peer, const char* arena_prefix, int peer_num_expert) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!arena_prefix) return fail(PM_ERR_INVALID, "null arena prefix");
  return rt_pool_open_peer(ctx, peer, arena_prefix, peer_num_expert);
}

int pm_pool_exchange(pm_ctx* ctx, int64_t seq, const int32_t* experts, int n, int32_t* lists_out, double timeout_s) {
  if (need(ctx)) return PM_ERR_INVALID;
  if ((n > 0 && !experts) || !lists_out) return fail(PM_ERR_INVALID, "null list");
  return rt_pool_exchange(ctx, seq, experts, n, lists_out, timeout_s);
}

int pm_pool_stage(pm_ctx* ctx, int layer, const int32_t* lists, void* send_dev, size_t send_cap, size_t recv_cap,
                  int64_t* send_split, int64_t* recv_split, void* stream) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!lists || !send_dev || !send_split || !recv_split) return fail(PM_ERR_INVALID, "null argument");
  return rt_pool_stage(ctx, layer, lists, send_dev, send_cap, recv_cap, send_split, recv_split, (cudaStream_t)stream);
}

int pm_pool_scatter(pm_ctx* ctx, const void* recv_dev, void* stream) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!recv_dev) return fail(PM_ERR_INVALID, "null receive buffer");
  return rt_pool_scatter(ctx, recv_dev, (cudaStream_t)stream);
}

int pm_pool_fetch_locally(pm_ctx* ctx) {
  if (need(ctx)) return PM_ERR_INVALID;
  return rt_pool_fetch_locally(ctx);
}

int pm_moe_forward_host(pm_ctx* ctx, int layer, const void* x_host, int T, void* y_host, void* stream) {
  if (need(ctx)) return PM_ERR_INVALID;
  return rt_forward_host(ctx, layer, x_host, T, y_host, (cudaStream_t)stream);
}

int pm_last_routing(pm_ctx* ctx, int layer, int32_t* topk_ids, float* topk_w, int cap_pairs) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (layer < 0 || layer >= ctx->cfg.num_layer) return fail(PM_ERR_INVALID, "layer out of range");
  if (!ctx->keep_routing) return fail(PM_ERR_STATE, "set keep_routing=1 before the forward");
  const std::vector<int32_t>& ids = ctx->last_ids[layer];
  if ((size_t)cap_pairs < ids.size()) return fail(PM_ERR_INVALID, "buffer too small");
  if (topk_ids) std::memcpy(topk_ids, ids.data(), ids.size() * 4);
  if (topk_w) std::memcpy(topk_w, ctx->last_w[layer].data(), ids.size() * 4);
  return PM_OK;
}

int pm_predictor_set(pm_ctx* ctx, int src_layer, int dst_layer, const void* w1, const float* b1, int d,
                     const void* w2, const float* b2) {
  if (need(ctx)) return PM_ERR_INVALID;
  const int L = ctx->cfg.num_layer;
  if (src_layer < 0 || src_layer > L || dst_layer < 0 || dst_layer >= L) return fail(PM_ERR_INVALID, "layer out of range");
  if (!w1 || !w2 || d <= 0 || d > 4096) return fail(PM_ERR_INVALID, "bad predictor weights");
  pm_ctx::Predictor& p = ctx->predictors[(size_t)src_layer * L + dst_layer];
  p.w1 = w1;
  p.b1 = b1;
  p.d = d;
  p.w2 = w2;
  p.b2 = b2;
  return PM_OK;
}

int pm_report_hidden(pm_ctx* ctx, int index, const void* hidden_dev, int B, int seq, void* stream) {
  if (need(ctx)) return PM_ERR_INVALID;
  if (!hidden_dev && B > 0 && seq == 1) return fail(PM_ERR_INVALID, "null hidden states");
  return rt_report_hidden(ctx, index, hidden_dev, B, seq, (cudaStream_t)stream);
}

}  // extern "C"
