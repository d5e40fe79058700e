#include "runtime.hpp"

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>

namespace pm {
namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// CUDA driver (virtual memory management) entry points, resolved through the runtime so the
// library has no link-time dependency on the driver.
struct Driver {
  CUresult (*GetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*AddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*Create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*Unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*Release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*AddressFree)(CUdeviceptr, size_t) = nullptr;
  bool ok = false;
};

Driver& driver() {
  static Driver d;
  static bool tried = false;
  if (tried) return d;
  tried = true;
  auto get = [](const char* name, void** fn) {
    cudaDriverEntryPointQueryResult q;
    return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess &&
           q == cudaDriverEntryPointSuccess && *fn != nullptr;
  };
  d.ok = get("cuMemGetAllocationGranularity", (void**)&d.GetGranularity) &&
         get("cuMemAddressReserve", (void**)&d.AddressReserve) && get("cuMemCreate", (void**)&d.Create) &&
         get("cuMemMap", (void**)&d.Map) && get("cuMemSetAccess", (void**)&d.SetAccess) &&
         get("cuMemUnmap", (void**)&d.Unmap) && get("cuMemRelease", (void**)&d.Release) &&
         get("cuMemAddressFree", (void**)&d.AddressFree);
  return d;
}

int fail_cu(CUresult r, const char* what) {
  return fail(PM_ERR_CUDA, std::string(what) + " failed with CUresult " + std::to_string((int)r));
}

// Waits for an event with a deadline instead of an unbounded block.
int wait_event(cudaEvent_t ev, double seconds) {
  auto t0 = std::chrono::steady_clock::now();
  while (true) {
    cudaError_t q = cudaEventQuery(ev);
    if (q == cudaSuccess) return PM_OK;
    if (q != cudaErrorNotReady) return fail_cuda(q, "cudaEventQuery");
    if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > seconds)
      return fail(PM_ERR_TIMEOUT, "device did not reach the routing read-back within the deadline");
  }
}

unsigned char* line_ptr(pm_ctx* c, int line) { return c->slab + (size_t)line * c->line_stride; }

cudaEvent_t next_seg_event(pm_ctx* c) {
  cudaEvent_t e = c->seg_events[c->seg_next];
  c->seg_next = (c->seg_next + 1) % c->seg_events.size();
  return e;
}

// stable_va: the line now belongs to expert f, so it leaves the previous owner's address range and
// appears in f's. Unmapping needs the line idle: the host waits for the last kernel that read it.
int remap_line(pm_ctx* c, int line, size_t f) {
  if (c->line_mapped_to[line] == (int32_t)f) return PM_OK;
  Driver& d = driver();
  if (c->line_read[line] != nullptr) PM_CUDA(cudaEventSynchronize(c->line_read[line]));
  if (c->line_mapped_to[line] >= 0) {
    CUresult r = d.Unmap((CUdeviceptr)(c->expert_va + (size_t)c->line_mapped_to[line] * c->line_stride), c->line_stride);
    if (r != CUDA_SUCCESS) return fail_cu(r, "cuMemUnmap (expert range)");
  }
  const CUdeviceptr va = (CUdeviceptr)(c->expert_va + f * c->line_stride);
  CUresult r = d.Map(va, c->line_stride, 0, c->line_handles[line], 0);
  if (r != CUDA_SUCCESS) return fail_cu(r, "cuMemMap (expert range)");
  CUmemAccessDesc acc{};
  acc.location = c->line_prop.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.SetAccess(va, c->line_stride, &acc, 1);
  if (r != CUDA_SUCCESS) return fail_cu(r, "cuMemSetAccess (expert range)");
  c->line_mapped_to[line] = (int32_t)f;
  return PM_OK;
}

int enqueue_copy(pm_ctx* c, const Action& a) {
  const int E = c->cfg.num_expert;
  const size_t f = (size_t)a.layer * E + a.expert;
  if (c->stable_va) {
    int rc = remap_line(c, a.line, f);
    if (rc != PM_OK) return rc;
  }
  const size_t b0 = c->param_offset[a.chunk_begin], b1 = c->param_offset[a.chunk_end];
  cudaStream_t cs = c->cfg.cache_only ? c->last_stream : (a.precise ? c->copy_stream : c->prefetch_stream);
  if (c->line_read[a.line] != nullptr) PM_CUDA(cudaStreamWaitEvent(cs, c->line_read[a.line], 0));
  if (c->line_copy_stream[a.line] != nullptr && c->line_copy_stream[a.line] != cs)
    PM_CUDA(cudaStreamWaitEvent(cs, c->line_ready[a.line], 0));  // behind the previous copy into this line
  c->line_copy_stream[a.line] = cs;
  PM_CUDA(cudaMemcpyAsync(line_ptr(c, a.line) + b0, c->host_rec[f] + b0, b1 - b0, cudaMemcpyHostToDevice, cs));
  PM_CUDA(cudaEventRecord(c->line_ready[a.line], cs));
  c->line_pending[a.line] = 1;
  c->line_waiter[a.line] = nullptr;
  c->h2d_bytes += (int64_t)(b1 - b0);
  c->h2d_copies += 1;
  return PM_OK;
}

int ensure_workspace(pm_ctx* c, int T, const pm_layer_weights& w) {
  const int E = c->cfg.num_expert;
  const int max_inter = std::max(w.inter, w.shared_inter);
  if (T <= c->ws_tokens && w.hidden <= c->ws_hidden && max_inter <= c->ws_inter && w.top_k <= c->ws_topk &&
      w.inter <= c->ws_inter_routed && w.shared_inter <= c->ws_inter_shared)
    return PM_OK;
  if (c->have_last_stream) PM_CUDA(cudaStreamSynchronize(c->last_stream));
  if (c->ws_dev) PM_CUDA(cudaFree(c->ws_dev));
  if (c->h_stage) PM_CUDA(cudaFreeHost(c->h_stage));
  c->ws_dev = nullptr;
  c->h_stage = nullptr;
  const int cap = std::max(T, std::max(16, c->ws_tokens * 2));
  const int H = std::max(w.hidden, c->ws_hidden), I = std::max(max_inter, c->ws_inter);
  const int k = std::max(w.top_k, c->ws_topk);
  // routed rows + one shared-expert row per token; decode batches (at most kSplitMaxRows tokens) cut the
  // shared expert into up to kMaxSharedSlices slices with a row per token each
  const size_t R = (size_t)cap * k, rows = R + cap + (size_t)kSplitMaxRows * kMaxSharedSlices;
  {
    // worst case of one layer call: every expert plus the shared expert, chunks of 64 rows, smallest
    // tiles, and a few extra segments each aligned to 256 bytes
    FfnPlanInfo worst;
    worst.n_desc = E + (int)(rows / kSplitMaxRows) + 8 + kMaxSharedSlices;
    worst.tiles_gu = worst.n_desc * ((I + kSplitTileGu - 1) / kSplitTileGu);
    worst.tiles_dn = worst.n_desc * ((H + kSplitTileDn - 1) / kSplitTileDn);
    c->plan_cap = align_up(worst.blob_bytes(), 256) + 64 * 256;
  }
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off += align_up(bytes, 256);
    return o;
  };
  size_t o_ids = take(R * 4), o_slot = take(R * 4), o_w = take(R * 4), o_ss = take((size_t)cap * 4);
  // counts [E], offsets [E + 1], the permutation's error word and the FFN kernels' error word travel
  // to the host in one copy
  size_t o_cnt = take((size_t)(2 * E + 3) * 4), o_rt = take(rows * 4), o_pos = take(R * 4);
  size_t o_h = take(rows * I * 2), o_y = take(rows * H * 4), o_desc = take(c->plan_cap);
  size_t o_sc = take((size_t)c->cfg.num_layer * E * 4), o_ph = take((size_t)cap * 4096 * 4);
  size_t o_x = take((size_t)cap * H * 2), o_yo = take((size_t)cap * H * 2);
  const int Ir = std::max(w.inter, c->ws_inter_routed);
  const int Is = std::max(w.shared_inter, c->ws_inter_shared);
  size_t o_res = take((size_t)(kMaxFusedGroups + 1) * 4);
  size_t o_xp = take(rows * H * 2);
  {
    const size_t m_tiles = rows / 128 + (size_t)E + 2;
    c->tc_plan_cap = 16 * ((size_t)E + 2) + 16 * m_tiles * ((size_t)(std::max(I, Is) + 127) / 128 + (size_t)(H + 127) / 128) + 1024 +
                     768 * ((size_t)E + 2);  // three 256-byte roundings per segment, at most one segment per expert
  }
  size_t o_tcp = take(c->tc_plan_cap);
  c->perm_scratch_ints = (R / 4096 + 2) * (size_t)E;
  size_t o_ps = take(c->perm_scratch_ints * 4);
  PM_CUDA(cudaMalloc(&c->ws_dev, off));
  PM_CUDA(cudaMemset(c->ws_dev, 0, off));
  c->ws_bytes = off;
  unsigned char* b = c->ws_dev;
  c->d_topk_ids = (int32_t*)(b + o_ids);
  c->d_topk_slot = (int32_t*)(b + o_slot);
  c->d_topk_w = (float*)(b + o_w);
  c->d_shared_scale = (float*)(b + o_ss);
  c->d_counts = (int32_t*)(b + o_cnt);
  c->d_offsets = c->d_counts + E;
  c->d_row_token = (int32_t*)(b + o_rt);
  c->d_pos = (int32_t*)(b + o_pos);
  c->d_err = c->d_counts + 2 * E + 1;
  c->d_tc_err = c->d_counts + 2 * E + 2;
  c->d_hbuf = (__nv_bfloat16*)(b + o_h);
  c->d_yexp = (float*)(b + o_y);
  c->d_plan = b + o_desc;
  c->d_scores = (float*)(b + o_sc);
  c->d_pred_hidden = (float*)(b + o_ph);
  c->d_xin = (__nv_bfloat16*)(b + o_x);
  c->d_yout = (__nv_bfloat16*)(b + o_yo);
  c->d_res_counters = (int32_t*)(b + o_res);
  c->d_xperm = (__nv_bfloat16*)(b + o_xp);
  c->d_tc_plan = b + o_tcp;
  c->d_perm_scratch = (int32_t*)(b + o_ps);
  if (c->h_tc_plan) PM_CUDA(cudaFreeHost(c->h_tc_plan));
  PM_CUDA(cudaHostAlloc((void**)&c->h_tc_plan, c->tc_plan_cap + 64, cudaHostAllocDefault));
  c->ws_inter_routed = Ir;
  c->ws_inter_shared = Is;
  // pinned staging: [counts+offsets | scores | routing ids | routing weights | descriptors]
  c->h_stage_bytes = align_up((size_t)(2 * E + 3) * 4, 256) + align_up((size_t)c->cfg.num_layer * E * 4, 256) +
                     2 * align_up(R * 4, 256) + align_up(c->plan_cap, 256) +
                     align_up((size_t)E * 4, 256);
  PM_CUDA(cudaHostAlloc((void**)&c->h_stage, c->h_stage_bytes, cudaHostAllocDefault));
  c->ws_tokens = cap;
  c->ws_hidden = H;
  c->ws_inter = I;
  c->ws_topk = k;
  return PM_OK;
}

struct Stage {
  int32_t* counts;  // [E] then offsets [E+1]
  float* scores;    // [L, E]
  int32_t* ids;
  float* w;
  unsigned char* plan;
  int32_t* slot_table;
};

Stage stage_of(pm_ctx* c) {
  const int E = c->cfg.num_expert;
  const size_t R = (size_t)c->ws_tokens * c->ws_topk;
  Stage s;
  unsigned char* p = c->h_stage;
  s.counts = (int32_t*)p;
  p += align_up((size_t)(2 * E + 3) * 4, 256);
  s.scores = (float*)p;
  p += align_up((size_t)c->cfg.num_layer * E * 4, 256);
  s.ids = (int32_t*)p;
  p += align_up(R * 4, 256);
  s.w = (float*)p;
  p += align_up(R * 4, 256);
  s.plan = p;
  p += align_up(c->plan_cap, 256);
  s.slot_table = (int32_t*)p;
  return s;
}

// Ranks one predicted layer and issues its prefetch (PredictWorker::do_one_task_impl,
// src/cpp_worker/worker.cpp:6-77). `scores` covers `width` experts of which this context holds
// [first, first + num_expert): the `top` best of the whole list are taken and those this context
// holds are prefetched in rank order (width = num_expert, first = 0: the plain single-context case).
constexpr int kTopCap = 64;  // most ids the device-side ranking returns per predicted layer

// How many of the best-ranked experts a prediction for layer `dst` takes.
int prediction_count(const pm_ctx* c, int dst, int width, int top) {
  int n = std::min(top >= 0 ? top : c->cfg.num_predict_expert_per_layer, width);
  if (dst == 0 && c->cfg.limit_layer_0_num_predict != -1) n = std::min(n, c->cfg.limit_layer_0_num_predict);
  return n;
}

bool topn_on_device(const pm_ctx* c, int n, int width) { return c->device_topn && n > 0 && n <= kTopCap && width <= 9000; }

int ensure_topn(pm_ctx* c) {
  if (c->d_topn != nullptr) return PM_OK;
  const size_t bytes = (size_t)2 * c->cfg.num_layer * kTopCap * 4;
  PM_CUDA(cudaMalloc((void**)&c->d_topn, bytes));
  PM_CUDA(cudaHostAlloc((void**)&c->h_topn, bytes, cudaHostAllocDefault));
  return PM_OK;
}

// `ranked`: the ids the device ranked best (prediction_count of them), or nullptr to rank here.
int issue_prediction(pm_ctx* c, int dst, const float* scores, int width = 0, int first = 0, int top = -1,
                     const int32_t* ranked = nullptr) {
  const int E = c->cfg.num_expert;
  if (width <= 0) width = E;
  if (c->cfg.cache_policy == "nn") {
    std::string err = c->eng->update_priority(scores + first, 1, dst);
    if (!err.empty()) return fail(PM_ERR_STATE, err);
  }
  const int n = prediction_count(c, dst, width, top);
  std::vector<int64_t> order;
  if (ranked != nullptr) {
    for (int i = 0; i < n; ++i) {
      if (ranked[i] < 0 || ranked[i] >= width) return fail(PM_ERR_STATE, "device ranking returned an id out of range");
      order.push_back(ranked[i]);
    }
  } else {
    order.resize(width);
    for (int i = 0; i < width; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return scores[a] > scores[b]; });
  }
  std::vector<int64_t> mine;
  for (int i = 0; i < n; ++i)
    if (order[i] >= first && order[i] < first + E) mine.push_back(order[i] - first);
  // the cache clamps a prefetch to its own num_predict (the lines of pool 0, src/cpp_worker/cache.cpp:130-131)
  if ((int)mine.size() > c->cfg.num_predict_expert_per_layer) mine.resize(c->cfg.num_predict_expert_per_layer);
  if (mine.empty()) return PM_OK;
  std::vector<Action> acts;
  std::string err = c->eng->prefetch_layer(dst, mine.data(), (int64_t)mine.size(), &acts);
  if (!err.empty()) return fail(PM_ERR_STATE, err);
  rt_mark_dirty(c, acts);
  return rt_execute_copies(c, acts);
}

// Launches the predictor MLPs of source index `src` on x [B, H]; returns how many ran.
int launch_predictors(pm_ctx* c, int src, const __nv_bfloat16* x, int B, int H, cudaStream_t s,
                      std::vector<int>* dsts) {
  dsts->clear();
  if (c->cfg.predict_input_mode != "moe_layer_logits" || c->cfg.num_predict_expert_per_layer <= 0) return PM_OK;
  const int L = c->cfg.num_layer, E = c->cfg.num_expert;
  auto map = c->cfg.predict_layer_mapping();
  if (src < 0 || src > L) return PM_OK;
  if ((src % L) % c->cfg.layer_predict_interval != 0) return PM_OK;
  if (c->cfg.cross_token_pred && src == 0) return PM_OK;
  for (int dst = map[src].first; dst < map[src].second; ++dst) {
    const pm_ctx::Predictor& p = c->predictors[(size_t)src * L + dst];
    if (p.w1 == nullptr) continue;
    if (p.d > 4096) return fail(PM_ERR_UNSUPPORTED, "predictor hidden width above 4096");
    PM_CUDA(launch_predictor_mlp(x, B, H, (const __nv_bfloat16*)p.w1, p.b1, p.d, (const __nv_bfloat16*)p.w2,
                                 p.b2, E, c->d_pred_hidden, c->d_scores + (size_t)dst * E, s));
    c->kernel_launches += 2;
    const int n = prediction_count(c, dst, E, -1);
    if (topn_on_device(c, n, E)) {  // rank on the device: the host reads n ids instead of sorting E scores
      int rc = ensure_topn(c);
      if (rc != PM_OK) return rc;
      PM_CUDA(launch_rank_topn(c->d_scores + (size_t)dst * E, E, n, c->d_topn + (size_t)dst * kTopCap, s));
      c->kernel_launches += 1;
      c->topn_launches += 1;
    }
    dsts->push_back(dst);
  }
  return PM_OK;
}

}  // namespace

void rt_mark_dirty(pm_ctx* c, const std::vector<Action>& actions) {
  for (const Action& a : actions)
    if (a.type == Action::kCopy) {
      if (c->cfg.per_layer_cache) {
        c->layers[a.layer].slot_table_dirty = true;
      } else {
        for (auto& l : c->layers) l.slot_table_dirty = true;  // a shared pool can evict across layers
      }
    }
}

int rt_execute_copies(pm_ctx* c, const std::vector<Action>& actions) {
  if (!c->slab_built) return PM_OK;
  for (const Action& a : actions)
    if (a.type == Action::kCopy) {
      int rc = enqueue_copy(c, a);
      if (rc != PM_OK) return rc;
    }
  return PM_OK;
}

// Turns the recorded FFN event triples into accumulated milliseconds. Waits for the last one.
int rt_profile_collect(pm_ctx* c) {
  for (pm_ctx::FfnSample& f : c->ffn_samples) {
    PM_CUDA(cudaEventSynchronize(f.e2));
    float a = 0.f, b = 0.f;
    if (f.fused) {
      PM_CUDA(cudaEventElapsedTime(&a, f.e0, f.e2));
      c->ffn_ms_fused += a;
      c->ffn_bytes_fused += f.bytes_gu + f.bytes_dn;
      c->ffn_fused_launches += 1;
      if (f.resident) {
        c->ffn_ms_resident += a;
        c->ffn_bytes_resident += f.bytes_gu + f.bytes_dn;
        c->ffn_resident_launches += 1;
      }
    } else {
      PM_CUDA(cudaEventElapsedTime(&a, f.e0, f.e1));
      PM_CUDA(cudaEventElapsedTime(&b, f.e1, f.e2));
      c->ffn_ms_gu += a;
      c->ffn_ms_dn += b;
      c->ffn_bytes_gu += f.bytes_gu;
      c->ffn_bytes_dn += f.bytes_dn;
      c->ffn_launches += 1;
      c->ffn_event_pool.push_back(f.e1);
    }
    c->ffn_event_pool.push_back(f.e0);
    c->ffn_event_pool.push_back(f.e2);
  }
  c->ffn_samples.clear();
  return PM_OK;
}

int rt_pin_all(pm_ctx* c) {
  if (c->pinned) return fail(PM_ERR_STATE, "pin_all called twice");
  const int L = c->cfg.num_layer, E = c->cfg.num_expert, N = c->cfg.num_per_expert_param();
  if (N <= 0) return fail(PM_ERR_STATE, "pin_all before set_param_list");
  c->param_offset.assign(N + 1, 0);
  for (int p = 0; p < N; ++p) {
    size_t mx = 0;
    for (size_t f = 0; f < (size_t)L * E; ++f) mx = std::max(mx, c->params[f * N + p].nbytes);
    c->param_offset[p + 1] = c->param_offset[p] + align_up(mx, 256);
  }
  // Zero-sized experts (routing-trace replay with stand-in modules) still get a line each.
  if (c->param_offset[N] == 0) c->param_offset[N] = 256;
  const size_t rec = c->param_offset[N];
  c->host_rec.assign((size_t)L * E, nullptr);
  for (int l = 0; l < L; ++l) {
    void* block = nullptr;
    if (!c->shared_prefix.empty()) {  // shared memory that other ranks of the node can map and register too
      std::string err;
      block = rt_shared_block(c, c->shared_prefix + "_L" + std::to_string(l), rec * E, true, &err);
      if (block == nullptr) return fail(PM_ERR_STATE, err);
    } else {
      PM_CUDA(cudaHostAlloc(&block, rec * E, cudaHostAllocDefault));
    }
    c->arena_blocks.push_back(block);
    for (int e = 0; e < E; ++e) {
      unsigned char* dst = (unsigned char*)block + rec * e;
      c->host_rec[(size_t)l * E + e] = dst;
      for (int p = 0; p < N; ++p) {
        const pm_ctx::Param& pr = c->params[((size_t)l * E + e) * N + p];
        if (pr.src != nullptr && pr.nbytes > 0) std::memcpy(dst + c->param_offset[p], pr.src, pr.nbytes);
      }
    }
  }
  c->pinned = true;
  return PM_OK;
}

int rt_build_slab(pm_ctx* c) {
  if (c->slab_built) return fail(PM_ERR_STATE, "slab already built");
  if (!c->pinned) return fail(PM_ERR_STATE, "build_slab before pin_all");
  if (!c->eng->built()) {
    std::string err = c->eng->build();
    if (!err.empty()) return fail(PM_ERR_STATE, err);
  }
  int n_lines = 0;
  for (const Pool& p : c->eng->pools()) n_lines += p.full_len;
  if (n_lines <= 0) return fail(PM_ERR_INVALID, "cache_rate gives zero cache lines");
  const int n_policy_lines = n_lines;
  n_lines += 1;  // the spare line of temp_move_expert_to_gpu: no pool owns it
  const size_t rec = c->param_offset.back();
  const char* impl = std::getenv("PM_SLAB_IMPL");
  const bool want_vmm = impl == nullptr || std::string(impl) != "cudamalloc";
  int dev = 0;
  PM_CUDA(cudaGetDevice(&dev));
  PM_CUDA(cudaFree(0));  // make sure the primary context exists before driver calls
  c->slab_vmm = false;
  if (want_vmm && driver().ok) {
    Driver& d = driver();
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev;
    size_t gran = 0;
    CUresult r = d.GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
    if (r != CUDA_SUCCESS) return fail_cu(r, "cuMemGetAllocationGranularity");
    c->line_stride = align_up(rec, gran);
    c->slab_va_bytes = c->line_stride * n_lines;
    CUdeviceptr base = 0;
    r = d.AddressReserve(&base, c->slab_va_bytes, gran, 0, 0);
    if (r != CUDA_SUCCESS) return fail_cu(r, "cuMemAddressReserve");
    c->slab = (unsigned char*)base;
    c->line_handles.resize(n_lines);
    for (int i = 0; i < n_lines; ++i) {
      r = d.Create(&c->line_handles[i], c->line_stride, &prop, 0);
      if (r != CUDA_SUCCESS) return fail_cu(r, "cuMemCreate");
      r = d.Map(base + (size_t)i * c->line_stride, c->line_stride, 0, c->line_handles[i], 0);
      if (r != CUDA_SUCCESS) return fail_cu(r, "cuMemMap");
    }
    CUmemAccessDesc acc{};
    acc.location = prop.location;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = d.SetAccess(base, c->slab_va_bytes, &acc, 1);
    if (r != CUDA_SUCCESS) return fail_cu(r, "cuMemSetAccess");
    c->slab_vmm = true;
    c->line_prop = prop;
    if (c->stable_va) {
      c->expert_va_bytes = c->line_stride * (size_t)c->cfg.num_layer * c->cfg.num_expert;
      CUdeviceptr eva = 0;
      r = d.AddressReserve(&eva, c->expert_va_bytes, gran, 0, 0);
      if (r != CUDA_SUCCESS) return fail_cu(r, "cuMemAddressReserve (expert ranges)");
      c->expert_va = (unsigned char*)eva;
      c->line_mapped_to.assign(n_lines, -1);
    }
  } else {
    if (c->stable_va) return fail(PM_ERR_UNSUPPORTED, "stable_va needs the VMM slab");
    c->line_stride = align_up(rec, 256);
    PM_CUDA(cudaMalloc((void**)&c->slab, c->line_stride * n_lines));
  }
  c->n_lines = n_policy_lines;
  // cache_only: copies run on the caller's compute stream (src/cpp_worker/prefetcher.cpp:420-424)
  if (!c->cfg.cache_only) {
    PM_CUDA(cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
    PM_CUDA(cudaStreamCreateWithFlags(&c->prefetch_stream, cudaStreamNonBlocking));
  }
  c->line_copy_stream.assign(n_lines, nullptr);
  c->line_ready.resize(n_lines);
  for (auto& e : c->line_ready) PM_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  c->line_read.assign(n_lines, nullptr);
  c->line_pending.assign(n_lines, 0);
  c->line_waiter.assign(n_lines, nullptr);
  c->seg_events.resize(64);
  for (auto& e : c->seg_events) PM_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  PM_CUDA(cudaEventCreateWithFlags(&c->sync_event, cudaEventDisableTiming));
  PM_CUDA(cudaEventCreateWithFlags(&c->routed_event, cudaEventDisableTiming));
  PM_CUDA(cudaStreamCreateWithFlags(&c->readback_stream, cudaStreamNonBlocking));
  for (auto& l : c->layers) {
    PM_CUDA(cudaMalloc((void**)&l.slot_table_dev, (size_t)c->cfg.num_expert * 4));
    PM_CUDA(cudaMemset(l.slot_table_dev, 0xff, (size_t)c->cfg.num_expert * 4));
    l.slot_table_dirty = true;
  }
  c->slab_built = true;
  return PM_OK;
}

namespace {

// One grouped FFN launch: the experts in it, and the lines whose copies it has to wait for.
struct Segment {
  std::vector<pm_ffn_group> groups;
  std::vector<int> group_line;  // cache line of each group, -1 = shared expert
  std::vector<int> lines;
  std::vector<int> waits;
  bool has_line(int line) const { return std::find(lines.begin(), lines.end(), line) != lines.end(); }
  bool empty() const { return groups.empty(); }
};

}  // namespace

// The part of a layer call that follows the cache decisions: the ordered actions (copy an expert into
// a line, use an expert from a line), the launch being assembled, and where the walk over the
// actions stands. A call made through pm_moe_forward_routed_begin can stop here, hand the demand
// copies it has collected to the caller (who fetches them over all ranks' host links) and go on in
// pm_moe_forward_routed_end once the data is in the lines.
struct PendingForward {
  bool active = false;
  int layer = 0, T = 0, R = 0, n_shared = 0, k = 1, H = 0;
  bool spec = false, is_routed = false;
  pm_layer_weights w{};
  const __nv_bfloat16* x = nullptr;
  void* yv = nullptr;
  float* rows_out = nullptr;
  cudaStream_t s = nullptr;
  std::vector<Action> acts;
  size_t next = 0;
  std::vector<int64_t> ids;
  std::vector<int32_t> counts, offsets;
  std::vector<int> resident_line;
  Segment seg;
  size_t desc_used = 0;
  std::vector<Action> pooled;       // demand copies left to the caller
  std::vector<char> line_is_pooled;  // per cache line: its copy is among `pooled`
  bool seg_waits_for_pooled = false;
};

namespace {

// Prefill-size segment on the tcgen05 path: gather the token rows once per layer call, plan the
// 128 x 128 tiles, upload groups and tiles, launch the gate/up and the down kernel.
int flush_segment_tc(pm_ctx* c, Segment* seg, const pm_layer_weights& w, const __nv_bfloat16* x, int n_rows,
                     cudaStream_t s, bool q4 = false) {
  if (!c->xperm_ready) {
    PM_CUDA(launch_gather_rows(x, c->d_row_token, n_rows, (size_t)w.hidden * 2, c->d_xperm, s));
    c->kernel_launches += 1;
    c->xperm_ready = true;
  }
  if (q4) {
    if (!c->tc_maps_q4_ready) {
      int rc = tc_build_maps_q4(c, w, c->ws_tokens * (c->ws_topk + 1), &c->tc_maps_q4);
      if (rc != PM_OK) return rc;
      c->tc_maps_q4_ready = true;
    }
  } else if (!c->tc_maps_ready) {
    int rc = tc_build_maps(c, w, c->ws_tokens * (c->ws_topk + 1), &c->tc_maps);
    if (rc != PM_OK) return rc;
    c->tc_maps_ready = true;
  }
  std::vector<TcGroup> groups;
  for (size_t i = 0; i < seg->groups.size(); ++i) {
    const pm_ffn_group& g = seg->groups[i];
    if (g.row_count <= 0) continue;
    int line = seg->group_line[i];
    if (q4 && line >= 0) {
      // expand the expert's packed matrices into scratch line n (stream order keeps the line's earlier
      // readers ahead of this write); the tensor-core kernels then read bf16 as for any other expert
      line = (int)groups.size();
      unsigned char* dst = c->q4_scratch + (size_t)line * c->q4_scratch_stride;
      const size_t mat = (size_t)w.inter * w.hidden * 2;
      PM_CUDA(launch_dequant_q4(g.w_gate, g.q_gate, w.inter, w.hidden, (__nv_bfloat16*)dst, s));
      PM_CUDA(launch_dequant_q4(g.w_up, g.q_up, w.inter, w.hidden, (__nv_bfloat16*)(dst + mat), s));
      PM_CUDA(launch_dequant_q4(g.w_down, g.q_down, w.hidden, w.inter, (__nv_bfloat16*)(dst + 2 * mat), s));
      c->kernel_launches += 3;
      c->q4_expanded += 1;
    }
    groups.push_back(TcGroup{g.row_start, g.row_count, g.inter, line});
  }
  const TcMaps& maps = q4 ? c->tc_maps_q4 : c->tc_maps;
  std::vector<TcTile> gu, dn;
  tc_plan(groups, w.hidden, &gu, &dn);
  const size_t g_bytes = align_up(groups.size() * sizeof(TcGroup), 256);
  const size_t gu_bytes = align_up(gu.size() * sizeof(TcTile), 256), dn_bytes = align_up(dn.size() * sizeof(TcTile), 256);
  const size_t total = g_bytes + gu_bytes + dn_bytes;
  if (c->tc_plan_used + total > c->tc_plan_cap) return fail(PM_ERR_STATE, "prefill plan buffer overflow");
  unsigned char* h = c->h_tc_plan + c->tc_plan_used;
  unsigned char* d = c->d_tc_plan + c->tc_plan_used;
  std::memcpy(h, groups.data(), groups.size() * sizeof(TcGroup));
  std::memcpy(h + g_bytes, gu.data(), gu.size() * sizeof(TcTile));
  std::memcpy(h + g_bytes + gu_bytes, dn.data(), dn.size() * sizeof(TcTile));
  PM_CUDA(cudaMemcpyAsync(d, h, total, cudaMemcpyHostToDevice, s));
  c->tc_plan_used += total;
  pm_ctx::FfnSample sample{};
  if (c->profile_ffn) {
    PM_CUDA(cudaEventCreate(&sample.e0));
    PM_CUDA(cudaEventCreate(&sample.e1));
    PM_CUDA(cudaEventCreate(&sample.e2));
    for (const TcGroup& g : groups) {
      sample.bytes_gu += 4ll * g.inter * w.hidden;
      sample.bytes_dn += 2ll * g.inter * w.hidden;
    }
    PM_CUDA(cudaEventRecord(sample.e0, s));
  }
  PM_CUDA(launch_prefill_ffn(maps, (const TcGroup*)d, (const TcTile*)(d + g_bytes), (int)gu.size(),
                             (const TcTile*)(d + g_bytes + gu_bytes), (int)dn.size(), w.hidden, c->d_hbuf, c->ws_inter,
                             c->d_yexp, c->d_tc_err, s, c->profile_ffn ? sample.e1 : nullptr));
  if (c->profile_ffn) {
    PM_CUDA(cudaEventRecord(sample.e2, s));
    c->ffn_samples.push_back(sample);
  }
  c->kernel_launches += 2;
  c->tc_launches += 1;
  return PM_OK;
}

// Rows per expert from which uint4 experts are expanded to bf16 and run on the tensor
// cores: below it, re-reading the packed weights once per 16 rows is cheaper than writing and
// re-reading four times as many bf16 bytes.
constexpr int kQ4ExpandMinRows = 64;

// The bf16 scratch slab for `n` expanded experts (grown on demand, at least one line per expert of
// a layer). False if the device cannot provide it: the caller then stays on the split-K tiles.
bool q4_scratch_ready(pm_ctx* c, const pm_layer_weights& w, int n) {
  const size_t stride = align_up((size_t)3 * w.inter * w.hidden * 2, 256);
  const size_t lines = (size_t)std::max(n, c->cfg.num_expert);
  if (c->q4_scratch != nullptr && c->q4_scratch_stride == stride && c->q4_scratch_lines >= lines) return true;
  if (c->q4_scratch != nullptr) {
    cudaDeviceSynchronize();  // earlier launches may still read the old slab
    cudaFree(c->q4_scratch);
    c->q4_scratch = nullptr;
    c->q4_scratch_lines = 0;
  }
  if (cudaMalloc((void**)&c->q4_scratch, stride * lines) != cudaSuccess) {
    cudaGetLastError();
    c->q4_scratch = nullptr;
    return false;
  }
  c->q4_scratch_stride = stride;
  c->q4_scratch_lines = lines;
  c->tc_maps_q4_ready = false;
  return true;
}

int flush_segment(pm_ctx* c, Segment* seg, const pm_layer_weights& w, const __nv_bfloat16* x, int n_rows,
                  size_t* desc_used, cudaStream_t s) {
  if (seg->empty()) return PM_OK;
  for (int line : seg->waits) {
    if (c->line_pending[line] || c->line_waiter[line] != s) {
      PM_CUDA(cudaStreamWaitEvent(s, c->line_ready[line], 0));
      c->line_pending[line] = 0;
      c->line_waiter[line] = s;
    }
  }
  // Groups with many rows go to the tensor cores; the others stay on the split-K tiles, which stream
  // the weights faster when there are only a few rows to use them for (a large decode batch has both
  // kinds in one layer call). uint4 groups change over later: expanding an expert to bf16 costs more
  // than re-reading its packed weights a few times.
  const bool tc_ok = w.quant4 ? tc_prefill_usable_q4(c, w) : tc_prefill_usable(c, w);
  // Up to kMaxChunkRows rows a group runs as chunks of 16 rows through the split-K tiles (its weights
  // are read once from HBM and again from L2 for the later chunks): a 128-row tensor-core tile would be
  // mostly padding there, and a few such groups alone give that kernel too few CTAs to stream from.
  const int most_small = w.quant4 ? kQ4ExpandMinRows - 1 : kMaxChunkRows;
  Segment big;
  if (tc_ok) {
    size_t keep = 0;
    for (size_t i = 0; i < seg->groups.size(); ++i) {
      if (seg->groups[i].row_count > most_small) {
        big.groups.push_back(seg->groups[i]);
        big.group_line.push_back(seg->group_line[i]);
      } else {
        seg->groups[keep] = seg->groups[i];
        seg->group_line[keep] = seg->group_line[i];
        ++keep;
      }
    }
    seg->groups.resize(keep);
    seg->group_line.resize(keep);
    if (w.quant4 && !big.groups.empty() && !q4_scratch_ready(c, w, (int)big.groups.size())) {
      seg->groups.insert(seg->groups.end(), big.groups.begin(), big.groups.end());
      seg->group_line.insert(seg->group_line.end(), big.group_line.begin(), big.group_line.end());
      big.groups.clear();
      big.group_line.clear();
    }
  }
  if (!big.groups.empty()) {
    int rc = flush_segment_tc(c, &big, w, x, n_rows, s, w.quant4 != 0);
    if (rc != PM_OK) return rc;
  }
  if (seg->groups.empty()) {
    if (!seg->lines.empty()) {
      cudaEvent_t ev = next_seg_event(c);
      PM_CUDA(cudaEventRecord(ev, s));
      for (int line : seg->lines) c->line_read[line] = ev;
    }
    seg->lines.clear();
    seg->waits.clear();
    return PM_OK;
  }
  FfnPlanInfo info;
  // without the tensor-core path (shapes it cannot tile) larger groups stay in 64-row chunks for the staged kernel
  const int chunk_rows = (w.quant4 || tc_ok) ? kSplitMaxRows : kMaxChunkRows;
  int rc = plan_groups_size(seg->groups.data(), (int)seg->groups.size(), w.hidden, &info, chunk_rows);
  if (rc != PM_OK) return rc;
  if (*desc_used + info.blob_bytes() > c->plan_cap) return fail(PM_ERR_STATE, "launch plan buffer overflow");
  Stage st = stage_of(c);
  rc = plan_groups_into(seg->groups.data(), (int)seg->groups.size(), w.hidden, st.plan + *desc_used,
                        c->plan_cap - *desc_used, &info, chunk_rows);
  if (rc != PM_OK) return rc;
  PM_CUDA(cudaMemcpyAsync(c->d_plan + *desc_used, st.plan + *desc_used, info.blob_bytes(), cudaMemcpyHostToDevice, s));
  pm_ctx::FfnSample sample{};
  if (c->profile_ffn) {
    auto take_event = [&](cudaEvent_t* e) -> cudaError_t {
      if (!c->ffn_event_pool.empty()) {
        *e = c->ffn_event_pool.back();
        c->ffn_event_pool.pop_back();
        return cudaSuccess;
      }
      return cudaEventCreate(e);
    };
    sample.fused = ffn_launch_is_fused(info, w.quant4);
    PM_CUDA(take_event(&sample.e0));
    if (!sample.fused) PM_CUDA(take_event(&sample.e1));
    PM_CUDA(take_event(&sample.e2));
    for (const pm_ffn_group& g : seg->groups) {
      int64_t mat = (int64_t)g.inter * w.hidden;
      // uint4: half a byte per weight plus one fp16 {scale, zero} pair per 128 weights
      int64_t one = w.quant4 ? mat / 2 + mat / 128 * 4 : mat * 2;
      sample.bytes_gu += 2 * one;
      sample.bytes_dn += one;
    }
    PM_CUDA(cudaEventRecord(sample.e0, s));
  }
  PM_CUDA(launch_swiglu_ffn(c->d_plan + *desc_used, info, w.quant4, x, w.hidden, c->d_row_token, c->d_hbuf,
                            c->ws_inter, c->d_yexp, s, (c->profile_ffn && !sample.fused) ? sample.e1 : nullptr,
                            c->d_tc_err));
  if (c->profile_ffn) {
    PM_CUDA(cudaEventRecord(sample.e2, s));
    c->ffn_samples.push_back(sample);
  }
  c->kernel_launches += ffn_launch_is_fused(info, w.quant4) ? 1 : 2;
  *desc_used += align_up(info.blob_bytes(), 256);
  if (!seg->lines.empty()) {
    cudaEvent_t ev = next_seg_event(c);
    PM_CUDA(cudaEventRecord(ev, s));
    for (int line : seg->lines) c->line_read[line] = ev;
  }
  seg->groups.clear();
  seg->group_line.clear();
  seg->lines.clear();
  seg->waits.clear();
  (void)n_rows;
  return PM_OK;
}

}  // namespace

namespace {

pm_ffn_group group_of_line(pm_ctx* c, const PendingForward& p, int e, int line) {
  const unsigned char* base = line_ptr(c, line);
  pm_ffn_group g{};
  g.w_gate = base + c->param_offset[c->role_gate];
  g.w_up = base + c->param_offset[c->role_up];
  g.w_down = base + c->param_offset[c->role_down];
  if (p.w.quant4) {
    g.q_gate = base + c->param_offset[c->role_qgate];
    g.q_up = base + c->param_offset[c->role_qup];
    g.q_down = base + c->param_offset[c->role_qdown];
  }
  g.row_start = p.offsets[e];
  g.row_count = p.counts[e];
  g.inter = p.w.inter;
  return g;
}

// Walks the actions from p.next on. With `collect`, full-record demand copies are not enqueued but
// collected in p.pooled (their lines are marked pending, so the launches that read them wait for
// the lines' ready events, which the caller's fetch records). The walk stops (*stopped = true)
// where a launch would have to be enqueued that waits for a collected copy; the caller resumes it
// with collect = false once those events have been recorded.
int run_actions(pm_ctx* c, PendingForward& p, bool collect, bool* stopped) {
  const int n_rows = p.R + p.n_shared * p.T;
  const int N = c->cfg.num_per_expert_param();
  cudaStream_t s = p.s;
  *stopped = false;
  for (; p.next < p.acts.size(); ++p.next) {
    const Action& a = p.acts[p.next];
    if (a.type == Action::kCopy) {
      if (p.seg.has_line(a.line)) {  // the victim is still waiting to run in the open segment
        if (collect && p.seg_waits_for_pooled) {
          *stopped = true;
          return PM_OK;
        }
        int rc = flush_segment(c, &p.seg, p.w, p.x, n_rows, &p.desc_used, s);
        if (rc != PM_OK) return rc;
        p.seg_waits_for_pooled = false;
      }
      if (collect && a.precise && a.chunk_begin == 0 && a.chunk_end == N && !c->stable_va) {
        p.pooled.push_back(a);
        p.line_is_pooled[a.line] = 1;
        c->line_pending[a.line] = 1;
        c->line_waiter[a.line] = nullptr;
        c->h2d_bytes += (int64_t)c->param_offset[N];
        c->h2d_copies += 1;
      } else {
        int rc = enqueue_copy(c, a);
        if (rc != PM_OK) return rc;
      }
    } else {
      // Already computed by the device-planned launch from the line it occupied at that time.
      if (p.spec && p.resident_line[a.expert] >= 0) continue;
      const bool must_wait = c->line_pending[a.line] || (c->line_waiter[a.line] != nullptr && c->line_waiter[a.line] != s);
      if (must_wait && p.seg.waits.empty() && !p.seg.empty()) {
        // let everything that is already resident run while the copies are in flight
        int rc = flush_segment(c, &p.seg, p.w, p.x, n_rows, &p.desc_used, s);
        if (rc != PM_OK) return rc;
      }
      p.seg.groups.push_back(group_of_line(c, p, a.expert, a.line));
      p.seg.group_line.push_back(a.line);
      p.seg.lines.push_back(a.line);
      if (must_wait) {
        p.seg.waits.push_back(a.line);
        if (p.line_is_pooled[a.line]) p.seg_waits_for_pooled = true;
      }
    }
  }
  if (collect && p.seg_waits_for_pooled) {
    *stopped = true;
    return PM_OK;
  }
  return flush_segment(c, &p.seg, p.w, p.x, n_rows, &p.desc_used, s);
}

int finish_forward(pm_ctx* c, PendingForward& p) {
  if (p.is_routed) {
    PM_CUDA(launch_gather_rows(c->d_yexp, c->d_pos, p.T, (size_t)p.H * 4, p.rows_out, p.s));
  } else {
    PM_CUDA(launch_combine(c->d_yexp, c->d_pos, c->d_topk_w, p.T, p.H, p.k, p.R, p.n_shared,
                           p.w.shared_gate_w ? c->d_shared_scale : nullptr, (__nv_bfloat16*)p.yv, p.s));
  }
  c->kernel_launches += 1;
  for (int64_t id : p.ids) c->eng->expert_done(p.layer, (int)id);
  c->eng->layer_done(p.layer);
  return PM_OK;
}

}  // namespace

int rt_forward(pm_ctx* c, int layer, const void* xv, int T, void* yv, cudaStream_t s, const RoutedRows* routed) {
  if (!c->slab_built) return fail(PM_ERR_STATE, "moe_forward before build_slab");
  if (layer < 0 || layer >= c->cfg.num_layer) return fail(PM_ERR_INVALID, "layer out of range");
  if (!c->pending) c->pending = new PendingForward();
  if (c->pending->active) return fail(PM_ERR_STATE, "a layer call begun with pm_moe_forward_routed_begin has not been ended");
  pm_ctx::Layer& ly = c->layers[layer];
  if (!ly.set) return fail(PM_ERR_STATE, "moe_forward before layer_set_weights");
  if (T < 0) return fail(PM_ERR_INVALID, "negative token count");
  if (T == 0) return PM_OK;
  if (!xv || (!yv && !routed)) return fail(PM_ERR_INVALID, "null activation pointer");
  if (routed && (!routed->row_expert || !routed->rows_out)) return fail(PM_ERR_INVALID, "null routed-row pointer");
  const pm_layer_weights& w = ly.w;
  if (!routed && w.gate_w == nullptr) return fail(PM_ERR_STATE, "this layer has no router weights (routed rows only)");
  const int E = c->cfg.num_expert, k = routed ? 1 : w.top_k, H = w.hidden, N = c->cfg.num_per_expert_param();
  const int R = T * k;
  // Decode batches give every slice of the shared expert its own output rows (the combine adds them);
  // larger batches keep the shared expert whole.
  const bool has_shared = !routed && w.shared_inter > 0;
  const bool sliced = has_shared && T <= kSplitMaxRows && !w.quant4;
  const int n_shared = !has_shared ? 0 : (sliced ? shared_slice_count(w.inter, w.shared_inter) : 1);
  int rc = ensure_workspace(c, T, w);
  if (rc != PM_OK) return rc;
  if (c->have_last_stream && c->last_stream != s) PM_CUDA(cudaStreamSynchronize(c->last_stream));
  c->last_stream = s;
  c->have_last_stream = true;
  const __nv_bfloat16* x = (const __nv_bfloat16*)xv;
  Stage st = stage_of(c);

  // Refresh this layer's expert -> slot table if the cache changed since the last upload.
  if (ly.slot_table_dirty) {
    for (int e = 0; e < E; ++e) st.slot_table[e] = c->eng->slot_of(layer, e);
    PM_CUDA(cudaMemcpyAsync(ly.slot_table_dev, st.slot_table, (size_t)E * 4, cudaMemcpyHostToDevice, s));
    ly.slot_table_dirty = false;
  }
  const int32_t* ids_dev = c->d_topk_ids;
  if (routed) {
    ids_dev = routed->row_expert;
  } else {
    PM_CUDA(launch_gate_topk(x, (const __nv_bfloat16*)w.gate_w, w.gate_bias, (const __nv_bfloat16*)w.shared_gate_w,
                             T, H, E, k, w.norm_topk, w.routed_scale, ly.slot_table_dev, c->d_topk_ids,
                             c->d_topk_w, c->d_topk_slot, c->d_shared_scale, nullptr, s));
    c->kernel_launches += 1;
  }
  // rows per expert <= T, or the bound the caller of the routed-rows form guarantees
  const int row_bound = (routed && routed->max_rows_per_expert > 0) ? std::min(T, routed->max_rows_per_expert) : T;
  const bool spec = c->device_plan && !w.quant4 && resident_ffn_available(row_bound);
  PM_CUDA(launch_permute(ids_dev, R, k, E, c->d_counts, c->d_offsets, c->d_row_token, c->d_pos, c->d_err,
                         n_shared * T, T, s, c->d_perm_scratch, c->perm_scratch_ints,
                         spec ? c->d_res_counters : nullptr, kMaxFusedGroups + 1));
  c->kernel_launches += 1;
  std::vector<int> pred_dsts;
  if (!routed && c->cfg.predict_from_moe_input && c->seq_len == 1) {
    rc = launch_predictors(c, layer, x, T, H, s, &pred_dsts);
    if (rc != PM_OK) return rc;
  }
  const bool routed_pred = routed && routed->n_pred > 0 && routed->pred_scores != nullptr && c->seq_len == 1;
  const int L_all = c->cfg.num_layer;
  bool routed_ranked = false;
  if (routed_pred && routed->n_pred <= L_all) {
    routed_ranked = true;
    for (int i = 0; i < routed->n_pred; ++i) {
      const int dst = routed->pred_layers[i];
      if (dst < 0 || dst >= L_all) return fail(PM_ERR_INVALID, "predicted layer out of range");
      if (!topn_on_device(c, prediction_count(c, dst, routed->pred_width, routed->pred_top), routed->pred_width))
        routed_ranked = false;
    }
    if (routed_ranked) {
      rc = ensure_topn(c);
      if (rc != PM_OK) return rc;
      for (int i = 0; i < routed->n_pred; ++i) {
        const int n = prediction_count(c, routed->pred_layers[i], routed->pred_width, routed->pred_top);
        PM_CUDA(launch_rank_topn(routed->pred_scores + (size_t)i * routed->pred_width, routed->pred_width, n,
                                 c->d_topn + (size_t)(L_all + i) * kTopCap, s));
        c->kernel_launches += 1;
        c->topn_launches += 1;
      }
    }
  }
  // The router's results travel to the host on a side stream, so the resident experts can start on
  // the compute stream at once instead of waiting for the host's decisions about the misses.
  PM_CUDA(cudaEventRecord(c->routed_event, s));
  cudaStream_t rb = c->readback_stream;
  PM_CUDA(cudaStreamWaitEvent(rb, c->routed_event, 0));
  const bool own_ranked = !pred_dsts.empty() && c->d_topn != nullptr &&
                          topn_on_device(c, prediction_count(c, pred_dsts.back(), E, -1), E);
  if (routed_ranked || own_ranked)
    PM_CUDA(cudaMemcpyAsync(c->h_topn, c->d_topn, (size_t)2 * L_all * kTopCap * 4, cudaMemcpyDeviceToHost, rb));
  const bool need_scores = c->cfg.cache_policy == "nn";  // the NN policy updates its priorities from the scores
  if (routed_pred && (need_scores || !routed_ranked)) {
    // scores computed elsewhere (the expert-parallel sources): they ride to the host with the counts
    const size_t bytes = (size_t)routed->n_pred * routed->pred_width * 4;
    if (routed->n_pred > c->cfg.num_layer) return fail(PM_ERR_INVALID, "more predicted layers than layers");
    for (int i = 0; i < routed->n_pred; ++i)
      if (routed->pred_layers[i] < 0 || routed->pred_layers[i] >= c->cfg.num_layer)
        return fail(PM_ERR_INVALID, "predicted layer out of range");
    if (c->h_routed_scores_cap < bytes) {
      if (c->h_routed_scores) PM_CUDA(cudaFreeHost(c->h_routed_scores));
      c->h_routed_scores = nullptr;
      PM_CUDA(cudaHostAlloc((void**)&c->h_routed_scores, bytes, cudaHostAllocDefault));
      c->h_routed_scores_cap = bytes;
    }
    PM_CUDA(cudaMemcpyAsync(c->h_routed_scores, routed->pred_scores, bytes, cudaMemcpyDeviceToHost, rb));
  } else if (!pred_dsts.empty() && (need_scores || !own_ranked)) {
    PM_CUDA(cudaMemcpyAsync(st.scores, c->d_scores, (size_t)c->cfg.num_layer * E * 4, cudaMemcpyDeviceToHost, rb));
  }
  PM_CUDA(cudaMemcpyAsync(st.counts, c->d_counts, (size_t)(2 * E + 3) * 4, cudaMemcpyDeviceToHost, rb));
  const bool keep = c->keep_routing && !routed;
  if (keep) {
    PM_CUDA(cudaMemcpyAsync(st.ids, c->d_topk_ids, (size_t)R * 4, cudaMemcpyDeviceToHost, rb));
    PM_CUDA(cudaMemcpyAsync(st.w, c->d_topk_w, (size_t)R * 4, cudaMemcpyDeviceToHost, rb));
  }
  PM_CUDA(cudaEventRecord(c->sync_event, rb));

  // Experts resident right now (the device slot table shows the same state).
  std::vector<int> resident_line(E, -1);
  pm_ctx::FfnSample spec_sample{};
  if (spec) {
    for (int e = 0; e < E; ++e) {
      const int line = c->eng->expert(layer, e).line;
      resident_line[e] = line;
      if (line < 0) continue;
      if (c->line_pending[line] || (c->line_waiter[line] != nullptr && c->line_waiter[line] != s)) {
        PM_CUDA(cudaStreamWaitEvent(s, c->line_ready[line], 0));  // a prefetch into the line may be in flight
        c->line_pending[line] = 0;
        c->line_waiter[line] = s;
      }
    }
    ResidentArgs a{};
    const Pool& pool = c->eng->pools()[c->eng->pool_index(layer)];
    a.counts = c->d_counts;
    a.offsets = c->d_offsets;
    a.slot_table = ly.slot_table_dev;
    a.pool_base = line_ptr(c, pool.base);
    a.line_stride = c->line_stride;
    a.off_gate = c->param_offset[c->role_gate];
    a.off_up = c->param_offset[c->role_up];
    a.off_down = c->param_offset[c->role_down];
    a.shared_w_gate = w.shared_w_gate;
    a.shared_w_up = w.shared_w_up;
    a.shared_w_down = w.shared_w_down;
    a.num_expert = E;
    a.inter = w.inter;
    a.shared_inter = has_shared ? w.shared_inter : 0;
    a.shared_slice = has_shared ? shared_slice_width(w.inter, w.shared_inter) : 0;
    a.tokens = T;
    a.n_routed_rows = R;
    if (c->profile_ffn) {
      auto take_event = [&](cudaEvent_t* e) -> cudaError_t {
        if (!c->ffn_event_pool.empty()) {
          *e = c->ffn_event_pool.back();
          c->ffn_event_pool.pop_back();
          return cudaSuccess;
        }
        return cudaEventCreate(e);
      };
      spec_sample.fused = true;
      spec_sample.resident = true;
      PM_CUDA(take_event(&spec_sample.e0));
      PM_CUDA(take_event(&spec_sample.e2));
      PM_CUDA(cudaEventRecord(spec_sample.e0, s));
    }
    PM_CUDA(launch_resident_ffn(a, c->d_res_counters, c->d_tc_err, row_bound, x, H, c->d_row_token, c->d_hbuf,
                                c->ws_inter, c->d_yexp, s));
    if (c->profile_ffn) PM_CUDA(cudaEventRecord(spec_sample.e2, s));
    c->kernel_launches += 1;
    cudaEvent_t ev = next_seg_event(c);
    PM_CUDA(cudaEventRecord(ev, s));
    for (int e = 0; e < E; ++e)
      if (resident_line[e] >= 0) c->line_read[resident_line[e]] = ev;
  }
  rc = wait_event(c->sync_event, 30.0);
  if (rc != PM_OK) return rc;
  // everything enqueued by earlier layer calls has finished: the staging buffers may be reused, and
  // an error the prefill kernel of an earlier call recorded is visible now
  c->tc_plan_used = 0;
  c->xperm_ready = false;
  c->tc_maps_ready = false;
  c->tc_maps_q4_ready = false;
  if (c->profile_ffn && !c->ffn_samples.empty()) {  // their events have fired: recycle them now
    rc = rt_profile_collect(c);
    if (rc != PM_OK) return rc;
  }
  if (st.counts[2 * E + 2] != 0) {
    // written by an FFN kernel of an earlier layer call (everything enqueued before this call's router
    // has finished by now): a bounded wait gave up
    const int code = st.counts[2 * E + 2];
    PM_CUDA(cudaMemsetAsync(c->d_tc_err, 0, 4, s));
    return fail(PM_ERR_TIMEOUT, "an expert FFN kernel of the previous layer call gave up a bounded wait (code " +
                                    std::to_string(code) + ")");
  }
  if (st.counts[2 * E + 1] != 0) {
    // only the caller's row_expert can be out of range (the router's ids never are); the rows were
    // dropped by the permutation, so nothing may be returned for this call
    PM_CUDA(cudaMemsetAsync(c->d_err, 0, 4, s));
    return fail(PM_ERR_INVALID, "an expert id outside [0, num_expert) was passed for a routed row");
  }
  if (keep) {
    c->last_ids[layer].assign(st.ids, st.ids + R);
    c->last_w[layer].assign(st.w, st.w + R);
  }

  // Prediction made from this layer's input comes before the layer's own report, as in the
  // reference (report_moe_layer_logits precedes report_one_layer for the same index).
  for (int dst : pred_dsts) {
    const bool dev = own_ranked && topn_on_device(c, prediction_count(c, dst, E, -1), E);
    rc = issue_prediction(c, dst, st.scores + (size_t)dst * E, 0, 0, -1,
                          dev ? c->h_topn + (size_t)dst * kTopCap : nullptr);
    if (rc != PM_OK) return rc;
  }
  if (routed_pred)
    for (int i = 0; i < routed->n_pred; ++i) {
      rc = issue_prediction(c, routed->pred_layers[i],
                            c->h_routed_scores != nullptr ? c->h_routed_scores + (size_t)i * routed->pred_width : nullptr,
                            routed->pred_width, routed->pred_first, routed->pred_top,
                            routed_ranked ? c->h_topn + (size_t)(L_all + i) * kTopCap : nullptr);
      if (rc != PM_OK) return rc;
    }

  const int32_t* counts = st.counts;
  const int32_t* offsets = st.counts + E;
  std::vector<int64_t> ids;
  for (int e = 0; e < E; ++e)
    if (counts[e] > 0) ids.push_back(e);
  std::vector<Action> acts;
  std::string err = c->eng->report_layer(layer, ids.data(), (int64_t)ids.size(), &acts);
  if (!err.empty()) return fail(PM_ERR_STATE, err);
  if (!c->cfg.early_preempt) {
    for (int64_t id : ids) {
      err = c->eng->report_expert(layer, (int)id, &acts);
      if (!err.empty()) return fail(PM_ERR_STATE, err);
    }
  }
  rt_mark_dirty(c, acts);

  if (spec && c->profile_ffn) {  // weight bytes the device-planned launch read: shared + activated residents
    const int64_t routed = (int64_t)w.inter * H * 2, sh = (int64_t)w.shared_inter * H * 2;
    int64_t n_res = 0;
    for (int e = 0; e < E; ++e)
      if (counts[e] > 0 && resident_line[e] >= 0) ++n_res;
    spec_sample.bytes_gu = 2 * (n_res * routed + sh);
    spec_sample.bytes_dn = n_res * routed + sh;
    c->ffn_samples.push_back(spec_sample);
  }

  PendingForward& p = *c->pending;
  p = PendingForward();
  p.layer = layer; p.T = T; p.R = R; p.n_shared = n_shared; p.k = k; p.H = H;
  p.spec = spec; p.is_routed = routed != nullptr;
  p.w = w; p.x = x; p.yv = yv; p.rows_out = routed ? routed->rows_out : nullptr; p.s = s;
  p.acts = std::move(acts);
  p.ids = ids;
  p.counts.assign(counts, counts + E);
  p.offsets.assign(offsets, offsets + E + 1);
  p.resident_line = resident_line;
  p.line_is_pooled.assign(c->line_pending.size(), 0);
  if (n_shared && !spec) {
    const int slice = sliced ? shared_slice_width(w.inter, w.shared_inter) : w.shared_inter;
    for (int j = 0; j < n_shared; ++j) {
      pm_ffn_group g{};
      g.w_gate = (const unsigned char*)w.shared_w_gate + (size_t)j * slice * H * 2;
      g.w_up = (const unsigned char*)w.shared_w_up + (size_t)j * slice * H * 2;
      g.w_down = (const unsigned char*)w.shared_w_down + (size_t)j * slice * 2;
      g.row_start = R + j * T;
      g.row_count = T;
      g.inter = std::min(slice, w.shared_inter - j * slice);
      g.ld_down = w.shared_inter;
      p.seg.groups.push_back(g);
      p.seg.group_line.push_back(-1);
    }
  }
  const bool collect = routed != nullptr && routed->collect_demand_copies && !c->cfg.cache_only;
  bool stopped = false;
  rc = run_actions(c, p, collect, &stopped);
  if (rc != PM_OK) return rc;
  if (stopped) {  // the caller fetches p.pooled, then calls rt_forward_end
    p.active = true;
    return PM_OK;
  }
  (void)N;
  return finish_forward(c, p);
}

int rt_forward_end(pm_ctx* c) {
  if (!c->pending || !c->pending->active) return PM_OK;  // the begin call had nothing left to do
  PendingForward& p = *c->pending;
  if (!p.active) return PM_OK;  // the begin call had nothing left to do
  p.active = false;
  bool stopped = false;
  int rc = run_actions(c, p, false, &stopped);
  if (rc != PM_OK) return rc;
  return finish_forward(c, p);
}

const std::vector<Action>& rt_pending_pooled(pm_ctx* c) {
  static const std::vector<Action> none;
  return c->pending ? c->pending->pooled : none;
}

int rt_forward_host(pm_ctx* c, int layer, const void* x, int T, void* y, cudaStream_t s) {
  if (layer < 0 || layer >= c->cfg.num_layer || !c->layers[layer].set)
    return fail(PM_ERR_STATE, "moe_forward_host: layer not configured");
  if (T <= 0) return T == 0 ? PM_OK : fail(PM_ERR_INVALID, "negative token count");
  if (!x || !y) return fail(PM_ERR_INVALID, "null activation pointer");
  const pm_layer_weights& w = c->layers[layer].w;
  int rc = ensure_workspace(c, T, w);
  if (rc != PM_OK) return rc;
  const size_t bytes = (size_t)T * w.hidden * 2;
  PM_CUDA(cudaMemcpyAsync(c->d_xin, x, bytes, cudaMemcpyHostToDevice, s));
  rc = rt_forward(c, layer, c->d_xin, T, c->d_yout, s);
  if (rc != PM_OK) return rc;
  PM_CUDA(cudaMemcpyAsync(y, c->d_yout, bytes, cudaMemcpyDeviceToHost, s));
  PM_CUDA(cudaStreamSynchronize(s));
  return PM_OK;
}

// The per-expert path: the caller computes the expert itself on `s` from the line's address.
int rt_expert_acquire(pm_ctx* c, int layer, int expert, cudaStream_t s, void** line_out) {
  if (!c->slab_built) return fail(PM_ERR_STATE, "expert_acquire before build_slab");
  if (layer < 0 || layer >= c->cfg.num_layer || expert < 0 || expert >= c->cfg.num_expert || !line_out)
    return fail(PM_ERR_INVALID, "layer or expert out of range");
  *line_out = nullptr;
  std::vector<Action> acts;
  std::string err = c->eng->report_expert(layer, expert, &acts);
  if (!err.empty()) return fail(PM_ERR_STATE, err);
  rt_mark_dirty(c, acts);
  int rc = rt_execute_copies(c, acts);
  if (rc != PM_OK) return rc;
  const int line = c->eng->expert(layer, expert).line;
  if (line < 0) return fail(PM_ERR_STATE, "the expert has no cache line after report_one_expert (report_one_layer missing?)");
  if (c->line_pending[line] || (c->line_waiter[line] != nullptr && c->line_waiter[line] != s)) {
    PM_CUDA(cudaStreamWaitEvent(s, c->line_ready[line], 0));
    c->line_pending[line] = 0;
    c->line_waiter[line] = s;
  }
  *line_out = c->stable_va ? (void*)(c->expert_va + ((size_t)layer * c->cfg.num_expert + expert) * c->line_stride)
                           : (void*)line_ptr(c, line);
  return PM_OK;
}

int rt_expert_release(pm_ctx* c, int layer, int expert, cudaStream_t s) {
  if (!c->slab_built) return fail(PM_ERR_STATE, "expert_release before build_slab");
  if (layer < 0 || layer >= c->cfg.num_layer || expert < 0 || expert >= c->cfg.num_expert)
    return fail(PM_ERR_INVALID, "layer or expert out of range");
  const int line = c->eng->expert(layer, expert).line;
  if (line >= 0) {  // a later copy into this line waits for the caller's kernels
    cudaEvent_t ev = next_seg_event(c);
    PM_CUDA(cudaEventRecord(ev, s));
    c->line_read[line] = ev;
  }
  std::string err = c->eng->expert_done(layer, expert);
  if (!err.empty()) return fail(PM_ERR_INVALID, err);
  return PM_OK;
}

int rt_temp_move(pm_ctx* c, int layer, int expert, bool to_gpu, cudaStream_t s, void** line_out) {
  if (!c->slab_built) return fail(PM_ERR_STATE, "temp_move_expert before build_slab");
  if (layer < 0 || layer >= c->cfg.num_layer || expert < 0 || expert >= c->cfg.num_expert)
    return fail(PM_ERR_INVALID, "layer or expert out of range");
  unsigned char* spare = line_ptr(c, c->n_lines);
  unsigned char* rec = c->host_rec[(size_t)layer * c->cfg.num_expert + expert];
  const size_t bytes = c->param_offset.back();
  if (to_gpu) {
    PM_CUDA(cudaMemcpyAsync(spare, rec, bytes, cudaMemcpyHostToDevice, s));
  } else {
    PM_CUDA(cudaMemcpyAsync(rec, spare, bytes, cudaMemcpyDeviceToHost, s));
  }
  PM_CUDA(cudaStreamSynchronize(s));
  if (line_out) *line_out = spare;
  return PM_OK;
}

int rt_report_hidden(pm_ctx* c, int index, const void* hidden, int B, int seq, cudaStream_t s) {
  if (index < 0 || index > c->cfg.num_layer) return fail(PM_ERR_INVALID, "hidden-state index out of range");
  if (seq != 1 || B <= 0) return PM_OK;  // prefill or empty: nothing is captured (predictor.cpp:657-661)
  {
    // nothing to run for this index (no predictor registered, or prediction off): not an error, the
    // hook reports every layer's hidden states whether or not a predictor exists
    const int L = c->cfg.num_layer;
    bool any = false;
    if (c->cfg.predict_input_mode == "moe_layer_logits" && c->cfg.num_predict_expert_per_layer > 0)
      for (int dst = 0; dst < L && !any; ++dst) any = c->predictors[(size_t)index * L + dst].w1 != nullptr;
    if (!any) return PM_OK;
  }
  if (!c->slab_built) return fail(PM_ERR_STATE, "report_hidden before build_slab");
  int H = 0;
  for (auto& l : c->layers)
    if (l.set) H = l.w.hidden;
  if (H == 0) return fail(PM_ERR_STATE, "report_hidden before layer_set_weights");
  pm_layer_weights shape{};
  shape.hidden = H;
  shape.top_k = std::max(1, c->ws_topk);
  int rc = ensure_workspace(c, B, shape);
  if (rc != PM_OK) return rc;
  std::vector<int> dsts;
  rc = launch_predictors(c, index, (const __nv_bfloat16*)hidden, B, H, s, &dsts);
  if (rc != PM_OK || dsts.empty()) return rc;
  Stage st = stage_of(c);
  const int E = c->cfg.num_expert;
  PM_CUDA(cudaMemcpyAsync(st.scores, c->d_scores, (size_t)c->cfg.num_layer * E * 4, cudaMemcpyDeviceToHost, s));
  PM_CUDA(cudaEventRecord(c->sync_event, s));
  rc = wait_event(c->sync_event, 30.0);
  if (rc != PM_OK) return rc;
  for (int dst : dsts) {
    rc = issue_prediction(c, dst, st.scores + (size_t)dst * E);
    if (rc != PM_OK) return rc;
  }
  return PM_OK;
}

}  // namespace pm

pm_ctx::~pm_ctx() {
  delete pending;
  // Best effort: the context may die with work in flight only if the caller ignored errors.
  if (have_last_stream) cudaStreamSynchronize(last_stream);
  for (cudaStream_t cs : {copy_stream, prefetch_stream})
    if (cs) {
      cudaStreamSynchronize(cs);
      cudaStreamDestroy(cs);
    }
  for (auto e : line_ready) cudaEventDestroy(e);
  for (auto e : seg_events) cudaEventDestroy(e);
  if (sync_event) cudaEventDestroy(sync_event);
  if (routed_event) cudaEventDestroy(routed_event);
  if (readback_stream) {
    cudaStreamSynchronize(readback_stream);
    cudaStreamDestroy(readback_stream);
  }
  for (auto& f : ffn_samples) {
    cudaEventDestroy(f.e0);
    if (f.e1) cudaEventDestroy(f.e1);
    cudaEventDestroy(f.e2);
  }
  for (auto e : ffn_event_pool) cudaEventDestroy(e);
  for (auto& l : layers)
    if (l.slot_table_dev) cudaFree(l.slot_table_dev);
  if (ws_dev) cudaFree(ws_dev);
  if (h_stage) cudaFreeHost(h_stage);
  if (h_tc_plan) cudaFreeHost(h_tc_plan);
  if (q4_scratch) cudaFree(q4_scratch);
  if (d_topn) cudaFree(d_topn);
  if (h_topn) cudaFreeHost(h_topn);
  if (h_routed_scores) cudaFreeHost(h_routed_scores);
  if (slab_built) {
    if (slab_vmm) {
      pm::Driver& d = pm::driver();
      if (expert_va != nullptr) {
        for (size_t i = 0; i < line_mapped_to.size(); ++i)
          if (line_mapped_to[i] >= 0) d.Unmap((CUdeviceptr)(expert_va + (size_t)line_mapped_to[i] * line_stride), line_stride);
        d.AddressFree((CUdeviceptr)expert_va, expert_va_bytes);
      }
      d.Unmap((CUdeviceptr)slab, slab_va_bytes);
      for (auto h : line_handles) d.Release(h);
      d.AddressFree((CUdeviceptr)slab, slab_va_bytes);
    } else {
      cudaFree(slab);
    }
  }
  if (shared_prefix.empty()) {
    for (void* b : arena_blocks) cudaFreeHost(b);
  }
  pm::rt_release_shared_blocks(this);
}
