#include "cache_engine.hpp"

#include <algorithm>
#include <cmath>
#include <queue>

namespace pm {

// ------------------------------------------------------------------------------------------
// Eviction policies. Experts are named by their flat id (layer * num_expert + expert).
// ------------------------------------------------------------------------------------------
class Policy {
 public:
  virtual ~Policy() = default;
  virtual int victim() = 0;
  virtual std::string evict(int f) = 0;
  virtual std::string on_hit(int f, bool precise) { return ""; }
  virtual std::string on_miss(int f, bool precise) = 0;
  virtual void refresh_all() {}
  virtual void set_priority(int f, float p) {}
  virtual std::string set_cur_seq(uint64_t seq) { return ""; }
};

namespace {

// Least recently used: a doubly linked list threaded through two index arrays; head side is
// the next victim (src/cpp_worker/cache.hpp:33-56, src/cpp_worker/cache.cpp:321-339).
class LruPolicy : public Policy {
 public:
  explicit LruPolicy(int n_flat) : prev_(n_flat + 2, -1), next_(n_flat + 2, -1), head_(n_flat), tail_(n_flat + 1) {
    next_[head_] = tail_;
    prev_[tail_] = head_;
  }
  int victim() override { return next_[head_] == tail_ ? -1 : next_[head_]; }
  std::string evict(int f) override {
    unlink(f);
    return "";
  }
  std::string on_hit(int f, bool) override {
    if (prev_[f] < 0) return "lru: hit on an expert the policy does not hold";
    unlink(f);
    append(f);
    return "";
  }
  std::string on_miss(int f, bool) override {
    if (prev_[f] >= 0) return "lru: miss on an expert the policy already holds";
    append(f);
    return "";
  }

 private:
  void unlink(int f) {
    next_[prev_[f]] = next_[f];
    prev_[next_[f]] = prev_[f];
    prev_[f] = next_[f] = -1;
  }
  void append(int f) {
    int last = prev_[tail_];
    next_[last] = f;
    prev_[f] = last;
    next_[f] = tail_;
    prev_[tail_] = f;
  }
  std::vector<int> prev_, next_;
  int head_, tail_;
};

// First in, first out (src/cpp_worker/cache.hpp:24-31, src/cpp_worker/cache.cpp:313-320).
class FifoPolicy : public Policy {
 public:
  int victim() override { return q_.empty() ? -1 : q_.front(); }
  std::string evict(int f) override {
    if (q_.empty() || q_.front() != f) return "fifo: evicting an expert that is not the oldest";
    q_.pop_front();
    return "";
  }
  std::string on_miss(int f, bool) override {
    q_.push_back(f);
    return "";
  }

 private:
  std::deque<int> q_;
};

// "static-n": the last n entrants rotate first-in-first-out, everything that entered earlier
// stays for good (src/cpp_worker/cache.cpp:340-381).
class StaticPolicy : public Policy {
 public:
  explicit StaticPolicy(int rotating) : rotating_(rotating) {}
  int victim() override { return alt_.empty() ? -1 : alt_.front(); }
  std::string evict(int f) override {
    auto it = std::find(alt_.begin(), alt_.end(), f);
    if (it == alt_.end()) return "static: evicting a pinned or unknown expert";
    alt_.erase(it);
    return "";
  }
  std::string on_miss(int f, bool) override {
    if ((int)alt_.size() == rotating_) alt_.pop_front();  // the oldest rotating entry becomes permanent
    alt_.push_back(f);
    return "";
  }

 private:
  int rotating_;
  std::deque<int> alt_;
};

// Binary min-heap over flat ids with position tracking. Sift rules, the rebuild sweep and the
// removal (swap with the last element, then sift DOWN only) follow
// src/cpp_worker/utils.hpp:270-357 exactly, because victim choice among equal or stale
// priorities depends on them.
class IndexedMinHeap {
 public:
  explicit IndexedMinHeap(int n_flat) : prio_(n_flat, 0.f), at_(n_flat, -1) {}
  bool holds(int f) const { return at_[f] >= 0; }
  int top() const { return buf_.empty() ? -1 : buf_[0]; }
  float& prio(int f) { return prio_[f]; }
  const std::vector<int>& items() const { return buf_; }
  void push(int f, float p) {
    prio_[f] = p;
    at_[f] = (int)buf_.size();
    buf_.push_back(f);
    up(at_[f]);
  }
  void update(int f, float p) {
    float old = prio_[f];
    prio_[f] = p;
    if (p < old) up(at_[f]); else down(at_[f]);
  }
  void remove(int f) {
    int i = at_[f];
    swap(i, (int)buf_.size() - 1);
    buf_.pop_back();
    at_[f] = -1;
    if (i < (int)buf_.size()) down(i);
  }
  void rebuild() {
    for (int i = (int)buf_.size() / 2; i >= 0; --i) down(i);
  }

 private:
  void swap(int i, int j) {
    std::swap(buf_[i], buf_[j]);
    at_[buf_[i]] = i;
    at_[buf_[j]] = j;
  }
  void down(int i) {
    const int n = (int)buf_.size();
    while (true) {
      int l = 2 * i + 1, r = 2 * i + 2, s = i;
      if (l < n && prio_[buf_[l]] < prio_[buf_[s]]) s = l;
      if (r < n && prio_[buf_[r]] < prio_[buf_[s]]) s = r;
      if (s == i) return;
      swap(i, s);
      i = s;
    }
  }
  void up(int i) {
    while (i > 0) {
      int p = (i - 1) / 2;
      if (!(prio_[buf_[p]] > prio_[buf_[i]])) return;
      swap(p, i);
      i = p;
    }
  }
  std::vector<int> buf_;
  std::vector<float> prio_;
  std::vector<int> at_;
};

// Predictor-scored eviction: lowest score goes first (src/cpp_worker/cache.hpp:81-126,
// src/cpp_worker/cache.cpp:383-399).
class NnPolicy : public Policy {
 public:
  NnPolicy(int n_flat, const CacheEngine* eng) : heap_(n_flat), eng_(eng) {}
  int victim() override { return heap_.top(); }
  std::string evict(int f) override {
    heap_.remove(f);
    return "";
  }
  std::string on_hit(int f, bool) override { return heap_.holds(f) ? "" : "nn: hit on an unknown expert"; }
  std::string on_miss(int f, bool) override {
    if (heap_.holds(f)) return "nn: miss on an expert the policy already holds";
    heap_.push(f, eng_->priority_of(f));
    return "";
  }
  void refresh_all() override {
    for (int f : heap_.items()) heap_.prio(f) = eng_->priority_of(f);
    heap_.rebuild();
  }
  void set_priority(int f, float p) override { heap_.update(f, p); }

 private:
  IndexedMinHeap heap_;
  const CacheEngine* eng_;
};

// Belady's MIN driven by a recorded trace: the expert whose next use lies furthest ahead goes
// first (src/cpp_worker/cache.hpp:148-224, src/cpp_worker/cache.cpp:490-583).
class MinPolicy : public Policy {
 public:
  MinPolicy(int n_flat, const CacheEngine* eng) : heap_(n_flat), eng_(eng) {}
  int victim() override { return heap_.top(); }
  std::string evict(int f) override {
    heap_.remove(f);
    return "";
  }
  std::string on_hit(int f, bool precise) override {
    const std::vector<int64_t>* t = nullptr;
    std::string err = times(f, &t);
    if (!err.empty()) return err;
    size_t& idx = next_idx_[f];
    if (precise) {
      err = advance(*t, &idx);
      if (!err.empty()) return err;
    }
    if (idx >= t->size()) return "min: trace exhausted";
    heap_.update(f, (float)(-(*t)[idx]));
    return "";
  }
  std::string on_miss(int f, bool precise) override {
    const std::vector<int64_t>* t = nullptr;
    std::string err = times(f, &t);
    if (!err.empty()) return err;
    size_t& idx = next_idx_[f];
    if (precise) {
      err = advance(*t, &idx);
      if (!err.empty()) return err;
    }
    if (idx >= t->size()) return "min: trace exhausted";
    if (heap_.holds(f)) return "min: miss on an expert the policy already holds";
    heap_.push(f, (float)(-(*t)[idx]));
    return "";
  }
  std::string set_cur_seq(uint64_t seq) override {
    seq_ = seq;
    have_seq_ = true;
    now_ = -1;
    for (auto& kv : next_idx_) kv.second = 0;
    for (int f : heap_.items()) {
      const std::vector<int64_t>* t = eng_->use_times(seq, f);
      if (t == nullptr || t->empty()) return "min: no trace for a resident expert in this sequence";
      heap_.prio(f) = (float)(-(*t)[0]);
    }
    heap_.rebuild();
    return "";
  }

 private:
  std::string times(int f, const std::vector<int64_t>** out) {
    if (!have_seq_) return "min: set_cur_seq has not been called";
    *out = eng_->use_times(seq_, f);
    if (*out == nullptr) return "min: expert missing from the trace of the current sequence";
    next_idx_.emplace(f, 0);
    return "";
  }
  std::string advance(const std::vector<int64_t>& t, size_t* idx) {
    if (*idx >= t.size()) return "min: trace exhausted";
    if (now_ > t[*idx]) return "min: access earlier than the trace position (trace and run disagree)";
    now_ = t[*idx];
    ++*idx;
    return "";
  }
  IndexedMinHeap heap_;
  const CacheEngine* eng_;
  std::unordered_map<int, size_t> next_idx_;
  uint64_t seq_ = 0;
  bool have_seq_ = false;
  int64_t now_ = -1;
};

// Breadth-first midpoint order of arr[begin, end); a single leftover element at the queue's
// tail ends the walk, otherwise the leftovers restart it (src/cpp_worker/cache.cpp:9-53).
void midpoint_order(const std::vector<int>& arr, std::vector<int>* out) {
  if (arr.empty()) return;
  std::queue<std::pair<int, int>> q;
  q.push({0, (int)arr.size()});
  while (!q.empty()) {
    auto [l, r] = q.front();
    q.pop();
    if (l == r) continue;
    if (r - l == 1) {
      if (q.empty()) {
        out->push_back(arr[l]);
        return;
      }
      std::vector<int> rest(arr.begin() + l, arr.begin() + r);
      while (!q.empty()) {
        auto [l2, r2] = q.front();
        q.pop();
        rest.insert(rest.end(), arr.begin() + l2, arr.begin() + r2);
      }
      midpoint_order(rest, out);
      return;
    }
    int mid = (l + r) / 2;
    out->push_back(arr[mid]);
    if (l < mid) q.push({l, mid});
    if (mid + 1 < r) q.push({mid + 1, r});
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------
CacheEngine::CacheEngine(Config& cfg) : cfg_(cfg) {
  experts_.resize((size_t)cfg_.num_layer * cfg_.num_expert);
  layer_q_.resize(cfg_.num_layer);
}
CacheEngine::~CacheEngine() = default;

int64_t CacheEngine::total_lines() const {
  return (int64_t)std::round((double)(cfg_.cache_rate * (float)cfg_.num_layer * (float)cfg_.num_expert));
}

std::vector<int32_t> CacheEngine::plan_lines(int n_pools, int64_t total) {
  std::vector<int> order;
  if (n_pools > 2) {
    order = {0, 1};
    std::vector<int> rest;
    for (int i = 2; i < n_pools; ++i) rest.push_back(i);
    midpoint_order(rest, &order);
  } else {
    for (int i = 0; i < n_pools; ++i) order.push_back(i);
  }
  std::vector<int32_t> out(n_pools, 0);
  const int64_t base = total / n_pools, rem = total % n_pools;
  for (int i = 0; i < n_pools; ++i) out[order[i]] = (int32_t)(base + (i < rem ? 1 : 0));
  return out;
}

std::string CacheEngine::build() {
  if (built()) return "cache already built";
  const int n_pools = cfg_.per_layer_cache ? cfg_.num_layer : 1;
  std::vector<int32_t> lens = plan_lines(n_pools, total_lines());
  const int n_flat = cfg_.num_layer * cfg_.num_expert;
  if (cfg_.cache_policy == "nn") priority_.assign(n_flat, 0.f);
  pools_.resize(n_pools);
  int32_t base = 0;
  for (int i = 0; i < n_pools; ++i) {
    Pool& p = pools_[i];
    p.base = base;
    p.full_len = lens[i];
    for (int s = 0; s < lens[i]; ++s) p.unused.push_back(s);
    base += lens[i];
    const std::string& name = cfg_.cache_policy;
    if (name == "lru") p.policy.reset(new LruPolicy(n_flat));
    else if (name == "fifo") p.policy.reset(new FifoPolicy());
    else if (name == "static-1") p.policy.reset(new StaticPolicy(1));
    else if (name == "static-2") p.policy.reset(new StaticPolicy(2));
    else if (name == "nn") p.policy.reset(new NnPolicy(n_flat, this));
    else if (name == "min") p.policy.reset(new MinPolicy(n_flat, this));
    else return "unknown cache_policy " + name;
  }
  cfg_.num_predict_expert_per_layer = std::min<int>(cfg_.num_predict_expert_per_layer, pools_[0].full_len);
  return "";
}

int CacheEngine::slot_of(int layer, int e) const {
  int line = experts_[(size_t)layer * cfg_.num_expert + e].line;
  if (line < 0) return -1;
  return line - pools_[pool_index(layer)].base;
}

const std::vector<int64_t>* CacheEngine::use_times(uint64_t seq, int f) const {
  auto s = traces_.find(seq);
  if (s == traces_.end()) return nullptr;
  auto e = s->second.find(f);
  return e == s->second.end() ? nullptr : &e->second;
}

void CacheEngine::record(int kind, int layer, int e, int victim_flat) {
  switch (kind) {
    case kPreciseHit: counters.precise_hit++; break;
    case kPreciseMiss: counters.precise_miss++; break;
    case kPrefetchHit: counters.prefetch_hit++; break;
    default: counters.prefetch_miss++; break;
  }
  if (!log_enabled) return;
  CacheEvent ev;
  ev.kind = kind;
  ev.layer = layer;
  ev.expert = e;
  ev.slot = slot_of(layer, e);
  ev.evicted = victim_flat < 0 ? -1 : victim_flat % cfg_.num_expert;
  ev.evicted_layer = victim_flat < 0 ? -1 : victim_flat / cfg_.num_expert;
  log.push_back(ev);
}

// CacheMngr::hit, src/cpp_worker/cache.cpp:236-246
void CacheEngine::hit(int layer, int e, bool precise) {
  const int f = flat(layer, e);
  Pool& p = pool_for(layer);
  std::string err = p.policy->on_hit(f, precise);
  if (!err.empty() && deferred_error_.empty()) deferred_error_ = err;
  if (precise) {
    max_priority_ += 1.f;
    p.policy->set_priority(f, max_priority_);
    if (!priority_.empty()) priority_[f] = max_priority_;
  }
  record(precise ? kPreciseHit : kPrefetchHit, layer, e, -1);
}

// CacheMngr::miss, src/cpp_worker/cache.cpp:248-312
std::string CacheEngine::miss(int layer, int e, bool precise) {
  const int f = flat(layer, e);
  Pool& p = pool_for(layer);
  if (precise) {
    max_priority_ += 1.f;
    if (!priority_.empty()) priority_[f] = max_priority_;
  }
  int victim = -1;
  if (!p.unused.empty()) {
    experts_[f].line = p.base + p.unused.back();
    p.unused.pop_back();
    std::string err = p.policy->on_miss(f, precise);
    if (!err.empty()) return err;
  } else {
    victim = p.policy->victim();
    if (victim < 0) return "cache pool of layer " + std::to_string(layer) + " has no line to evict (cache_rate too small)";
    if (victim == f) return "policy chose the incoming expert as victim";
    std::string err = p.policy->evict(victim);
    if (!err.empty()) return err;
    err = p.policy->on_miss(f, precise);
    if (!err.empty()) return err;
    ExpertState& v = experts_[victim];
    experts_[f].line = v.line;
    v.line = -1;
    v.num_ready = 0;
    v.status = kIdle;  // a victim still in use is protected on the device by its read event
  }
  record(precise ? kPreciseMiss : kPrefetchMiss, layer, e, victim);
  return "";
}

// FetchScheduleWorker::reorder_experts, src/cpp_worker/prefetcher.cpp:6-42. No copy is ever
// "current" between two requests here, so the classes are: complete, partial, absent.
void CacheEngine::reorder(int layer, int64_t* ids, int64_t n) {
  const int N = cfg_.num_per_expert_param();
  std::vector<int64_t> done, partial, absent;
  for (int64_t i = 0; i < n; ++i) {
    const ExpertState& st = experts_[flat(layer, (int)ids[i])];
    if (st.line < 0) absent.push_back(ids[i]);
    else if (st.num_ready == N) done.push_back(ids[i]);
    else partial.push_back(ids[i]);
  }
  int64_t o = 0;
  for (int64_t v : done) ids[o++] = v;
  for (int64_t v : partial) ids[o++] = v;
  for (int64_t v : absent) ids[o++] = v;
}

// FetchScheduleWorker::preempt_one_layer_without_reorder_, src/cpp_worker/prefetcher.cpp:72-125
void CacheEngine::preempt_layer(int layer, const int64_t* ids, int64_t n, std::vector<Action>* out) {
  const int N = cfg_.num_per_expert_param();
  bool all_before_resident = true;
  for (int64_t i = 0; i < n; ++i) {
    const int e = (int)ids[i];
    ExpertState& st = experts_[flat(layer, e)];
    if (st.line < 0) {
      all_before_resident = false;
      push_task(&precise_q_, layer, e, 0, N, true);
    } else if (!all_before_resident) {
      // resident now, but an earlier miss of this list may evict it before its turn
      push_task(&precise_q_, layer, e, 0, N, true);
    } else if (st.num_ready == N) {
      st.status = kLaunching;
      hit(layer, e, true);
      counters.ready++;
      if (out) out->push_back(Action{Action::kUse, layer, e, st.line, 0, N, 1});
    } else {
      push_task(&precise_q_, layer, e, st.num_ready, N, true);
    }
  }
}

// FetchScheduleWorker::send_one_job + FetchDoneTask, src/cpp_worker/prefetcher.cpp:613-659,556-570
std::string CacheEngine::send(Task t, std::vector<Action>* out) {
  const int N = cfg_.num_per_expert_param();
  ExpertState& st = experts_[flat(t.layer, t.expert)];
  bool copied_before = false;
  if (st.line < 0) {
    if (t.chunk_begin != 0 || st.num_ready != 0)
      return "a partial copy task outlived the eviction of its expert";
    std::string err = miss(t.layer, t.expert, t.precise);
    if (!err.empty()) return err;
    st.status = kFetching;
  } else {
    if (t.precise || t.chunk_begin == 0) hit(t.layer, t.expert, t.precise);
    if (st.num_ready >= t.chunk_end) {  // nothing left to copy
      if (t.precise) {
        if (st.status == kReady) st.status = kLaunching;
        counters.ready++;
        if (out) out->push_back(Action{Action::kUse, t.layer, t.expert, st.line, 0, N, 1});
      }
      return "";
    }
    if (st.num_ready > t.chunk_begin) t.chunk_begin = st.num_ready;
    copied_before = true;
  }
  (void)copied_before;
  if (out) out->push_back(Action{Action::kCopy, t.layer, t.expert, st.line, t.chunk_begin, t.chunk_end, t.precise ? 1 : 0});
  st.num_ready = t.chunk_end;
  if (t.chunk_end == N) {
    st.status = t.precise ? kLaunching : kReady;
    if (t.precise) {
      counters.unready++;
      if (out) out->push_back(Action{Action::kUse, t.layer, t.expert, st.line, 0, N, 1});
    }
  }
  return "";
}

// FetchScheduleWorker::pop_next_task, src/cpp_worker/prefetcher.cpp:143-161: demand tasks first,
// then the prefetch queue of the lowest layer.
std::string CacheEngine::drain(std::vector<Action>* out) {
  while (true) {
    Task t;
    if (!precise_q_.empty()) {
      t = precise_q_.front();
      precise_q_.pop_front();
    } else {
      int l = 0;
      while (l < cfg_.num_layer && layer_q_[l].empty()) ++l;
      if (l == cfg_.num_layer) {
        std::string e = deferred_error_;
        deferred_error_.clear();
        return e;
      }
      t = layer_q_[l].front();
      layer_q_[l].pop_front();
    }
    std::string err = send(t, out);
    if (err.empty() && !deferred_error_.empty()) {
      err = deferred_error_;
      deferred_error_.clear();
    }
    if (!err.empty()) return err;
  }
}

std::string CacheEngine::report_layer(int layer, int64_t* ids, int64_t n, std::vector<Action>* out) {
  if (!built()) return "report_layer before the cache was built";
  if (layer < 0 || layer >= cfg_.num_layer) return "layer out of range";
  for (int64_t i = 0; i < n; ++i)
    if (ids[i] < 0 || ids[i] >= cfg_.num_expert) return "expert id out of range";
  counters.layer_calls++;
  // PreemptTask, src/cpp_worker/prefetcher.cpp:521-537
  if (cfg_.reorder_experts) reorder(layer, ids, n);
  if (cfg_.early_preempt) preempt_layer(layer, ids, n, out);
  layer_q_[layer].clear();
  std::string err = drain(out);
  counters.activated_experts += n;
  record_history(layer, ids, n);
  return err;
}

// LegacyPredictor::add_one_layer / start_of_new_sequence (src/cpp_worker/predictor.cpp:48-80,351-365),
// called as PrefetchMngr::record_then_predict_and_prefetch does (src/cpp_worker/prefetcher.cpp:462-479):
// a report of at most num_expert_per_token ids is a decode step and enters the history; a larger one
// is a prompt pass, and at layer 0 it starts a new sequence.
void CacheEngine::record_history(int layer, const int64_t* ids, int64_t n) {
  const std::string& mode = cfg_.predict_input_mode;
  const bool counts = mode == "one_token" || mode == "decode_cumsum";
  const bool distance = mode == "last_use_distance", weighted = mode == "weighted_decode_cumsum";
  if (!counts && !distance && !weighted) return;
  const size_t LE = (size_t)cfg_.num_layer * cfg_.num_expert;
  if (access_count_.empty()) {
    access_count_.assign(LE, 0.f);
    last_use_distance_.assign(LE, 0.f);
    weighted_access_.assign(LE, 0.f);
  }
  if (n > cfg_.num_expert_per_token) {
    if (layer == 0) {
      if (mode == "decode_cumsum") std::fill(access_count_.begin(), access_count_.end(), 0.f);
      if (distance) std::fill(last_use_distance_.begin(), last_use_distance_.end(), 0.f);
      if (weighted) std::fill(weighted_access_.begin(), weighted_access_.end(), 0.f);
    }
    return;
  }
  const size_t row = (size_t)layer * cfg_.num_expert;
  if (distance)
    for (int e = 0; e < cfg_.num_expert; ++e) last_use_distance_[row + e] += 1.f;
  if (weighted)
    for (int e = 0; e < cfg_.num_expert; ++e) weighted_access_[row + e] /= (float)cfg_.predict_input_decay;
  for (int64_t i = 0; i < n; ++i) {
    if (counts) access_count_[row + ids[i]] += 1.f;
    if (distance) last_use_distance_[row + ids[i]] = 0.f;
    if (weighted) weighted_access_[row + ids[i]] += 1.f;
  }
}

std::vector<float> CacheEngine::history_input() const {
  const size_t LE = (size_t)cfg_.num_layer * cfg_.num_expert;
  std::vector<float> out(LE, 0.f);
  if (access_count_.empty()) return out;
  const std::string& mode = cfg_.predict_input_mode;
  if (mode == "one_token") {
    out = access_count_;
  } else if (mode == "decode_cumsum") {  // each layer's counts divided by their sum, 0 where the sum is 0
    for (int l = 0; l < cfg_.num_layer; ++l) {
      float sum = 0.f;
      for (int e = 0; e < cfg_.num_expert; ++e) sum += access_count_[(size_t)l * cfg_.num_expert + e];
      for (int e = 0; e < cfg_.num_expert; ++e)
        out[(size_t)l * cfg_.num_expert + e] = sum > 0.f ? access_count_[(size_t)l * cfg_.num_expert + e] / sum : 0.f;
    }
  } else if (mode == "last_use_distance") {  // max(dmax - d, 0) / dmax
    const float dmax = (float)cfg_.predict_input_reuse_distance_max;
    for (size_t i = 0; i < LE; ++i) out[i] = std::max(dmax - last_use_distance_[i], 0.f) / dmax;
  } else if (mode == "weighted_decode_cumsum") {
    out = weighted_access_;
  }
  return out;
}

// PrefetchLayerTask, src/cpp_worker/prefetcher.cpp:585-611
std::string CacheEngine::prefetch_layer(int layer, const int64_t* ids, int64_t n, std::vector<Action>* out) {
  if (!built()) return "prefetch_layer before the cache was built";
  if (layer < 0 || layer >= cfg_.num_layer) return "layer out of range";
  if (!layer_q_[layer].empty()) return "prefetch queue of the layer is not empty";
  const int N = cfg_.num_per_expert_param();
  for (int64_t i = 0; i < n; ++i) {
    if (ids[i] < 0 || ids[i] >= cfg_.num_expert) return "expert id out of range";
    const int e = (int)ids[i];
    if (cfg_.promote_hit_in_prefetch && in_cache(flat(layer, e))) hit(layer, e, false);
    if (cfg_.chunk_prefetch) {
      for (int c = 0; c < N; ++c) push_task(&layer_q_[layer], layer, e, c, c + 1, false);
    } else {
      push_task(&layer_q_[layer], layer, e, 0, N, false);
    }
  }
  return drain(out);
}

// PrefetchMngr::report_one_expert -> preempt_one_expert, src/cpp_worker/prefetcher.cpp:225-235,44-70
std::string CacheEngine::report_expert(int layer, int e, std::vector<Action>* out) {
  if (!built()) return "report_expert before the cache was built";
  if (layer < 0 || layer >= cfg_.num_layer || e < 0 || e >= cfg_.num_expert) return "expert out of range";
  if (cfg_.early_preempt) return "";  // decided at report_layer already
  const int N = cfg_.num_per_expert_param();
  ExpertState& st = experts_[flat(layer, e)];
  if (st.line < 0) {
    push_task(&precise_q_, layer, e, 0, N, true);
  } else if (st.num_ready == N) {
    st.status = kLaunching;
    hit(layer, e, true);
    counters.ready++;
    if (out) out->push_back(Action{Action::kUse, layer, e, st.line, 0, N, 1});
  } else {
    push_task(&precise_q_, layer, e, st.num_ready, N, true);
  }
  return drain(out);
}

// PrefetchMngr::one_expert_done + ExpertUnlockWorker, src/cpp_worker/prefetcher.cpp:236-267,
// src/cpp_worker/worker.cpp:78-83
std::string CacheEngine::expert_done(int layer, int e) {
  if (layer < 0 || layer >= cfg_.num_layer || e < 0 || e >= cfg_.num_expert) return "expert out of range";
  ExpertState& st = experts_[flat(layer, e)];
  if (st.status == kLaunching || st.status == kUsing) st.status = kReady;
  return "";
}

std::string CacheEngine::layer_done(int layer) {
  if (layer < 0 || layer >= cfg_.num_layer) return "layer out of range";
  if (layer == cfg_.num_layer - 1) iter_marks.push_back(counters);  // one model iteration ends
  return "";
}

std::string CacheEngine::set_cur_seq(uint64_t seq) {
  for (Pool& p : pools_) {
    std::string err = p.policy->set_cur_seq(seq);
    if (!err.empty()) return err;
  }
  return "";
}

std::string CacheEngine::add_use_times(uint64_t seq, int layer, int e, const int64_t* t, int64_t n) {
  if (layer < 0 || layer >= cfg_.num_layer || e < 0 || e >= cfg_.num_expert) return "expert out of range";
  std::vector<int64_t>& v = traces_[seq][flat(layer, e)];
  v.assign(t, t + n);
  // every list ends with "never again" (src/cpp_worker/cache.cpp:637-642)
  if (v.empty() || v.back() != std::numeric_limits<int64_t>::max()) v.push_back(std::numeric_limits<int64_t>::max());
  return "";
}

// CacheMngr::update_priority / update_all_priority / update_some_priority,
// src/cpp_worker/cache.cpp:400-430,584-591
std::string CacheEngine::update_priority(const float* prob, int n_layers, int start_layer) {
  if (cfg_.cache_policy != "nn") return "update_priority needs cache_policy nn";
  if (!built()) return "update_priority before the cache was built";
  if (start_layer < 0 || n_layers < 0 || start_layer + n_layers > cfg_.num_layer) return "layer range out of bounds";
  if (n_layers == cfg_.num_layer && start_layer != 0) return "a full update must start at layer 0";
  const int E = cfg_.num_expert;
  std::copy(prob, prob + (size_t)n_layers * E, priority_.begin() + (size_t)start_layer * E);
  max_priority_ = *std::max_element(priority_.begin(), priority_.end());
  std::vector<char> touched(pools_.size(), 0);
  for (int l = start_layer; l < start_layer + n_layers; ++l) touched[pool_index(l)] = 1;
  if (n_layers == cfg_.num_layer) std::fill(touched.begin(), touched.end(), 1);
  for (size_t i = 0; i < pools_.size(); ++i)
    if (touched[i]) pools_[i].policy->refresh_all();
  return "";
}

}  // namespace pm
