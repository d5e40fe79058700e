// Host-side expert cache: slot pools, eviction policies and the fetch schedule.
//
// The reference spreads this over CacheMngr (src/cpp_worker/cache.cpp:57-312), the policy
// classes (src/cpp_worker/cache.hpp:24-224) and the FetchScheduleWorker state machine
// (src/cpp_worker/prefetcher.cpp:6-161,494-659), driven by four busy-polling threads. Here it
// is one single-threaded engine that makes every decision at the moment the request is
// issued ("sequential schedule"): a copy counts as complete for bookkeeping as soon as it
// has been handed to the copy stream, and ordering between copies and kernels is enforced on
// the device with events instead of host spin-waits. Decisions (hit, miss, victim, slot) are
// therefore independent of timing and match the reference whenever its own threads are not
// racing (always when prediction is off).
#pragma once
#include <cstdint>
#include <deque>
#include <limits>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "config.hpp"

namespace pm {

enum EventKind : int32_t { kPreciseHit = 0, kPreciseMiss = 1, kPrefetchHit = 2, kPrefetchMiss = 3 };

struct CacheEvent {
  int32_t kind, layer, expert, slot, evicted, evicted_layer;
};

// What the device executor has to do, in schedule order.
struct Action {
  enum Type : int32_t { kUse = 0, kCopy = 1 } type;
  int32_t layer, expert;
  int32_t line;         // global cache-line index (pool base + slot)
  int32_t chunk_begin;  // kCopy: tensors [chunk_begin, chunk_end) of the expert
  int32_t chunk_end;
  int32_t precise;
};

enum ExpertStatus : int32_t { kIdle = 0, kFetching, kReady, kLaunching, kUsing };

struct ExpertState {
  int32_t line = -1;      // global line index, -1 = not in the cache
  int32_t num_ready = 0;  // tensors already copied
  int32_t status = kIdle;
};

struct Counters {
  int64_t precise_hit = 0, precise_miss = 0, prefetch_hit = 0, prefetch_miss = 0;
  int64_t ready = 0, unready = 0, activated_experts = 0, layer_calls = 0;
};

class Policy;

struct Pool {
  int32_t base = 0;       // global index of this pool's first line
  int32_t full_len = 0;
  std::vector<int32_t> unused;  // free slots; taken from the back
  std::unique_ptr<Policy> policy;
};

class CacheEngine {
 public:
  explicit CacheEngine(Config& cfg);  // keeps a reference: the context owns the configuration
  ~CacheEngine();

  // Lines per pool for `total` lines: floor share plus one for the first `total % n` pools in
  // the priority order 0, 1, then breadth-first midpoints of 2..n-1 (src/cpp_worker/cache.cpp:9-83).
  static std::vector<int32_t> plan_lines(int n_pools, int64_t total);
  int64_t total_lines() const;  // round(cache_rate * L * E), src/cpp_worker/prefetcher.cpp:162-177

  // Creates the pools. Also clamps num_predict to pool 0's length (src/cpp_worker/cache.cpp:130-131).
  std::string build();
  bool built() const { return !pools_.empty(); }

  std::string report_layer(int layer, int64_t* ids, int64_t n, std::vector<Action>* out);
  std::string prefetch_layer(int layer, const int64_t* ids, int64_t n, std::vector<Action>* out);
  std::string report_expert(int layer, int expert, std::vector<Action>* out);
  std::string expert_done(int layer, int expert);
  std::string layer_done(int layer);
  std::string set_cur_seq(uint64_t seq);
  std::string add_use_times(uint64_t seq, int layer, int expert, const int64_t* t, int64_t n);
  std::string update_priority(const float* prob, int n_layers, int start_layer);

  const ExpertState& expert(int layer, int e) const { return experts_[(size_t)layer * cfg_.num_expert + e]; }
  int pool_index(int layer) const { return cfg_.per_layer_cache ? layer : 0; }
  const std::vector<Pool>& pools() const { return pools_; }
  int slot_of(int layer, int e) const;  // slot inside its pool, -1 if absent

  Config& config() { return cfg_; }
  const Config& config() const { return cfg_; }
  Counters counters;
  // Snapshot of `counters` at the end of every model iteration (layer_done of the last layer): the
  // per-forward series of the reference's TimeProfiler (src/cpp_worker/profiler.hpp:262-275,
  // pushed in PrefetchMngr::one_moe_layer_done, src/cpp_worker/prefetcher.cpp:209-218) are the
  // differences of consecutive snapshots.
  std::vector<Counters> iter_marks;
  bool log_enabled = false;
  std::vector<CacheEvent> log;

  // The history-based predictor inputs of the reference's LegacyPredictor
  // (src/cpp_worker/predictor.cpp:48-80,351-365), fed by every decode-size report_layer
  // (PrefetchMngr::record_then_predict_and_prefetch, src/cpp_worker/prefetcher.cpp:462-479):
  // access counts, layer steps since the last use, and access counts decayed by predict_input_decay.
  // history_input() gives the tensor the predictor model receives for the configured
  // predict_input_mode (src/cpp_worker/predictor.cpp:143-175), [num_layer * num_expert].
  std::vector<float> history_input() const;

  // use-time lookup for the Belady policy
  const std::vector<int64_t>* use_times(uint64_t seq, int flat) const;
  float priority_of(int flat) const { return priority_.empty() ? 0.f : priority_[flat]; }

 private:
  struct Task {
    int32_t layer, expert, chunk_begin, chunk_end;
    bool precise;
  };
  int flat(int layer, int e) const { return layer * cfg_.num_expert + e; }
  Pool& pool_for(int layer) { return pools_[pool_index(layer)]; }
  bool in_cache(int f) const { return experts_[f].line >= 0; }
  void hit(int layer, int e, bool precise);
  std::string miss(int layer, int e, bool precise);
  void reorder(int layer, int64_t* ids, int64_t n);
  void preempt_layer(int layer, const int64_t* ids, int64_t n, std::vector<Action>* out);
  void push_task(std::deque<Task>* q, int layer, int e, int b, int en, bool precise) {
    q->push_back(Task{layer, e, b, en, precise});
  }
  std::string send(Task t, std::vector<Action>* out);
  std::string drain(std::vector<Action>* out);
  void record(int kind, int layer, int e, int victim_flat);

  Config& cfg_;
  std::vector<Pool> pools_;
  std::vector<ExpertState> experts_;
  void record_history(int layer, const int64_t* ids, int64_t n);
  std::vector<float> access_count_, last_use_distance_, weighted_access_;  // [L * E] each
  std::vector<float> priority_;  // "nn" policy only: [L * E]
  float max_priority_ = std::numeric_limits<float>::min();
  std::string deferred_error_;  // first policy error raised inside hit()
  std::deque<Task> precise_q_;
  std::vector<std::deque<Task>> layer_q_;
  std::unordered_map<uint64_t, std::unordered_map<int, std::vector<int64_t>>> traces_;
};

}  // namespace pm
