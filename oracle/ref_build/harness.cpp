// Drives the REFERENCE's own cache classes (CacheMngr, the CachePolicy family, ModelLoader,
// ModuleMeta and the FetchScheduleWorker state machine, compiled unmodified from the
// reference tree) through a request stream and prints the cache decisions they make.
// TEST INFRASTRUCTURE ONLY: it produces the golden event logs that pin oracle/srs_policy.py.
//
// The reference runs the scheduler on a busy-polling thread and copies on another. Here no
// thread is launched: each scheduler task is executed directly, and every copy task the
// scheduler hands to the fetch worker is answered at once with a FetchDoneTask, i.e. the
// timing in which the copy engine always keeps up ("sequential schedule").
//
// Input (stdin), one request per line:
//   config <key>=<value> ...            (before "init"; keys of ModuleMeta::init_from_map)
//   init <num_layer> <num_expert> <num_param>
//   layer <l> <n> <id>*n                 PrefetchMngr::report_one_layer + per-expert hooks
//   prefetch <l> <n> <id>*n              PrefetchLayerTask
//   priority <start_layer> <rows> <float>*(rows*E)   CacheMngr::update_priority
//   trace <seq> <l> <e> <n> <time>*n     use times for CachePolicyMIN
//   seq <id>                             CacheMngr::set_cur_seq
// Output (stdout): "plan <lens...>", then per decision
//   "ev <kind> <layer> <expert> <slot> <evicted_expert> <evicted_layer>", and per layer request
//   "order <l> <ids...>" (the list after the in-place reorder). At the end, the per-forward series of
//   the reference's TimeProfiler, "series <name> <v0> <v1> ..." for activated, hit, miss,
//   prefetch_hit and prefetch_miss: the scheduler adds to them as it decides
//   (prefetcher.hpp:71-78) and a new entry starts after the last layer of every iteration, as in
//   PrefetchMngr::one_moe_layer_done (prefetcher.cpp:209-218).
// System and torch headers first, so that the access overrides below touch only the
// reference's own headers (whose members are otherwise private to their threads).
#include <ATen/cuda/CUDAContext.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <dirent.h>
#include <pthread.h>
#include <semaphore.h>
#include <sys/stat.h>
#include <torch/extension.h>
#include <torch/script.h>
#include <torch/torch.h>
#include <unistd.h>

#include <atomic>
#include <bitset>
#include <cassert>
#include <chrono>
#include <condition_variable>
#include <cstddef>
#include <cstdint>
#include <fstream>
#include <functional>
#include <iostream>
#include <map>
#include <memory>
#include <mutex>
#include <queue>
#include <sstream>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#define class struct
#define private public
#define protected public
#include "prefetcher.hpp"
#undef class
#undef private
#undef protected

#include <iostream>
#include <sstream>

void cuda_sleep(uint, int64_t) {}  // the reference defines it in a .cu file that is not built here

namespace {

struct StubLine : ExpertMemHanlderBase {  // a cache line that owns no memory
  void allocate_like(HostExpertMemHanlderBase*, MemMngrCtx*) override { total_allocation_nbytes = 0; }
  void* ptr(int) override { return nullptr; }
};

struct Ev { int kind; ExpertHandler* e; ExpertHandler* victim; };
std::vector<Ev> g_pending;
ExpertHandler* g_last_victim = nullptr;
ExpertHandler* g_victim_of_last_miss = nullptr;

// Decorates the policy the reference created: forwards every call and notes what happened.
struct Spy : CachePolicy {
  std::shared_ptr<CachePolicy> in;
  explicit Spy(std::shared_ptr<CachePolicy> p) : CachePolicy(nullptr), in(p) {}
  ExpertHandler* select_for_evict(ExpertHandler* e) override { return in->select_for_evict(e); }
  void evict(ExpertHandler* e) override { g_last_victim = e; in->evict(e); }
  void access_on_hit(ExpertHandler* e) override { in->access_on_hit(e); }
  void access_on_hit(ExpertHandler* e, bool precise) override {
    in->access_on_hit(e, precise);
    g_pending.push_back({precise ? 0 : 2, e, nullptr});
  }
  void access_on_miss(ExpertHandler* e) override { in->access_on_miss(e); }
  void access_on_miss(ExpertHandler* e, bool precise) override {
    in->access_on_miss(e, precise);
    g_pending.push_back({precise ? 1 : 3, e, g_last_victim});
    g_victim_of_last_miss = g_last_victim;
    g_last_victim = nullptr;
  }
  void update_all_priority() override { in->update_all_priority(); }
  void update_priority(ExpertHandler* e, float p) override { in->update_priority(e, p); }
  void set_cur_seq(uint64_t s) override { in->set_cur_seq(s); }
  std::string toString() override { return in->toString(); }
};

struct Rig {
  std::shared_ptr<ModuleMeta> metas;
  std::shared_ptr<ModelLoader> loader;
  std::shared_ptr<CacheMngr> cache;
  std::shared_ptr<PredictWorker> predict;
  std::shared_ptr<FetchWorker> fetch;
  std::shared_ptr<FetchScheduleWorker> sched;
  std::shared_ptr<CacheStatistics> stats;
  std::shared_ptr<TimeProfiler> profiler;
  std::unordered_map<ExpertMemHanlderBase*, int> slot_of_line;
  std::vector<torch::Tensor> keep;
  // The fetch worker waits for a victim that the model is still using before it overwrites the
  // line (CacheMngr::miss returns that wait, FetchWorker runs it). With no second thread the
  // wait is parked here and completed when the per-expert loop releases the victim.
  std::vector<std::pair<ExpertHandler*, std::function<void()>>> parked_waits;

  void release_expert(ExpertHandler* e) {
    e->expert_status.transfer(kLaunching, kUsing);  // PrefetchMngr::mark_expert_using
    e->expert_status.transfer(kUsing, kReady);      // ExpertUnlockWorker
    for (size_t i = 0; i < parked_waits.size();) {
      if (parked_waits[i].first == e) {
        parked_waits[i].second();
        parked_waits.erase(parked_waits.begin() + i);
      } else {
        ++i;
      }
    }
  }

  void flush_events() {
    for (auto& ev : g_pending) {
      int slot = slot_of_line.at(ev.e->gpu_data);
      std::cout << "ev " << ev.kind << ' ' << ev.e->layer_idx << ' ' << ev.e->expert_idx << ' ' << slot << ' '
                << (ev.victim ? ev.victim->expert_idx : -1) << ' ' << (ev.victim ? ev.victim->layer_idx : -1) << '\n';
    }
    g_pending.clear();
  }

  // Runs the idle task until it finds nothing to send; answers each sent copy with FetchDone.
  void drain() {
    while (true) {
      sched->current_task.expert = nullptr;
      bool found = false, sent = false;
      sched->pop_next_task(sched->current_task, found);
      if (!found) break;
      g_victim_of_last_miss = nullptr;
      sent = sched->send_one_job(&sched->current_task);
      flush_events();
      if (sent) {
        ExpertHandler* v = g_victim_of_last_miss;
        auto wait_for_victim = sched->current_task.lambda_wait;
        if (v != nullptr && (v->expert_status.get() == kLaunching || v->expert_status.get() == kUsing)) {
          parked_waits.push_back({v, wait_for_victim});
        } else {
          wait_for_victim();
        }
        FetchDoneTask done;
        sched->do_one_task_impl(&done);
      }
    }
    sched->current_task.expert = nullptr;
  }
};

}  // namespace

int main() {
  std::unordered_map<std::string, std::string> cfg;
  Rig r;
  std::string line;
  while (std::getline(std::cin, line)) {
    std::istringstream in(line);
    std::string cmd;
    if (!(in >> cmd)) continue;
    if (cmd == "config") {
      std::string kv;
      while (in >> kv) cfg[kv.substr(0, kv.find('='))] = kv.substr(kv.find('=') + 1);
    } else if (cmd == "init") {
      int L, E, N;
      in >> L >> E >> N;
      r.metas = std::make_shared<ModuleMeta>(L, E);
      std::vector<std::string> names;
      for (int i = 0; i < N; ++i) names.push_back("p" + std::to_string(i));
      r.metas->init_param_list(names);
      r.metas->init_from_map(cfg);
      r.metas->handle_uninited_configs();
      r.metas->physical_mem_impl = "oracle_stub";
      ExpertMemParamFactory::get().physical_registry["oracle_stub"] = []() { return new StubLine(); };
      r.loader = std::make_shared<ModelLoader>(r.metas);
      for (int l = 0; l < L; ++l)
        for (int e = 0; e < E; ++e)
          for (int p = 0; p < N; ++p) {
            r.keep.push_back(torch::zeros({4}, torch::kFloat32));
            r.loader->add_one_expert_param(r.keep.back(), l, e, p, 0);
          }
      r.cache = std::make_shared<CacheMngr>(r.metas, r.loader);
      for (auto& slot : r.cache->cache_slots->slots) slot.policy = std::make_shared<Spy>(slot.policy);
      uint64_t cache_len = round(r.metas->cache_rate * r.metas->num_layer * r.metas->num_expert);  // prefetcher.cpp:171
      r.cache->init_gpu_mem_buffer(cache_len);
      std::cout << "plan";
      for (auto& slot : r.cache->cache_slots->slots) {
        std::cout << ' ' << slot.full_len;
        for (size_t i = 0; i < slot.unused_mems.size(); ++i) r.slot_of_line[slot.unused_mems[i]] = (int)i;
      }
      std::cout << '\n';
      r.predict = std::make_shared<PredictWorker>();
      r.fetch = std::make_shared<FetchWorker>();
      r.sched = std::make_shared<FetchScheduleWorker>();
      r.stats = std::make_shared<CacheStatistics>();
      r.profiler = std::make_shared<TimeProfiler>();
      r.predict->init(r.sched.get(), nullptr, r.cache.get(), r.metas.get());
      r.fetch->init(r.metas.get(), r.sched.get(), r.loader->mem_mngr_ctx.get(), nullptr);
      r.sched->init(r.metas.get(), r.loader.get(), r.cache.get(), r.fetch.get(), r.predict.get(), r.stats.get(),
                    r.profiler.get());
    } else if (cmd == "layer") {
      int l, n;
      in >> l >> n;
      std::vector<int64_t> ids(n);
      for (auto& v : ids) in >> v;
      r.stats->forward();
      r.profiler->add(TimeProfiler::kCntActivatedExpert, n);  // PrefetchMngr::report_one_layer, prefetcher.cpp:199
      PreemptTask t;
      t.layer_idx = l;
      t.expert_idxs = ids.data();
      t.num_expert = ids.size();
      r.sched->do_one_task_impl(&t);
      r.flush_events();
      r.drain();
      std::cout << "order " << l;
      for (auto v : ids) std::cout << ' ' << v;
      std::cout << '\n';
      for (auto v : ids) {  // ExpertHook.pre_forward / post_forward around each expert
        if (!r.metas->early_preempt) {
          PreemptOneExpertTask pt;
          pt.layer_id = l;
          pt.expert_id = v;
          r.sched->do_one_task_impl(&pt);
          r.flush_events();
          r.drain();
        }
        auto e = r.loader->get_source(l, v);
        CHECK(e->expert_status.get() == kLaunching) << "expert not launchable after its fetch";
        r.release_expert(e);
      }
      if (l == r.metas->num_layer - 1) {  // PrefetchMngr::one_moe_layer_done of the last layer
        for (auto kind : {TimeProfiler::kCntActivatedExpert, TimeProfiler::kHitCnt, TimeProfiler::kMissCnt,
                          TimeProfiler::kReadyCnt, TimeProfiler::kUnreadyCnt, TimeProfiler::kPrefetchHitCnt,
                          TimeProfiler::kPrefetchMissCnt, TimeProfiler::kWaitTime})
          r.profiler->push(kind, 0);
      }
    } else if (cmd == "prefetch") {
      int l, n;
      in >> l >> n;
      std::vector<int64_t> ids(n);
      for (auto& v : ids) in >> v;
      PrefetchLayerTask t;
      t.layer_idx = l;
      t.expert_idxs = ids.data();
      t.num_expert = ids.size();
      r.sched->do_one_task_impl(&t);
      r.flush_events();
      r.drain();
    } else if (cmd == "priority") {
      int start, rows;
      in >> start >> rows;
      auto p = torch::zeros({rows, r.metas->num_expert}, torch::kFloat32);
      float* d = p.data_ptr<float>();
      for (int i = 0; i < rows * r.metas->num_expert; ++i) in >> d[i];
      r.cache->update_priority(p, start);
    } else if (cmd == "trace") {
      uint64_t seq;
      int l, e, n;
      in >> seq >> l >> e >> n;
      auto& o = r.cache->cache_oracle->sequence_oracles[seq].expert_oracles[r.loader->get_source(l, e)];
      o.use_times.resize(n);
      for (auto& v : o.use_times) in >> v;
    } else if (cmd == "seq") {
      uint64_t s;
      in >> s;
      r.cache->set_cur_seq(s);
    } else {
      std::cerr << "unknown request " << cmd << "\n";
      return 2;
    }
  }
  if (r.profiler) {
    const std::pair<const char*, TimeProfiler::TimeType> kinds[] = {
        {"activated", TimeProfiler::kCntActivatedExpert}, {"hit", TimeProfiler::kHitCnt}, {"miss", TimeProfiler::kMissCnt},
        {"prefetch_hit", TimeProfiler::kPrefetchHitCnt}, {"prefetch_miss", TimeProfiler::kPrefetchMissCnt}};
    for (auto& k : kinds) {
      auto t = r.profiler->to_tensor(k.second);  // drops the open entry of the iteration in progress
      std::cout << "series " << k.first;
      for (int64_t i = 0; i < t.numel(); ++i) std::cout << ' ' << t[i].item<int64_t>();
      std::cout << '\n';
    }
  }
  std::cout.flush();
  _exit(0);  // skip the reference's end-of-run reporters, which need a full PrefetchMngr
}
