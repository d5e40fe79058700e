// Device side of a context: pinned expert records on the host, the VMM-backed slab of cache
// lines on the GPU, the side copy stream with its events, and the fused MoE layer forward.
//
// The reference keeps experts in pinned torch tensors (src/cpp_worker/model_loader.cpp:23-31,
// :43-58), carves cache lines out of one cudaMalloc or maps them with the CUDA VMM API
// (src/cpp_worker/model_loader.cpp:102-164,222-233) and copies on a FetchWorker thread that
// drains the copy stream after every task (src/cpp_worker/worker.cpp:84-105). Here a copy is
// one cudaMemcpyAsync of the expert's contiguous record, ordered against the kernels that read
// or last read the line by events, and the host never waits for a copy.
#pragma once
#include <cuda.h>

#include <memory>
#include <vector>

#include "cache_engine.hpp"
#include "pm_common.cuh"

namespace pm {
struct PendingForward;
}

struct pm_ctx {
  pm::Config cfg;
  pm::PendingForward* pending = nullptr;  // the layer call in progress (defined and freed in runtime.cu)
  std::unique_ptr<pm::CacheEngine> eng;
  std::string error;  // scratch for building messages

  // ---- expert registry -------------------------------------------------------------
  struct Param {
    const void* src = nullptr;
    size_t nbytes = 0;
  };
  std::vector<Param> params;            // [(layer * E + expert) * N + param]
  std::vector<size_t> param_offset;     // [N + 1] offsets inside a record; [N] = record size
  std::vector<unsigned char*> host_rec; // [L * E] pinned record of each expert
  std::vector<void*> arena_blocks;      // one pinned block per layer
  // ---- pooled miss fetch (expert-parallel ranks of one node; see pool_fetch.cu) ------------
  std::string shared_prefix;            // non-empty: the arena blocks live in POSIX shared memory "<prefix>_L<layer>"
  struct SharedBlock {
    void* ptr;
    size_t bytes;
    std::string unlink_name;            // set by the creator, who removes the name at destruction
  };
  std::vector<SharedBlock> shared_blocks;
  void* pool_mail = nullptr;            // mailbox through which ranks exchange their miss lists
  std::string pool_mail_name;           // rank 0 removes the name at destruction
  size_t pool_mail_bytes = 0;
  int pool_rank = 0, pool_world = 0;
  size_t pool_slice = 0;                // bytes of one rank's slice of a record (the last may be shorter)
  std::vector<std::vector<void*>> peer_arena;  // [rank][layer] mapped, CUDA-registered arena blocks
  std::vector<int> peer_num_expert;
  int64_t pool_bytes_pulled = 0;        // host-to-device bytes this rank pulled for the pool
  bool pinned = false;
  int role_gate = 0, role_up = 1, role_down = 2;        // which tensor plays which part
  int role_qgate = -1, role_qup = -1, role_qdown = -1;  // uint4 experts: scale/zero tensors

  // ---- slab -------------------------------------------------------------------------
  bool slab_built = false;
  bool slab_vmm = false;
  unsigned char* slab = nullptr;
  size_t line_stride = 0;
  int n_lines = 0;  // lines the policy owns; one more (index n_lines) is the spare line of temp_move_expert_*
  std::vector<CUmemGenericAllocationHandle> line_handles;
  size_t slab_va_bytes = 0;
  // Optional (context option stable_va=1, VMM slab only): every expert also has an address range of
  // its own that never changes; the line that holds the expert is mapped there a second time, so raw
  // pointers a caller captured once stay valid across evictions and refetches (what the reference's
  // ExpertParamWrapperCUDriver gives exllama kernels, src/cpp_worker/model_loader.cpp:102-164).
  bool stable_va = false;
  unsigned char* expert_va = nullptr;   // [L * E] ranges of line_stride bytes
  size_t expert_va_bytes = 0;
  std::vector<int32_t> line_mapped_to;  // flat expert whose range the line is mapped into, -1 = none
  CUmemAllocationProp line_prop{};

  // ---- streams and events -------------------------------------------------------------
  // Demand copies (an activated expert is missing) and prefetch copies (a predicted expert) run on
  // separate streams: a demand copy then starts at once and shares the link with a prefetch in
  // flight instead of queueing behind every prefetch issued before it, which is what the
  // reference's scheduler achieves by popping demand tasks first (src/cpp_worker/prefetcher.cpp:143-161).
  // Back-to-back copies on one stream already run at the link's rate (51.4 GB/s against 52.4 GB/s
  // for bare pinned copies), so this changes latency, not throughput. Two copies into the same
  // line from different streams are ordered through the line's ready event.
  cudaStream_t copy_stream = nullptr;      // demand copies
  cudaStream_t prefetch_stream = nullptr;  // prefetch copies
  std::vector<cudaStream_t> line_copy_stream;  // stream of the last copy into the line
  cudaStream_t last_stream = nullptr;
  bool have_last_stream = false;
  std::vector<cudaEvent_t> line_ready;    // recorded on the copy stream after a copy into the line
  std::vector<cudaStream_t> line_waiter;  // compute stream that already waits for line_ready
  std::vector<char> line_pending;         // a copy was issued that no compute stream waits for yet
  std::vector<cudaEvent_t> line_read;     // event after the last kernel that read the line (or null)
  std::vector<cudaEvent_t> seg_events;    // ring of read events
  size_t seg_next = 0;
  cudaEvent_t sync_event = nullptr;
  cudaStream_t readback_stream = nullptr;  // carries the router's counts to the host beside the FFN
  cudaEvent_t routed_event = nullptr;      // router + permute done on the compute stream
  bool device_plan = true;                 // plan and launch the resident experts without a host round trip
  int32_t* d_res_counters = nullptr;       // dependency counters of that launch (cleared by the permutation)

  // ---- per-layer model weights ----------------------------------------------------------
  struct Layer {
    pm_layer_weights w{};
    bool set = false;
    int32_t* slot_table_dev = nullptr;  // [E] slot of each expert, -1 if absent
    bool slot_table_dirty = true;
  };
  std::vector<Layer> layers;
  struct Predictor {
    const void* w1 = nullptr;
    const float* b1 = nullptr;
    int d = 0;
    const void* w2 = nullptr;
    const float* b2 = nullptr;
  };
  std::vector<Predictor> predictors;  // [(L + 1) * L], index src * L + dst

  // ---- forward workspace ------------------------------------------------------------------
  int ws_tokens = 0;  // capacity in tokens
  int ws_hidden = 0, ws_inter = 0, ws_topk = 0, ws_inter_routed = 0, ws_inter_shared = 0;
  unsigned char* ws_dev = nullptr;
  size_t ws_bytes = 0;
  int32_t *d_topk_ids = nullptr, *d_topk_slot = nullptr, *d_counts = nullptr, *d_offsets = nullptr;
  int32_t *d_row_token = nullptr, *d_pos = nullptr, *d_err = nullptr;
  float *d_topk_w = nullptr, *d_shared_scale = nullptr, *d_yexp = nullptr, *d_scores = nullptr;
  float* d_pred_hidden = nullptr;
  __nv_bfloat16 *d_hbuf = nullptr, *d_xin = nullptr, *d_yout = nullptr;
  unsigned char* d_plan = nullptr;  // launch plans of one layer call (descriptors + tile tables)
  size_t plan_cap = 0;              // bytes
  float* h_routed_scores = nullptr;  // pinned: predictor scores handed to the routed-rows form
  size_t h_routed_scores_cap = 0;
  unsigned char* h_stage = nullptr;  // pinned: counts+offsets, scores, descriptors, slot tables, routing
  size_t h_stage_bytes = 0;

  // ---- prefill (tcgen05) path ---------------------------------------------------------------------
  bool tc_prefill = true;             // use it for experts with more than 64 rows in a call
  __nv_bfloat16* d_xperm = nullptr;   // expert-sorted copy of the token rows [rows, hidden]
  unsigned char* d_tc_plan = nullptr; // groups + tiles of the segments of one layer call
  unsigned char* h_tc_plan = nullptr; // pinned staging of the same
  size_t tc_plan_cap = 0, tc_plan_used = 0;
  int32_t* d_perm_scratch = nullptr;  // per-chunk expert counts of the multi-CTA permutation
  size_t perm_scratch_ints = 0;
  int32_t* d_tc_err = nullptr;        // set by an FFN kernel when a bounded wait gave up; sits behind the
                                      // permutation's counts and reaches the host with them at the next layer call
  bool xperm_ready = false, tc_maps_ready = false;  // per layer call
  pm::TcMaps tc_maps;
  int64_t tc_launches = 0;
  // device-side ranking of the predictor scores: [2 * num_layer][kTopCap] ids (own predictions by
  // target layer, then the caller-supplied score rows of the routed-rows form)
  bool device_topn = true;
  int32_t* d_topn = nullptr;
  int32_t* h_topn = nullptr;
  int64_t topn_launches = 0;
  // uint4 experts on the prefill path: the packed weights of a segment's experts are expanded into
  // this bf16 slab (one line per expert of the segment) and the tensor-core kernels read it
  unsigned char* q4_scratch = nullptr;
  size_t q4_scratch_lines = 0, q4_scratch_stride = 0;
  pm::TcMaps tc_maps_q4;
  bool tc_maps_q4_ready = false;  // per layer call
  int64_t q4_expanded = 0;        // experts expanded so far

  bool keep_routing = false;
  int seq_len = 1;
  std::vector<std::vector<int32_t>> last_ids;  // per layer routing copies (keep_routing)
  std::vector<std::vector<float>> last_w;

  int64_t h2d_bytes = 0, h2d_copies = 0, kernel_launches = 0;

  // ---- optional timing of the grouped FFN launches (for the roofline figure) ------------------
  struct FfnSample {
    cudaEvent_t e0, e1, e2;  // before gate/up, between (null for a fused launch), after down
    int64_t bytes_gu, bytes_dn;
    bool fused;
    bool resident;  // the device-planned launch (shared expert + experts already resident)
  };
  bool profile_ffn = false;
  std::vector<FfnSample> ffn_samples;      // recorded, not yet read
  std::vector<cudaEvent_t> ffn_event_pool; // free events
  double ffn_ms_gu = 0, ffn_ms_dn = 0, ffn_ms_fused = 0;
  int64_t ffn_bytes_gu = 0, ffn_bytes_dn = 0, ffn_launches = 0, ffn_bytes_fused = 0, ffn_fused_launches = 0;
  double ffn_ms_resident = 0;  // part of the fused totals that belongs to device-planned launches
  int64_t ffn_bytes_resident = 0, ffn_resident_launches = 0;

  ~pm_ctx();
};

namespace pm {

int rt_pin_all(pm_ctx* c);
int rt_build_slab(pm_ctx* c);
int rt_execute_copies(pm_ctx* c, const std::vector<Action>& actions);
// routed: the caller supplies one local expert id per row (row_expert, device int32 [T]); there is
// no router, no shared expert and no weighted combine, and rows_out (device f32 [T, hidden])
// receives every row's expert output in row order. Used by the expert-parallel receive side.
// row_expert -1 marks a padding row (no expert runs on it, its output row is zeros).
// max_rows_per_expert (0 = unknown): an upper bound on the rows any one expert receives that the
// caller guarantees (e.g. the global number of tokens); with a bound of at most 16 the resident
// experts are launched without waiting for the host. pred_scores (optional): device f32
// [n_pred, pred_width], predictor scores of layers pred_layers[i] over the experts of the whole
// model (this context holds [pred_first, pred_first + num_expert) of them); they travel to the
// host with the row counts, the pred_top best of the whole list are taken and those this context
// holds are prefetched, before this layer's own report.
struct RoutedRows {
  const int32_t* row_expert = nullptr;
  float* rows_out = nullptr;
  int max_rows_per_expert = 0;
  const float* pred_scores = nullptr;
  const int32_t* pred_layers = nullptr;  // host
  int n_pred = 0, pred_width = 0, pred_first = 0, pred_top = 0;
  // Leave the copies of missing activated experts to the caller: the call returns after the cache
  // decisions and the launches that need no such copy; rt_pending_pooled lists the copies, and
  // rt_forward_end finishes the call once the lines' ready events have been recorded.
  bool collect_demand_copies = false;
};
int rt_forward_end(pm_ctx* c);
const std::vector<Action>& rt_pending_pooled(pm_ctx* c);
constexpr int kPoolMaxMiss = 64;  // most demand copies one rank can put into one exchange
void* rt_shared_block(pm_ctx* c, const std::string& name, size_t bytes, bool create, std::string* err);
void rt_release_shared_blocks(pm_ctx* c);
int rt_pool_init(pm_ctx* c, int rank, int world, const char* mailbox_name);
int rt_pool_open_peer(pm_ctx* c, int peer, const char* prefix, int peer_num_expert);
int rt_pool_exchange(pm_ctx* c, int64_t seq, const int32_t* experts, int n, int32_t* out, double timeout_s);
int rt_pool_stage(pm_ctx* c, int layer, const int32_t* lists, void* send_dev, size_t send_cap, size_t recv_cap,
                  int64_t* send_split, int64_t* recv_split, cudaStream_t s);
int rt_pool_scatter(pm_ctx* c, const void* recv_dev, cudaStream_t s);
int rt_pool_fetch_locally(pm_ctx* c);
int rt_forward(pm_ctx* c, int layer, const void* x, int T, void* y, cudaStream_t s, const RoutedRows* routed = nullptr);
int rt_forward_host(pm_ctx* c, int layer, const void* x, int T, void* y, cudaStream_t s);
int rt_report_hidden(pm_ctx* c, int index, const void* hidden, int B, int seq, cudaStream_t s);
int rt_expert_acquire(pm_ctx* c, int layer, int expert, cudaStream_t s, void** line);
int rt_expert_release(pm_ctx* c, int layer, int expert, cudaStream_t s);
int rt_temp_move(pm_ctx* c, int layer, int expert, bool to_gpu, cudaStream_t s, void** line);
void rt_mark_dirty(pm_ctx* c, const std::vector<Action>& actions);
int rt_profile_collect(pm_ctx* c);
bool tc_prefill_usable(const pm_ctx* c, const pm_layer_weights& w);
bool tc_prefill_usable_q4(const pm_ctx* c, const pm_layer_weights& w);
int tc_build_maps(pm_ctx* c, const pm_layer_weights& w, int rows_cap, TcMaps* m);
// Same with the routed experts' bf16 weights in `slab` (gate, up, down back to back in every line).
int tc_build_maps_q4(pm_ctx* c, const pm_layer_weights& w, int rows_cap, TcMaps* m);
void tc_plan(const std::vector<TcGroup>& groups, int hidden, std::vector<TcTile>* gu, std::vector<TcTile>* dn);

}  // namespace pm
