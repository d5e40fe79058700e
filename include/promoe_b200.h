/*
 * promoe_b200 -- C ABI of the B200-native MoE hot path (expert cache + fused MoE layer).
 *
 * Every function returns 0 on success or a PM_ERR_* code; none aborts the process.
 * pm_last_error() gives the message of the last failure on the calling thread.
 * Device pointers are plain CUDA device addresses; `stream` is a cudaStream_t
 * passed as void* (NULL = the legacy default stream). A context must be used by
 * one thread at a time.
 *
 * The citations name the reference (huwf5/promoe) interface each entry point
 * stands in for, by the file's path inside that project.
 */
#ifndef PROMOE_B200_H_
#define PROMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PM_OK 0
#define PM_ERR_INVALID 1   /* bad argument or configuration */
#define PM_ERR_CUDA 2      /* a CUDA runtime / driver call failed */
#define PM_ERR_STATE 3     /* call made in the wrong phase (e.g. forward before build_slab) */
#define PM_ERR_UNSUPPORTED 4
#define PM_ERR_TIMEOUT 5   /* a bounded host wait ran out */

typedef struct pm_ctx pm_ctx;

/* ---- library ---------------------------------------------------------- */
int pm_version(void);
/* Message of the last error on this thread ("" if none). */
const char* pm_last_error(void);

/* ---- configuration (ModuleMeta: src/cpp_worker/utils.hpp:127-192,
 *      init_from_map / handle_uninited_configs: src/cpp_worker/utils.cpp:54-273) ---- */

/* Creates a context for num_layer MoE layers of num_expert routed experts.
 * config_kv holds "key=value" lines with the reference's config keys (cache_rate,
 * cache_policy, num_expert_per_token, num_predict_expert_per_layer, reorder_experts,
 * early_preempt, chunk_prefetch, per_layer_cache, promote_hit_in_prefetch,
 * layer_predict_interval, layer_predict_max_window, limit_layer_0_window,
 * limit_layer_0_num_predict, model_arch_string, ... and their dialect aliases).
 * Values "None" or "" select the default. Unknown keys are an error (the reference aborts). */
int pm_ctx_create(pm_ctx** out, int num_layer, int num_expert, const char* config_kv);
int pm_ctx_destroy(pm_ctx* ctx);
/* Reads one resolved configuration value as text into buf (NUL-terminated). */
int pm_ctx_get(pm_ctx* ctx, const char* key, char* buf, size_t cap);
/* Overrides one configuration value after creation (same keys as pm_ctx_get). */
int pm_ctx_set(pm_ctx* ctx, const char* key, const char* value);
/* Names of the per-expert tensors, in chunk order (ModuleMeta::init_param_list,
 * src/cpp_worker/utils.cpp:47-53). names = '\n'-separated. */
int pm_ctx_set_param_list(pm_ctx* ctx, const char* names);

/* ---- expert registry and slab (ModelLoader: src/cpp_worker/model_loader.hpp:276-319,
 *      src/cpp_worker/model_loader.cpp:8-31; CacheMngr::init_gpu_mem_buffer:
 *      src/cpp_worker/cache.cpp:57-132; PrefetchMngr::init_gpu_mem_buffer:
 *      src/cpp_worker/prefetcher.cpp:162-177) ---- */

/* Registers the host copy of one tensor of one expert. The bytes stay owned by the caller
 * until pm_pin_all, which copies them into the library's pinned arena (one contiguous
 * record per expert, so a miss is a single DMA). */
int pm_register_expert_param(pm_ctx* ctx, int layer, int expert, int param_id, const void* host_ptr,
                             size_t nbytes);
int pm_pin_all(pm_ctx* ctx);
/* Address of one tensor inside the pinned record of an expert (valid after pm_pin_all), for
 * callers that registered the tensor with host_ptr == NULL and fill the record in place. */
int pm_expert_host_ptr(pm_ctx* ctx, int layer, int expert, int param_id, void** out, size_t* nbytes);
/* Number of cache lines each layer gets (length num_layer, or 1 when per_layer_cache is off). */
int pm_plan_slots(pm_ctx* ctx, int32_t* per_pool_len, int cap, int* n_pools);
/* Reserves the VMM range and maps one physical allocation per cache line. */
int pm_build_slab(pm_ctx* ctx);
/* Builds the slot pools without any device memory (policy-only use, no GPU needed). */
int pm_build_policy_only(pm_ctx* ctx);
/* Device address the tensor currently has in the slab, NULL if the expert is not resident
 * (ModelLoader::ref_one_expert_param, src/cpp_worker/model_loader.hpp:309-314). With the context
 * option stable_va=1 (set before pm_build_slab; VMM slab only) every expert has an address range of
 * its own into which the line that holds it is mapped a second time: the address returned here is
 * then the same for the life of the context, and readable whenever the expert is resident (the
 * reference's ExpertParamWrapperCUDriver, src/cpp_worker/model_loader.cpp:102-164, for kernels that
 * capture raw pointers once). In that mode a line that changes hands is remapped on the host,
 * which waits for the last kernel that read it. */
int pm_param_device_ptr(pm_ctx* ctx, int layer, int expert, int param_id, void** out);
/* Slot (index inside the layer's pool, creation order) of an expert, -1 if absent. */
int pm_expert_slot(pm_ctx* ctx, int layer, int expert, int32_t* slot);

/* ---- cache policy and fetch schedule (PrefetchMngr / FetchScheduleWorker:
 *      src/cpp_worker/prefetcher.cpp:6-161,188-267,494-659; CacheMngr::hit/miss:
 *      src/cpp_worker/cache.cpp:236-312; policies: src/cpp_worker/cache.hpp:24-224) ---- */

/* Reports the unique experts one layer call activates. ids is reordered in place when
 * reorder_experts is on (PrefetchMngr::report_one_layer). Runs the hit/miss/evict
 * decisions of the sequential schedule and, when a slab exists, enqueues the copies. */
int pm_report_layer(pm_ctx* ctx, int layer, int64_t* ids, int64_t n);
/* Queues a prefetch of `ids` (rank order) for `layer` and drains it
 * (FetchScheduleWorker PrefetchLayerTask, src/cpp_worker/prefetcher.cpp:585-611). */
int pm_prefetch_layer(pm_ctx* ctx, int layer, const int64_t* ids, int64_t n);
/* PrefetchMngr::report_one_expert / one_expert_done / one_moe_layer_done
 * (src/cpp_worker/prefetcher.cpp:203-267). */
int pm_report_expert(pm_ctx* ctx, int layer, int expert);
int pm_expert_done(pm_ctx* ctx, int layer, int expert);
int pm_layer_done(pm_ctx* ctx, int layer);
/* The same two calls for a caller that computes the expert itself on `stream` (the reference's
 * per-expert module loop under ExpertHook, src/sparse_llm_cache/utils/hooks.py:187-198):
 * pm_expert_acquire = report_one_expert + wait_expert (src/cpp_worker/prefetcher.cpp:225-258): after
 * the bookkeeping it makes `stream` wait for the copy into the expert's cache line (the host does
 * not wait) and returns the line's device address; tensor i of the expert sits at
 * *line + pm_param_offset(i), which is what the reference's logical parameter is re-pointed to on
 * a fetch (src/cpp_worker/worker.cpp:91-97, src/cpp_worker/model_loader.hpp:290-313).
 * pm_expert_release = one_expert_done (src/cpp_worker/prefetcher.cpp:259-267): it records on
 * `stream` the point after which a later copy may overwrite the line. */
int pm_expert_acquire(pm_ctx* ctx, int layer, int expert, void* stream, void** line);
int pm_expert_release(pm_ctx* ctx, int layer, int expert, void* stream);
/* Byte offset of tensor param_id inside every cache line and pinned record (256-byte aligned). */
int pm_param_offset(pm_ctx* ctx, int param_id, size_t* offset);
/* PrefetchMngr::temp_move_expert_to_gpu / temp_move_expert_back_to_host
 * (src/cpp_worker/prefetcher.cpp:664-697): copies the expert's host record into a spare cache line
 * that no policy owns and returns its address (a quantised layer's post_init can then transform
 * the tensors on the device), or copies the spare line back into the host record. Both wait for
 * their copy on `stream`. */
int pm_temp_move_expert_to_gpu(pm_ctx* ctx, int layer, int expert, void* stream, void** line);
int pm_temp_move_expert_back_to_host(pm_ctx* ctx, int layer, int expert, void* stream);
/* CacheMngr::set_cur_seq (src/cpp_worker/cache.hpp:310-314), Belady policy only. */
int pm_set_cur_seq(pm_ctx* ctx, uint64_t seq_id);
/* Loads the Belady (MIN) trace: per (seq, layer, expert) ascending use times
 * (CacheOracle::load_from_tensor, src/cpp_worker/cache.cpp:592-644). */
int pm_oracle_add_use_times(pm_ctx* ctx, uint64_t seq_id, int layer, int expert, const int64_t* times,
                            int64_t n);
/* CacheMngr::update_priority (src/cpp_worker/cache.cpp:400-430,584-591): prob is
 * [n_layers, num_expert] float32 for layers start_layer.. */
int pm_update_priority(pm_ctx* ctx, const float* prob, int n_layers, int start_layer);
/* The input the reference's LegacyPredictor hands its model for the history-based
 * predict_input_mode values one_token, decode_cumsum, last_use_distance and
 * weighted_decode_cumsum (src/cpp_worker/predictor.cpp:48-80,143-175,351-365): out receives
 * [num_layer, num_expert] float32. The history is kept by pm_report_layer (decode-size reports
 * enter it, a prompt-size report at layer 0 starts a new sequence,
 * src/cpp_worker/prefetcher.cpp:462-479); other modes read as zeros. */
int pm_history_input(pm_ctx* ctx, float* out, size_t cap);

/* One cache decision, in the order the schedule performed it. */
typedef struct pm_event {
  int32_t kind;    /* 0 precise hit, 1 precise miss, 2 prefetch hit, 3 prefetch miss */
  int32_t layer;
  int32_t expert;
  int32_t slot;    /* index of the cache line inside its pool, creation order */
  int32_t evicted; /* expert that lost the line (same pool), -1 if the line was free */
  int32_t evicted_layer;
} pm_event;
int pm_event_log_enable(pm_ctx* ctx, int on);
int pm_event_log_read(pm_ctx* ctx, pm_event* out, size_t cap, size_t* n);
int pm_event_log_clear(pm_ctx* ctx);

/* Counters (TimeProfiler series, src/cpp_worker/profiler.hpp:262-275), totals since creation. */
typedef struct pm_stats {
  int64_t precise_hit, precise_miss, prefetch_hit, prefetch_miss;
  int64_t ready, unready;
  int64_t activated_experts, layer_calls;
  int64_t h2d_bytes, h2d_copies;
  int64_t kernel_launches;
} pm_stats;
int pm_stats_read(pm_ctx* ctx, pm_stats* out);
/* The counters as they stood at the end of every model iteration (pm_layer_done of the last
 * layer), oldest first: differences of consecutive entries are the per-forward series the
 * reference's TimeProfiler keeps (src/cpp_worker/profiler.hpp:262-319, pushed in
 * PrefetchMngr::one_moe_layer_done, src/cpp_worker/prefetcher.cpp:209-218) and its end-of-run
 * report averages (src/cpp_worker/prefetcher.cpp:327-402). The copy and launch fields are 0. */
int pm_iter_marks_read(pm_ctx* ctx, pm_stats* out, size_t cap, size_t* n);

/* Device time and weight bytes of the grouped FFN launches made while the context option
 * profile_ffn=1 was set (CUDA events on the caller's stream around each launch). */
typedef struct pm_profile {
  int64_t ffn_launches;  /* gate/up + down launch pairs (tensor-core tiles, staged kernel) */
  double gateup_ms, down_ms;
  int64_t gateup_bytes, down_bytes; /* weight bytes those launches had to read once */
  int64_t fused_launches; /* single cooperative launches (gate/up and down tiles, per-chunk counters) */
  double fused_ms;
  int64_t fused_bytes;
  int64_t resident_launches; /* the part of the fused figures that belongs to device-planned launches */
  double resident_ms;        /* (shared expert + experts already resident, enqueued behind the router) */
  int64_t resident_bytes;
} pm_profile;
int pm_profile_read(pm_ctx* ctx, pm_profile* out, int reset);

/* ---- fused MoE layer ---------------------------------------------------- */
typedef struct pm_layer_weights {
  const void* gate_w;        /* device bf16 [num_expert, hidden] */
  const float* gate_bias;    /* device f32 [num_expert] or NULL */
  const void* shared_gate_w; /* device bf16 [hidden] or NULL (sigmoid gate on the shared expert) */
  const void* shared_w_gate; /* device bf16 [shared_inter, hidden] or NULL */
  const void* shared_w_up;   /* device bf16 [shared_inter, hidden] */
  const void* shared_w_down; /* device bf16 [hidden, shared_inter] */
  int32_t hidden;
  int32_t inter;        /* routed expert intermediate size */
  int32_t shared_inter; /* 0 = no shared expert */
  int32_t top_k;
  int32_t norm_topk;    /* renormalise the k selected probabilities */
  float routed_scale;   /* multiplies the routing weights */
  int32_t quant4;       /* routed experts are uint4 group-128 (params: q, scale/zero per matrix) */
} pm_layer_weights;
int pm_layer_set_weights(pm_ctx* ctx, int layer, const pm_layer_weights* w);

/* One MoE layer forward on device buffers: x [T, hidden] bf16 -> y [T, hidden] bf16.
 * Runs K1 (route) and K2 (permute), reads the expert counts back, performs the
 * report_layer bookkeeping and copies, then K3 (grouped SwiGLU FFN by slot) and K4 (combine).
 * Stands in for the MoE block forward the reference patches into transformers
 * (src/sparse_llm_cache/utils/__init__.py:82-89) plus the ExpertHook / MoeLayerHook calls
 * around it (src/sparse_llm_cache/utils/hooks.py:187-223). */
int pm_moe_forward(pm_ctx* ctx, int layer, const void* x_dev, int T, void* y_dev, void* stream);
/* Expert-parallel receive side: the rows were routed elsewhere. x_rows [n_rows, hidden] bf16 and
 * row_expert [n_rows] int32 (expert ids local to this context; -1 marks a padding row) are device
 * buffers; rows_out [n_rows, hidden] f32 receives each row's unweighted expert output, in row order
 * (zeros for padding rows). Cache bookkeeping, copies and the grouped FFN are those of
 * pm_moe_forward; there is no router, no shared expert and no combine (gate_w of the layer may be
 * NULL). An id outside [-1, num_expert) is PM_ERR_INVALID. max_rows_per_expert (0 = unknown) is a
 * bound on the rows one expert can receive that the caller guarantees, e.g. the number of tokens
 * in flight on all ranks: up to 16, the resident experts start before the host has read the row
 * counts. pred_scores (device f32 [n_pred, pred_width], may be NULL) are predictor scores for the
 * layers pred_layers[0..n_pred) (host int32) over the pred_width experts of the WHOLE model, of
 * which this context holds [pred_first, pred_first + num_expert): the pred_top best of the whole
 * list are taken (descending score, ties to the lower id) and those among them that this context
 * holds are prefetched in that order, before this layer's own report, so that all the contexts
 * of an expert-parallel run together prefetch what one context holding every expert would.
 * pred_width = num_expert, pred_first = 0 and pred_top = num_predict_expert_per_layer give the
 * ranking of pm_report_hidden. No counterpart in the reference, which is single-GPU
 * (src/cpp_worker/model_loader.cpp:75-79). */
int pm_moe_forward_routed(pm_ctx* ctx, int layer, const void* x_rows, int n_rows, const int32_t* row_expert,
                          float* rows_out, int max_rows_per_expert, const float* pred_scores,
                          const int32_t* pred_layers, int n_pred, int pred_width, int pred_first, int pred_top,
                          void* stream);
/* ---- pooled miss fetch for expert-parallel ranks of one node (no counterpart in the reference,
 *      which is single-GPU) -------------------------------------------------------------------
 * A layer call of an expert-parallel stack ends when the rank with the most missing experts has
 * them, and each rank's misses arrive over that rank's host link alone. With the pool every rank
 * pulls 1/world of every missing record over ITS link and the slices meet at the owner over
 * NVLink, so a layer call costs the node's total miss bytes over all links. Cache decisions are
 * the same as without it. Set-up: context option shared_arena=<name> before pm_pin_all (the
 * pinned records then live in POSIX shared memory "<name>_L<layer>"), pm_pool_init on every rank
 * with one mailbox name, then, after every rank has pinned, pm_pool_open_peer for every other rank.
 * Per layer call on every rank, in this order:
 *   pm_moe_forward_routed_begin  as pm_moe_forward_routed, but the copies of missing activated
 *                                experts are not enqueued: their local expert ids come back in
 *                                miss_experts (n_miss <= miss_cap; if there are more, the rank
 *                                copies them itself and reports 0)
 *   pm_pool_exchange             host-to-host exchange of the miss lists; lists_out is int32
 *                                [world][1 + 64]: count, then ids; waits at most timeout_s per peer
 *   pm_pool_stage                this rank's slice of every listed record, host to device into
 *                                send_dev, grouped by owner; returns the all-to-all's byte splits
 *   (the caller's all-to-all of send_dev into recv_dev with those splits, on `stream`)
 *   pm_pool_scatter              slices of this rank's records from recv_dev into their cache
 *                                lines; records the lines' ready events
 *   pm_moe_forward_routed_end    the launches that waited for those lines, then the output rows
 * pm_pool_fetch_locally makes this rank copy its collected misses itself (when the ranks agree
 * that an exchange does not fit the buffers). */
int pm_moe_forward_routed_begin(pm_ctx* ctx, int layer, const void* x_rows, int n_rows, const int32_t* row_expert,
                                float* rows_out, int max_rows_per_expert, const float* pred_scores,
                                const int32_t* pred_layers, int n_pred, int pred_width, int pred_first, int pred_top,
                                void* stream, int32_t* miss_experts, int miss_cap, int* n_miss);
int pm_moe_forward_routed_end(pm_ctx* ctx);
int pm_pool_init(pm_ctx* ctx, int rank, int world, const char* mailbox_name);
int pm_pool_open_peer(pm_ctx* ctx, int peer, const char* arena_prefix, int peer_num_expert);
int pm_pool_exchange(pm_ctx* ctx, int64_t seq, const int32_t* experts, int n, int32_t* lists_out, double timeout_s);
int pm_pool_stage(pm_ctx* ctx, int layer, const int32_t* lists, void* send_dev, size_t send_cap, size_t recv_cap,
                  int64_t* send_split, int64_t* recv_split, void* stream);
int pm_pool_scatter(pm_ctx* ctx, const void* recv_dev, void* stream);
int pm_pool_fetch_locally(pm_ctx* ctx);
/* Same with host buffers (pinned or pageable): copies x in and y out on the stream and waits. */
int pm_moe_forward_host(pm_ctx* ctx, int layer, const void* x_host, int T, void* y_host, void* stream);
/* Routing of the most recent pm_moe_forward on `layer` (host copies): ids/weights [T, k]. */
int pm_last_routing(pm_ctx* ctx, int layer, int32_t* topk_ids, float* topk_w, int cap_pairs);

/* Next-layer expert predictor (SepPredictor + PredictWorker: src/cpp_worker/predictor.cpp:558-607,
 * src/cpp_worker/worker.cpp:6-77). Weights are device pointers of one MLP
 * hidden -> d -> num_expert (bf16 matrices, f32 biases, ReLU) used for hidden states captured
 * at input index src_layer to predict dst_layer. */
int pm_predictor_set(pm_ctx* ctx, int src_layer, int dst_layer, const void* w1, const float* b1, int d,
                     const void* w2, const float* b2);
/* PrefetchMngr::report_moe_layer_logits (src/cpp_worker/prefetcher.cpp:447-460): hidden states
 * [B, seq, hidden] bf16 entering layer `index` (index == num_layer: output of the last layer).
 * Decode (seq == 1) runs the predictor on the device and issues the prefetches it ranks. */
int pm_report_hidden(pm_ctx* ctx, int index, const void* hidden_dev, int B, int seq, void* stream);

/* ---- stateless kernels (each usable on its own) -------------------------- */
int pm_k_gate_topk(const void* x, const void* gate_w, const float* gate_bias, const void* shared_gate_w,
                   int T, int H, int E, int k, int norm_topk, float routed_scale,
                   const int32_t* expert_slot, int32_t* topk_ids, float* topk_w, int32_t* topk_slot,
                   float* shared_scale, float* logits_out, void* stream);
int pm_k_permute(const int32_t* topk_ids, int R, int k, int E, int32_t* counts, int32_t* offsets,
                 int32_t* row_token, int32_t* pos, int32_t* err_flag, void* stream);

/* dst row r = src row row_index[r]; rows are row_bytes long (a multiple of 16). Used to lay token
 * rows out per expert (dispatch) and to put expert outputs back in arrival order. */
int pm_k_gather_rows(const void* src, const int32_t* row_index, int n_rows, size_t row_bytes, void* dst,
                     void* stream);

/* One group of rows sharing one set of FFN weights (device pointers). */
typedef struct pm_ffn_group {
  const void* w_gate; /* bf16 [inter, hidden], or packed uint4 [inter, hidden/2] when quant4 */
  const void* w_up;
  const void* w_down; /* bf16 [hidden, inter], or packed uint4 [hidden, inter/2] */
  const void* q_gate; /* quant4: fp16 {scale, zero} pairs [inter, hidden/128]; else NULL */
  const void* q_up;
  const void* q_down; /* quant4: [hidden, inter/128] */
  int32_t row_start;  /* first permuted row */
  int32_t row_count;
  int32_t inter;
  int32_t ld_down;    /* row pitch of w_down in elements; 0 = inter. A larger pitch (the group is a slice of
                         a wider matrix's columns) is accepted for bf16 launches of at most 16 rows per group */
} pm_ffn_group;
/* Bytes of device scratch pm_k_swiglu_ffn needs for n_rows rows in n_groups groups (launch plan:
 * group descriptors and per-tile tables, plus the bf16 intermediate rows). */
size_t pm_k_swiglu_ffn_scratch_bytes(int n_groups, int n_rows, int max_inter, int hidden);
/* Grouped SwiGLU FFN: yexp[r, :] = down(silu(gate(x[row_token[r]])) * up(x[row_token[r]])) for
 * every row r of every group. groups is a HOST array; scratch is device memory of at least
 * pm_k_swiglu_ffn_scratch_bytes(). yexp is f32 [n_rows, hidden]. Returns PM_ERR_UNSUPPORTED when
 * `stream` is being captured (the launch plan is uploaded from temporary host memory). */
int pm_k_swiglu_ffn(const pm_ffn_group* groups, int n_groups, int quant4, const void* x, int hidden,
                    const int32_t* row_token, int n_rows, float* yexp, void* scratch,
                    size_t scratch_bytes, void* stream);
/* No counterpart in the reference. The same grouped SwiGLU FFN for callers that cannot supply
 * scratch: hosts whose own pools already own all device memory, or code paths where an
 * allocation (which synchronises the device) is not acceptable. Plan and intermediate rows live
 * in an array built into the library image (pm_k_swiglu_ffn_static_capacity() bytes, 8 MiB, held
 * by every GPU that loads the library until exit); this call performs no cudaMalloc / cudaFree
 * and no allocating library call. A launch that needs more than the array holds (plan above
 * 64 KiB, or plan + n_rows * max_inter * 2 bytes above the capacity) is rejected with
 * PM_ERR_INVALID. bf16 experts only (groups with scale/zero tensors are rejected). The first call
 * on a device looks the array's device address up. A call on a stream that is being captured is
 * refused with PM_ERR_UNSUPPORTED. All calls share the array: calls that overlap on the GPU race,
 * serialise them. */
size_t pm_k_swiglu_ffn_static_capacity(void);
int pm_k_swiglu_ffn_static(const pm_ffn_group* groups, int n_groups, const void* x, int hidden,
                           const int32_t* row_token, int n_rows, float* yexp, void* stream);
/* Expert-parallel exchange buffers (no counterpart in the reference, which is single-GPU). One
 * fixed-size message per peer and direction, so the per-layer dispatch is one all-to-all with
 * split sizes known in advance. Message of a source to owner g: 1 + cap rows of `hidden` bf16;
 * row 0 = header (int32 counts[max_block] of the rows for each of g's experts, then float
 * scores[n_pred][num_expert], the source's predictor scores of all experts), rows 1.. = the token
 * rows routed to g's experts in expert order. pm_k_ep_pack builds the n_ranks messages from the
 * permutation's outputs (counts, offsets, row_token, pos; bounds_dev = device int32 [n_ranks + 1],
 * rank g owns experts [bounds[g], bounds[g+1])) and writes pos_reply [n_pairs]: the row of the
 * reply buffer [n_ranks * (1 + cap), hidden] f32 where the output of routed pair (t, j) returns.
 * pm_k_ep_unpack turns a receive buffer into row_expert [n_ranks * (1 + cap)] (local expert id,
 * -1 for header and unused rows: the row list pm_moe_forward_routed takes) and scores_sum
 * [n_pred, num_expert] (the sources' scores added in rank order: identical on every owner). */
int pm_k_ep_pack(const void* x, int hidden, const int32_t* counts, const int32_t* offsets,
                 const int32_t* row_token, const int32_t* pos, int n_pairs, const int32_t* bounds_dev,
                 int n_ranks, int max_block, int cap, const float* scores, int n_pred, int num_expert,
                 void* send, int32_t* pos_reply, void* stream);
int pm_k_ep_unpack(const void* recv, int hidden, int n_ranks, int n_local, int max_block, int cap, int n_pred,
                   int num_expert, int32_t* row_expert, float* scores_sum, int32_t* err_flag, void* stream);
int pm_k_combine(const float* yexp, const int32_t* pos, const float* topk_w, int T, int H, int k, int R,
                 int n_shared, const float* shared_scale, void* y, void* stream);
/* scores[e] = sum_b (W2 relu(W1 x_b + b1) + b2)[e]; hidden_scratch is f32 [B, d] device scratch. */
int pm_k_predictor_mlp(const void* x, int B, int H, const void* w1, const float* b1, int d,
                       const void* w2, const float* b2, int E, float* hidden_scratch, float* scores,
                       void* stream);
/* out[r] = id of the r-th best of scores[0 .. width), r < n: descending score, equal scores in
 * ascending id (rank_experts, src/cpp_worker/predictor.hpp:24-28, ranks the same way on the host). */
int pm_k_rank_topn(const float* scores, int width, int n, int32_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PROMOE_B200_H_ */
