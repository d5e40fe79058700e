// Shared declarations for the sm_100a kernels and the host runtime of the MoE hot path.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#pragma GCC visibility push(default)
#include "../../include/promoe_b200.h"
#pragma GCC visibility pop

namespace pm {

// Records a message retrievable through pm_last_error(NULL) and returns `code`.
int fail(int code, const std::string& msg);
int fail_cuda(cudaError_t e, const char* what);
// PM_ERR_UNSUPPORTED (with a message naming `who`) while stream `s` is being captured into a graph.
int refuse_if_capturing(cudaStream_t s, const char* who);

#define PM_CUDA(expr)                                         \
  do {                                                        \
    cudaError_t pm_e_ = (expr);                               \
    if (pm_e_ != cudaSuccess) return pm::fail_cuda(pm_e_, #expr); \
  } while (0)

// One chunk of rows that share one set of FFN weights: a routed expert resolved
// to its cache slot, or a shared expert. Rows are positions in the permuted
// (expert-sorted) row order; a chunk never holds more than kMaxChunkRows rows.
struct GroupDesc {
  const void* w_gate;   // [inter, hidden] bf16, or packed uint4 [inter, hidden/2]
  const void* w_up;     // same layout as w_gate
  const void* w_down;   // [hidden, inter] bf16, or packed uint4 [hidden, inter/2]
  const void* q_gate;   // int4 only: per (row, 128-group) {scale, zero} fp16 pairs
  const void* q_up;
  const void* q_down;
  int32_t row_start;
  int32_t row_count;
  int32_t inter;
  int32_t tile_start_gu;  // first CTA tile of this chunk in the gate/up launch
  int32_t tile_start_dn;  // first CTA tile of this chunk in the down launch
  int32_t ld_down;        // row pitch of w_down in elements (0 = inter); larger when the chunk is one
                          // slice of a wider matrix's reduction dimension (fused decode kernel only)
};

constexpr int kTileRows = 64;       // weight rows per CTA tile of the staged kernel (4 warps x 16)
constexpr int kMaxChunkRows = 64;   // token rows per chunk (8 MMA n-tiles)
constexpr int kSplitMaxRows = 16;   // launches whose chunks all fit use the split-K decode kernel,
constexpr int kSplitTileGu = 16;    // whose tiles are 16 gate+up rows
constexpr int kSplitTileDn = 32;    // or 32 down rows

// Kernel launchers (defined in the .cu files). All take the caller's stream.
cudaError_t launch_gate_topk(const __nv_bfloat16* x, const __nv_bfloat16* w_gate, const float* bias,
                             const __nv_bfloat16* w_shared_gate, int T, int H, int E, int k,
                             int norm_topk, float routed_scale, const int32_t* expert_slot,
                             int32_t* topk_ids, float* topk_w, int32_t* topk_slot,
                             float* shared_scale, float* logits_out, cudaStream_t s);

// zero_words / zero_n: an int32 array the permutation also clears (the dependency counters of the
// fused FFN launch that follows on the same stream), or nullptr.
cudaError_t launch_permute(const int32_t* topk_ids, int R, int k, int E, int32_t* counts,
                           int32_t* offsets, int32_t* row_token, int32_t* pos, int32_t* err_flag,
                           int tail_rows, int T, cudaStream_t s, int32_t* scratch = nullptr,
                           size_t scratch_ints = 0, int32_t* zero_words = nullptr, int zero_n = 0);

// Geometry of one grouped FFN launch pair. The device blob it describes holds, 16-byte aligned
// and in this order: n_desc GroupDesc, tiles_gu int32 (chunk index of every gate/up CTA tile),
// tiles_dn int32 (same for the down launch), then n_desc + 1 int32 dependency counters that start
// at zero (the fused kernel counts the finished gate/up tiles per chunk and in total there) and one
// int32 error word.
struct FfnPlanInfo {
  int n_desc = 0, tiles_gu = 0, tiles_dn = 0, max_rows = 0, max_inter = 0;
  size_t off_tile_gu() const { return ((size_t)n_desc * sizeof(GroupDesc) + 15) / 16 * 16; }
  size_t off_tile_dn() const { return off_tile_gu() + ((size_t)tiles_gu * 4 + 15) / 16 * 16; }
  size_t off_counters() const { return off_tile_dn() + ((size_t)tiles_dn * 4 + 15) / 16 * 16; }
  size_t counter_bytes() const { return ((size_t)(n_desc + 2) * 4 + 15) / 16 * 16; }
  size_t blob_bytes() const { return off_counters() + counter_bytes(); }
};

// Splits caller groups into chunks of at most kMaxChunkRows rows, assigns CTA tile ranges and
// writes the blob into `blob` (host memory, `cap` bytes). Allocates nothing.
int plan_groups_into(const pm_ffn_group* groups, int n_groups, int hidden, unsigned char* blob, size_t cap,
                     FfnPlanInfo* info, int chunk_rows = kMaxChunkRows);
// Size pass of the same planner (blob == nullptr): fills `info` only.
int plan_groups_size(const pm_ffn_group* groups, int n_groups, int hidden, FfnPlanInfo* info,
                     int chunk_rows = kMaxChunkRows);

constexpr int kMaxSharedSlices = 8;
constexpr int kMaxFusedGroups = 256 + kMaxSharedSlices;  // groups of one fused launch
constexpr int kMaxFusedGroupsQ4 = 128;                    // same for uint4 experts (larger table records)

// What the fused kernel needs to describe, on the device, the shared expert and the routed experts
// a layer's slot table shows resident (no host round trip between the router and this launch).
// The shared expert is cut along its intermediate dimension into slices of `shared_slice` columns,
// each a group of its own with its own output rows (the combine adds them), so that every tile
// of the launch has about the same weight bytes.
struct ResidentArgs {
  const int32_t* counts;      // [num_expert] routed rows per expert (permutation output)
  const int32_t* offsets;     // [num_expert + 1]
  const int32_t* slot_table;  // [num_expert] cache slot of each expert, -1 = absent
  const unsigned char* pool_base;  // first cache line of the layer's pool
  size_t line_stride;
  size_t off_gate, off_up, off_down;  // tensor offsets inside a line
  const void *shared_w_gate, *shared_w_up, *shared_w_down;
  int32_t num_expert, inter, shared_inter, shared_slice;
  int32_t tokens, n_routed_rows;
};
// Width of one slice of a shared expert of width shared_inter beside routed experts of width inter.
inline int shared_slice_width(int inter, int shared_inter) {
  int w = inter > 0 ? inter : shared_inter;
  const int least = (shared_inter + kMaxSharedSlices - 1) / kMaxSharedSlices;
  if (w < least) w = least;
  w = (w + 31) / 32 * 32;
  return w < shared_inter ? w : shared_inter;
}
inline int shared_slice_count(int inter, int shared_inter) {
  if (shared_inter <= 0) return 0;
  const int w = shared_slice_width(inter, shared_inter);
  return (shared_inter + w - 1) / w;
}
// Launches the fused FFN for the shared expert (sliced) and every activated resident expert.
// counters: kMaxFusedGroups + 1 int32 (per chunk, then the launch total), zero at launch. err: a device word that receives a non-zero
// code if a bounded dependency wait gives up. Needs cooperative launch and at most kSplitMaxRows
// rows per expert.
cudaError_t launch_resident_ffn(const ResidentArgs& a, int32_t* counters, int32_t* err, int max_rows,
                                const __nv_bfloat16* x, int hidden, const int32_t* row_token,
                                __nv_bfloat16* hbuf, int ld_h, float* yexp, cudaStream_t s);
bool resident_ffn_available(int max_rows);

// Launches of at most kSplitMaxRows rows per chunk run as ONE cooperative kernel (gate/up tiles,
// then down tiles, a chunk's down tiles waiting on its gate/up tiles through the blob's counters),
// bf16 and uint4 alike (up to kMaxFusedGroups / kMaxFusedGroupsQ4 chunks); anything else runs as a gate/up and
// a down launch, and mid_event (optional) is recorded between the two. err (optional): device word
// that receives a code when a bounded wait of the fused kernel gives up (default: the blob's own
// error word).
cudaError_t launch_swiglu_ffn(const unsigned char* blob_dev, const FfnPlanInfo& info, int quant4,
                              const __nv_bfloat16* x, int H, const int32_t* row_token,
                              __nv_bfloat16* hbuf, int ld_h, float* yexp, cudaStream_t s,
                              cudaEvent_t mid_event = nullptr, int32_t* err = nullptr);
inline bool ffn_launch_is_fused(const FfnPlanInfo& info, int quant4) {
  return info.max_rows <= kSplitMaxRows && info.n_desc <= (quant4 ? kMaxFusedGroupsQ4 : kMaxFusedGroups);
}

// uint4 group-128 matrix [rows, K] (packed words + {scale, zero} fp16 pairs) -> bf16 [rows, K].
cudaError_t launch_dequant_q4(const void* packed, const void* scale_zero, int rows, int K, __nv_bfloat16* out,
                              cudaStream_t s);

cudaError_t launch_gather_rows(const void* src, const int32_t* index, int n_rows, size_t row_bytes, void* dst,
                               cudaStream_t s);

cudaError_t launch_combine(const float* yexp, const int32_t* pos, const float* topk_w, int T, int H,
                           int k, int R, int n_shared, const float* shared_scale,
                           __nv_bfloat16* y, cudaStream_t s);

// ---- prefill path (tcgen05) ---------------------------------------------------------------------
// Tensor maps of one launch pair: token rows (expert-sorted x, intermediate h), the slab (3-D:
// k, weight row, cache line) per projection, and the layer's shared expert (2-D).
struct TcMaps {
  CUtensorMap a_x, a_h, slab_gate, slab_up, slab_down, sh_gate, sh_up, sh_down;
};
struct TcGroup {
  int32_t row_start, row_count, inter;
  int32_t line;  // global cache line of the expert, -1 = the shared expert
};
struct TcTile {
  int32_t group, m0, n0, pad;
};
cudaError_t launch_prefill_ffn(const TcMaps& maps, const TcGroup* groups_dev, const TcTile* tiles_gu_dev, int n_gu,
                               const TcTile* tiles_dn_dev, int n_dn, int hidden, __nv_bfloat16* hbuf, int ld_h,
                               float* yexp, int32_t* err_dev, cudaStream_t s, cudaEvent_t mid_event);

// out[r] = index of the r-th best of scores[0 .. width) (descending, ties to the lower index), r < n.
cudaError_t launch_rank_topn(const float* scores, int width, int n, int32_t* out, cudaStream_t s);

cudaError_t launch_predictor_mlp(const __nv_bfloat16* x, int B, int H, const __nv_bfloat16* w1,
                                 const float* b1, int D, const __nv_bfloat16* w2, const float* b2,
                                 int E, float* hidden_scratch, float* scores, cudaStream_t s);

}  // namespace pm
