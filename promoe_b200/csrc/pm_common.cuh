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
  int32_t pad;
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

cudaError_t launch_permute(const int32_t* topk_ids, int R, int k, int E, int32_t* counts,
                           int32_t* offsets, int32_t* row_token, int32_t* pos, int32_t* err_flag,
                           int tail_rows, int T, cudaStream_t s, int32_t* scratch = nullptr,
                           size_t scratch_ints = 0);

// Geometry of one grouped FFN launch pair. The device blob it describes holds, 16-byte aligned
// and in this order: n_desc GroupDesc, tiles_gu int32 (chunk index of every gate/up CTA tile),
// tiles_dn int32 (same for the down launch), then two int32 tile counters that start at zero.
struct FfnPlanInfo {
  int n_desc = 0, tiles_gu = 0, tiles_dn = 0, max_rows = 0, max_inter = 0;
  size_t off_tile_gu() const { return ((size_t)n_desc * sizeof(GroupDesc) + 15) / 16 * 16; }
  size_t off_tile_dn() const { return off_tile_gu() + ((size_t)tiles_gu * 4 + 15) / 16 * 16; }
  size_t off_counters() const { return off_tile_dn() + ((size_t)tiles_dn * 4 + 15) / 16 * 16; }
  size_t blob_bytes() const { return off_counters() + 16; }  // two zeroed tile counters (fused kernel)
};

// Splits caller groups into chunks of at most kMaxChunkRows rows, assigns CTA tile ranges and
// writes the blob into `blob` (host memory, `cap` bytes). Allocates nothing.
int plan_groups_into(const pm_ffn_group* groups, int n_groups, int hidden, unsigned char* blob, size_t cap,
                     FfnPlanInfo* info, int chunk_rows = kMaxChunkRows);
// Size pass of the same planner (blob == nullptr): fills `info` only.
int plan_groups_size(const pm_ffn_group* groups, int n_groups, int hidden, FfnPlanInfo* info,
                     int chunk_rows = kMaxChunkRows);

// Everything the device-side planner needs to describe the resident experts of one layer.
struct ResidentPlanArgs {
  const unsigned char* pool_base;  // first cache line of the layer's pool
  size_t line_stride;
  size_t off_gate, off_up, off_down;  // tensor offsets inside a line
  const void *shared_w_gate, *shared_w_up, *shared_w_down;
  int32_t num_expert, inter, shared_inter, hidden;
  int32_t tokens, n_routed_rows;
  // byte offsets of the sections inside the device blob (header of five int32 at offset 0)
  size_t off_desc, off_tile_gu, off_tile_dn;
  // Section sizes for num_expert experts plus the shared expert.
  static size_t blob_bytes(int num_expert, int inter, int shared_inter, int hidden, size_t* off_desc,
                           size_t* off_gu, size_t* off_dn) {
    const size_t n = (size_t)num_expert + 1;
    const size_t gu = (size_t)num_expert * (inter / kSplitTileGu) + shared_inter / kSplitTileGu;
    const size_t dn = n * (hidden / kSplitTileDn);
    *off_desc = 64;
    *off_gu = *off_desc + n * sizeof(GroupDesc);
    *off_dn = *off_gu + (gu * 4 + 15) / 16 * 16;
    return *off_dn + (dn * 4 + 15) / 16 * 16;
  }
};
// Plans (on the device) and launches the fused FFN for the shared expert and every activated
// expert that the slot table shows resident. start_event (optional) is recorded between the
// planner and the FFN kernel. Needs cooperative launch and at most kSplitMaxRows rows per expert.
cudaError_t launch_resident_ffn(const int32_t* counts, const int32_t* offsets, const int32_t* slot_table,
                                const ResidentPlanArgs& a, unsigned char* blob_dev, int max_rows,
                                const __nv_bfloat16* x, const int32_t* row_token, __nv_bfloat16* hbuf, int ld_h,
                                float* yexp, cudaStream_t s, cudaEvent_t start_event);
bool resident_ffn_available(int max_rows);

// Launches of at most kSplitMaxRows rows per chunk run as ONE cooperative kernel (gate/up tiles,
// grid barrier, down tiles) unless `fused` is false or a mid_event is wanted; mid_event
// (optional) is recorded between the gate/up and the down launch of the two-launch path.
cudaError_t launch_swiglu_ffn(const unsigned char* blob_dev, const FfnPlanInfo& info, int quant4,
                              const __nv_bfloat16* x, int H, const int32_t* row_token,
                              __nv_bfloat16* hbuf, int ld_h, float* yexp, cudaStream_t s,
                              cudaEvent_t mid_event = nullptr, bool fused = true);

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

cudaError_t launch_predictor_mlp(const __nv_bfloat16* x, int B, int H, const __nv_bfloat16* w1,
                                 const float* b1, int D, const __nv_bfloat16* w2, const float* b2,
                                 int E, float* hidden_scratch, float* scores, cudaStream_t s);

}  // namespace pm
