// C-ABI entry points of the stateless kernels, plus the per-thread error message.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "pm_common.cuh"

namespace pm {

static thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

int fail_cuda(cudaError_t e, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return PM_ERR_CUDA;
}

// One planner for both passes: with blob == nullptr it only sizes the launch.
static int plan_core(const pm_ffn_group* groups, int n_groups, int hidden, unsigned char* blob, size_t cap,
                     FfnPlanInfo* info, int chunk_rows) {
  if (hidden <= 0 || hidden % 64 != 0) return fail(PM_ERR_INVALID, "hidden must be a positive multiple of 64");
  // The kernel variant, and with it the tile size, follows from the largest chunk of the launch.
  int largest = 0;
  for (int i = 0; i < n_groups; ++i) largest = std::max(largest, std::min(groups[i].row_count, chunk_rows));
  const bool split = largest <= kSplitMaxRows;
  const int tile_gu = split ? kSplitTileGu : kTileRows;
  const int tile_dn = split ? kSplitTileDn : kTileRows;
  FfnPlanInfo sized;
  if (blob != nullptr) {
    sized = *info;  // result of the size pass
    if (sized.blob_bytes() > cap) return fail(PM_ERR_INVALID, "launch plan does not fit its buffer");
  }
  GroupDesc* desc = reinterpret_cast<GroupDesc*>(blob);
  int32_t* t_gu = blob ? reinterpret_cast<int32_t*>(blob + sized.off_tile_gu()) : nullptr;
  int32_t* t_dn = blob ? reinterpret_cast<int32_t*>(blob + sized.off_tile_dn()) : nullptr;
  int n = 0, tg = 0, td = 0, mr = 0, mi = 0;
  for (int i = 0; i < n_groups; ++i) {
    const pm_ffn_group& g = groups[i];
    if (g.row_count <= 0) continue;
    if (g.inter % 32 != 0 || g.inter <= 0) return fail(PM_ERR_INVALID, "inter must be a positive multiple of 32");
    if (g.ld_down != 0 && g.ld_down != g.inter && (g.ld_down < g.inter || !split))
      return fail(PM_ERR_INVALID, "ld_down must be 0 or at least inter, and a wider pitch needs chunks of at most 16 rows");
    for (int r0 = 0; r0 < g.row_count; r0 += chunk_rows) {
      const int n_gu = (g.inter + tile_gu - 1) / tile_gu, n_dn = hidden / tile_dn;
      if (blob != nullptr) {
        GroupDesc d{};
        d.w_gate = g.w_gate; d.w_up = g.w_up; d.w_down = g.w_down;
        d.q_gate = g.q_gate; d.q_up = g.q_up; d.q_down = g.q_down;
        d.row_start = g.row_start + r0;
        d.row_count = std::min(chunk_rows, g.row_count - r0);
        d.inter = g.inter;
        d.ld_down = g.ld_down;
        d.tile_start_gu = tg;
        d.tile_start_dn = td;
        desc[n] = d;
        for (int t = 0; t < n_gu; ++t) t_gu[tg + t] = n;
        for (int t = 0; t < n_dn; ++t) t_dn[td + t] = n;
      }
      tg += n_gu;
      td += n_dn;
      mr = std::max(mr, std::min(chunk_rows, g.row_count - r0));
      mi = std::max(mi, g.inter);
      ++n;
    }
  }
  info->n_desc = n; info->tiles_gu = tg; info->tiles_dn = td; info->max_rows = mr; info->max_inter = mi;
  if (blob != nullptr) std::memset(blob + info->off_counters(), 0, info->counter_bytes());
  return PM_OK;
}

int plan_groups_size(const pm_ffn_group* groups, int n_groups, int hidden, FfnPlanInfo* info, int chunk_rows) {
  return plan_core(groups, n_groups, hidden, nullptr, 0, info, chunk_rows);
}

int plan_groups_into(const pm_ffn_group* groups, int n_groups, int hidden, unsigned char* blob, size_t cap,
                     FfnPlanInfo* info, int chunk_rows) {
  return plan_core(groups, n_groups, hidden, blob, cap, info, chunk_rows);
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// The grouped FFN entry points upload their launch plan from host memory that dies when the call
// returns. Outside a capture the bytes are staged before cudaMemcpyAsync returns; inside one the
// graph would keep the host pointer and read it at every graph launch. So they refuse.
int refuse_if_capturing(cudaStream_t s, const char* who) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  PM_CUDA(cudaStreamIsCapturing(s, &st));
  if (st != cudaStreamCaptureStatusNone)
    return fail(PM_ERR_UNSUPPORTED, std::string(who) + ": the stream is capturing; this call uploads a launch plan "
                                    "from temporary host memory and cannot be part of a CUDA graph");
  return PM_OK;
}

}  // namespace pm

using namespace pm;

extern "C" {

int pm_version(void) { return 100; }

const char* pm_last_error(void) { return g_last_error.c_str(); }

int pm_k_gate_topk(const void* x, const void* gate_w, const float* gate_bias, const void* shared_gate_w,
                   int T, int H, int E, int k, int norm_topk, float routed_scale,
                   const int32_t* expert_slot, int32_t* topk_ids, float* topk_w, int32_t* topk_slot,
                   float* shared_scale, float* logits_out, void* stream) {
  if (T < 0 || H <= 0 || H % 8 != 0) return fail(PM_ERR_INVALID, "gate_topk: hidden must be a positive multiple of 8");
  if (E <= 0 || E > 256) return fail(PM_ERR_INVALID, "gate_topk: num_expert must be in [1, 256]");
  if (k <= 0 || k > 16 || k > E) return fail(PM_ERR_INVALID, "gate_topk: top_k must be in [1, min(16, num_expert)]");
  if (T == 0) return PM_OK;
  if (!x || !gate_w || !topk_ids || !topk_w) return fail(PM_ERR_INVALID, "gate_topk: null pointer");
  PM_CUDA(launch_gate_topk((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate_w, gate_bias,
                           (const __nv_bfloat16*)shared_gate_w, T, H, E, k, norm_topk, routed_scale,
                           expert_slot, topk_ids, topk_w, topk_slot, shared_scale, logits_out,
                           (cudaStream_t)stream));
  return PM_OK;
}

int pm_k_permute(const int32_t* topk_ids, int R, int k, int E, int32_t* counts, int32_t* offsets,
                 int32_t* row_token, int32_t* pos, int32_t* err_flag, void* stream) {
  if (R < 0 || k <= 0 || E <= 0 || E > 256) return fail(PM_ERR_INVALID, "permute: bad sizes");
  if (!counts || !offsets) return fail(PM_ERR_INVALID, "permute: null pointer");
  if (R > 0 && (!topk_ids || !row_token || !pos)) return fail(PM_ERR_INVALID, "permute: null pointer");
  PM_CUDA(launch_permute(topk_ids, R, k, E, counts, offsets, row_token, pos, err_flag, 0, 1, (cudaStream_t)stream));
  return PM_OK;
}

int pm_k_gather_rows(const void* src, const int32_t* row_index, int n_rows, size_t row_bytes, void* dst,
                     void* stream) {
  if (n_rows < 0 || row_bytes == 0 || row_bytes % 16 != 0) return fail(PM_ERR_INVALID, "gather_rows: row_bytes must be a positive multiple of 16");
  if (n_rows == 0) return PM_OK;
  if (!src || !row_index || !dst) return fail(PM_ERR_INVALID, "gather_rows: null pointer");
  PM_CUDA(launch_gather_rows(src, row_index, n_rows, row_bytes, dst, (cudaStream_t)stream));
  return PM_OK;
}

size_t pm_k_swiglu_ffn_scratch_bytes(int n_groups, int n_rows, int max_inter, int hidden) {
  if (n_groups < 0 || n_rows < 0 || max_inter < 0 || hidden < 0) return 0;
  // worst case: every group split into chunks of kMaxChunkRows rows, smallest tiles
  FfnPlanInfo worst;
  worst.n_desc = n_groups + n_rows / kSplitMaxRows + 1;
  worst.tiles_gu = worst.n_desc * ((max_inter + kSplitTileGu - 1) / kSplitTileGu);
  worst.tiles_dn = worst.n_desc * ((hidden + kSplitTileDn - 1) / kSplitTileDn);
  return align_up(worst.blob_bytes(), 256) + align_up((size_t)n_rows * max_inter * 2, 256);
}

int pm_k_swiglu_ffn(const pm_ffn_group* groups, int n_groups, int quant4, const void* x, int hidden,
                    const int32_t* row_token, int n_rows, float* yexp, void* scratch,
                    size_t scratch_bytes, void* stream) {
  if (n_groups < 0 || n_rows < 0) return fail(PM_ERR_INVALID, "swiglu_ffn: negative size");
  if (n_groups == 0 || n_rows == 0) return PM_OK;
  if (!groups || !x || !row_token || !yexp || !scratch) return fail(PM_ERR_INVALID, "swiglu_ffn: null pointer");
  {
    int rc = refuse_if_capturing((cudaStream_t)stream, "swiglu_ffn");
    if (rc != PM_OK) return rc;
  }
  for (int i = 0; i < n_groups; ++i)
    if (groups[i].row_count > 0 && (groups[i].row_start < 0 || groups[i].row_start + groups[i].row_count > n_rows))
      return fail(PM_ERR_INVALID, "swiglu_ffn: group rows outside [0, n_rows)");
  if (quant4) {
    if (hidden % 128 != 0) return fail(PM_ERR_INVALID, "swiglu_ffn: uint4 experts need hidden % 128 == 0");
    for (int i = 0; i < n_groups; ++i) {
      if (groups[i].row_count > 0 && groups[i].inter % 128 != 0)
        return fail(PM_ERR_INVALID, "swiglu_ffn: uint4 experts need inter % 128 == 0");
      if (groups[i].row_count > 0 && (!groups[i].q_gate || !groups[i].q_up || !groups[i].q_down))
        return fail(PM_ERR_INVALID, "swiglu_ffn: uint4 experts need scale/zero tensors");
    }
  }
  const int chunk_rows = quant4 ? kSplitMaxRows : kMaxChunkRows;
  FfnPlanInfo info;
  int rc = plan_groups_size(groups, n_groups, hidden, &info, chunk_rows);
  if (rc != PM_OK) return rc;
  if (info.n_desc == 0) return PM_OK;
  const size_t plan_bytes = align_up(info.blob_bytes(), 256);
  const size_t need = plan_bytes + align_up((size_t)n_rows * info.max_inter * 2, 256);
  if (scratch_bytes < need) return fail(PM_ERR_INVALID, "swiglu_ffn: scratch too small");
  std::vector<unsigned char> blob(info.blob_bytes());
  rc = plan_groups_into(groups, n_groups, hidden, blob.data(), blob.size(), &info, chunk_rows);
  if (rc != PM_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  // The plan upload is from pageable memory, so it is staged before this call returns.
  PM_CUDA(cudaMemcpyAsync(scratch, blob.data(), blob.size(), cudaMemcpyHostToDevice, s));
  __nv_bfloat16* hbuf = (__nv_bfloat16*)((unsigned char*)scratch + plan_bytes);
  if (quant4)
    for (int i = 0; i < n_groups; ++i)
      if (groups[i].row_count > 0 && groups[i].ld_down != 0 && groups[i].ld_down != groups[i].inter)
        return fail(PM_ERR_INVALID, "swiglu_ffn: uint4 experts take no ld_down");
  PM_CUDA(launch_swiglu_ffn((const unsigned char*)scratch, info, quant4, (const __nv_bfloat16*)x, hidden,
                            row_token, hbuf, info.max_inter, yexp, s, nullptr));
  return PM_OK;
}

int pm_k_combine(const float* yexp, const int32_t* pos, const float* topk_w, int T, int H, int k, int R,
                 int n_shared, const float* shared_scale, void* y, void* stream) {
  if (T < 0 || H <= 0 || H % 4 != 0 || k <= 0 || k > 16) return fail(PM_ERR_INVALID, "combine: bad sizes");
  if (T == 0) return PM_OK;
  if (!yexp || !pos || !topk_w || !y) return fail(PM_ERR_INVALID, "combine: null pointer");
  PM_CUDA(launch_combine(yexp, pos, topk_w, T, H, k, R, n_shared, shared_scale, (__nv_bfloat16*)y,
                         (cudaStream_t)stream));
  return PM_OK;
}

int pm_k_predictor_mlp(const void* x, int B, int H, const void* w1, const float* b1, int d,
                       const void* w2, const float* b2, int E, float* hidden_scratch, float* scores,
                       void* stream) {
  if (B < 0 || H <= 0 || H % 8 != 0 || d <= 0 || E <= 0) return fail(PM_ERR_INVALID, "predictor_mlp: bad sizes");
  if (B == 0) return PM_OK;
  if (!x || !w1 || !w2 || !hidden_scratch || !scores) return fail(PM_ERR_INVALID, "predictor_mlp: null pointer");
  PM_CUDA(launch_predictor_mlp((const __nv_bfloat16*)x, B, H, (const __nv_bfloat16*)w1, b1, d,
                               (const __nv_bfloat16*)w2, b2, E, hidden_scratch, scores,
                               (cudaStream_t)stream));
  return PM_OK;
}

int pm_k_rank_topn(const float* scores, int width, int n, int32_t* out, void* stream) {
  if (width <= 0 || n < 0 || n > width || width > 9000) return fail(PM_ERR_INVALID, "rank_topn: bad sizes");
  if (n == 0) return PM_OK;
  if (!scores || !out) return fail(PM_ERR_INVALID, "rank_topn: null pointer");
  PM_CUDA(launch_rank_topn(scores, width, n, out, (cudaStream_t)stream));
  return PM_OK;
}

}  // extern "C"
