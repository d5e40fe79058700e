// Expert-parallel exchange buffers: what one rank sends to and receives from every peer in one
// fixed-size all-to-all per direction.
//
// The reference has no multi-GPU path (device 0 is hard-coded, src/cpp_worker/model_loader.cpp:75-79);
// these two kernels only lay tokens out so that the per-layer exchange is ONE collective each way
// with split sizes known in advance: no count exchange and no host round trip before the dispatch.
//
// Message of source rank s to owner rank g: `seg_rows` = 1 + cap rows of `hidden` bf16.
//   row 0      header: int32 counts[max_block] (rows for each of g's experts, ascending expert id),
//              then float scores[n_pred][num_expert] (this source's predictor scores of ALL experts:
//              every owner adds up the same vectors, so all owners rank the same global list)
//   row 1 + i  the i-th token row routed to one of g's experts, sorted by expert id; i < sum(counts)
//   the rest   unused
// The owner treats the whole receive buffer [G * seg_rows, hidden] as its row list: header rows
// and unused rows get expert id -1 (padding), so nothing has to be compacted.
// The reply has the same geometry in f32: row 1 + i of segment g carries the expert output of the
// row the source put there, so a source finds the output of its sorted row r, owned by rank g,
// at g * seg_rows + 1 + (r - first sorted row of g).
#include "pm_common.cuh"

namespace pm {
namespace {

constexpr int kMaxRanks = 64;

__global__ void __launch_bounds__(256)
ep_pack_kernel(const uint4* __restrict__ x, int row_vec, const int32_t* __restrict__ counts,
               const int32_t* __restrict__ offsets, const int32_t* __restrict__ row_token,
               const int32_t* __restrict__ pos, int n_pairs, const int32_t* __restrict__ bounds, int n_ranks,
               int max_block, int cap, const float* __restrict__ scores, int n_pred, int num_expert,
               uint4* __restrict__ send, int32_t* __restrict__ pos_reply) {
  const int g = blockIdx.x;  // destination rank
  const int seg_rows = 1 + cap;
  const int e0 = bounds[g], e1 = bounds[g + 1];
  const int start = offsets[e0], n = offsets[e1] - start;
  uint4* seg = send + (size_t)g * seg_rows * row_vec;
  // header (first CTA of the segment)
  if (blockIdx.y == 0) {
    int32_t* hdr_counts = reinterpret_cast<int32_t*>(seg);
    float* hdr_scores = reinterpret_cast<float*>(seg) + max_block;
    for (int i = threadIdx.x; i < max_block; i += blockDim.x) hdr_counts[i] = (e0 + i < e1) ? counts[e0 + i] : 0;
    for (int i = threadIdx.x; i < n_pred * num_expert; i += blockDim.x) hdr_scores[i] = scores[i];
  }
  // rows, dealt to the CTAs of the segment
  for (int i = blockIdx.y; i < n; i += gridDim.y) {
    const uint4* src = x + (size_t)row_token[start + i] * row_vec;
    uint4* dst = seg + (size_t)(1 + i) * row_vec;
    for (int v = threadIdx.x; v < row_vec; v += blockDim.x) dst[v] = src[v];
  }
  // where each routed pair's expert output will sit in the reply buffer
  const int n_cta = gridDim.x * gridDim.y, cta = blockIdx.y * gridDim.x + blockIdx.x;
  for (int p = cta * blockDim.x + threadIdx.x; p < n_pairs; p += n_cta * blockDim.x) {
    const int r = pos[p];
    int owner = 0;
    while (owner + 1 < n_ranks && offsets[bounds[owner + 1]] <= r) ++owner;
    pos_reply[p] = r < 0 ? -1 : owner * seg_rows + 1 + (r - offsets[bounds[owner]]);
  }
}

__global__ void __launch_bounds__(256)
ep_unpack_kernel(const uint4* __restrict__ recv, int row_vec, int n_ranks, int n_local, int max_block, int cap,
                 int n_pred, int num_expert, int32_t* __restrict__ row_expert, float* __restrict__ scores_sum,
                 int32_t* __restrict__ err) {
  __shared__ int prefix[257];
  const int seg_rows = 1 + cap;
  for (int s = 0; s < n_ranks; ++s) {
    const int32_t* hdr = reinterpret_cast<const int32_t*>(recv + (size_t)s * seg_rows * row_vec);
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      bool bad = false;
      for (int e = 0; e < n_local; ++e) {
        prefix[e] = run;
        const int c = hdr[e];
        if (c < 0 || c > cap) bad = true;
        run += bad ? 0 : c;
      }
      if (run > cap) bad = true;
      prefix[n_local] = bad ? 0 : run;  // a corrupt header voids the whole segment
      if (bad && err != nullptr) atomicExch(err, 1);
    }
    __syncthreads();
    const int total = prefix[n_local];
    int32_t* out = row_expert + (size_t)s * seg_rows;
    if (threadIdx.x == 0) out[0] = -1;  // the header row
    for (int i = threadIdx.x; i < cap; i += blockDim.x) {
      int e = -1;
      if (i < total) {
        e = 0;
        while (e + 1 < n_local && prefix[e + 1] <= i) ++e;
      }
      out[1 + i] = e;
    }
  }
  // predictor scores of all experts, summed over the sources in rank order (the same on every owner)
  for (int i = threadIdx.x; i < n_pred * num_expert; i += blockDim.x) {
    float sum = 0.f;
    for (int s = 0; s < n_ranks; ++s) {
      const float* sc = reinterpret_cast<const float*>(recv + (size_t)s * seg_rows * row_vec) + max_block;
      sum += sc[i];
    }
    scores_sum[i] = sum;
  }
}

}  // namespace
}  // namespace pm

using namespace pm;

extern "C" {

int pm_k_ep_pack(const void* x, int hidden, const int32_t* counts, const int32_t* offsets,
                 const int32_t* row_token, const int32_t* pos, int n_pairs, const int32_t* bounds_dev,
                 int n_ranks, int max_block, int cap, const float* scores, int n_pred, int num_expert,
                 void* send, int32_t* pos_reply, void* stream) {
  if (hidden <= 0 || hidden % 8 != 0 || n_ranks <= 0 || n_ranks > kMaxRanks || max_block <= 0 || max_block > 256 ||
      cap < 0 || n_pairs < 0 || n_pred < 0)
    return fail(PM_ERR_INVALID, "ep_pack: bad sizes");
  if ((size_t)(max_block + n_pred * num_expert) * 4 > (size_t)hidden * 2)
    return fail(PM_ERR_INVALID, "ep_pack: the header (counts and predictor scores) does not fit one row");
  if (!x || !counts || !offsets || !row_token || !pos || !bounds_dev || !send || !pos_reply || (n_pred > 0 && !scores))
    return fail(PM_ERR_INVALID, "ep_pack: null pointer");
  const int ctas_per_seg = cap < 16 ? (cap < 1 ? 1 : cap) : 16;
  ep_pack_kernel<<<dim3(n_ranks, ctas_per_seg), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)x, hidden * 2 / 16, counts, offsets, row_token, pos, n_pairs, bounds_dev, n_ranks, max_block, cap,
      scores, n_pred, num_expert, (uint4*)send, pos_reply);
  PM_CUDA(cudaGetLastError());
  return PM_OK;
}

int pm_k_ep_unpack(const void* recv, int hidden, int n_ranks, int n_local, int max_block, int cap, int n_pred,
                   int num_expert, int32_t* row_expert, float* scores_sum, int32_t* err_flag, void* stream) {
  if (hidden <= 0 || hidden % 8 != 0 || n_ranks <= 0 || n_ranks > kMaxRanks || n_local <= 0 || n_local > max_block ||
      max_block > 256 || cap < 0 || n_pred < 0 || num_expert < n_local ||
      (size_t)(max_block + n_pred * num_expert) * 4 > (size_t)hidden * 2)
    return fail(PM_ERR_INVALID, "ep_unpack: bad sizes");
  if (!recv || !row_expert || (n_pred > 0 && !scores_sum)) return fail(PM_ERR_INVALID, "ep_unpack: null pointer");
  ep_unpack_kernel<<<1, 256, 0, (cudaStream_t)stream>>>((const uint4*)recv, hidden * 2 / 16, n_ranks, n_local,
                                                        max_block, cap, n_pred, num_expert, row_expert, scores_sum,
                                                        err_flag);
  PM_CUDA(cudaGetLastError());
  return PM_OK;
}

}  // extern "C"
