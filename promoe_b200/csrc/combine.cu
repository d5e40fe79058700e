// K4: weighted combine. For every token gathers the outputs of its k routed
// expert rows in fixed j order, scales them by the routing weights and adds the
// shared-expert rows (optionally scaled by the sigmoid shared gate). A gather
// (not an atomic scatter-add) keeps the sum order fixed, so results are
// reproducible run to run.
//
// It replaces the weighted index_add / shared-expert tail of the MoE block that
// the reference leaves to its patched transformers fork (contract:
// eval/demo-simulate/transformers-deepseek-moe.py:36-49).
#include "pm_common.cuh"

namespace pm {
namespace {

constexpr int kCombineThreads = 256;
constexpr int kMaxTopK = 16;

__global__ void __launch_bounds__(kCombineThreads)
combine_kernel(const float* __restrict__ yexp, const int32_t* __restrict__ pos,
               const float* __restrict__ topk_w, int T, int H, int k, int R, int n_shared,
               const float* __restrict__ shared_scale, __nv_bfloat16* __restrict__ y) {
  const int t = blockIdx.x;
  __shared__ int p_s[kMaxTopK];
  __shared__ float w_s[kMaxTopK];
  if (threadIdx.x < k) {
    p_s[threadIdx.x] = pos[(size_t)t * k + threadIdx.x];
    w_s[threadIdx.x] = topk_w[(size_t)t * k + threadIdx.x];
  }
  __syncthreads();
  const float ss = (shared_scale != nullptr) ? shared_scale[t] : 1.f;
  for (int h = threadIdx.x * 4; h < H; h += kCombineThreads * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; ++j) {
      float4 v = *reinterpret_cast<const float4*>(yexp + (size_t)p_s[j] * H + h);
      float w = w_s[j];
      acc.x = fmaf(w, v.x, acc.x);
      acc.y = fmaf(w, v.y, acc.y);
      acc.z = fmaf(w, v.z, acc.z);
      acc.w = fmaf(w, v.w, acc.w);
    }
    for (int s = 0; s < n_shared; ++s) {
      // Shared-expert rows follow the R routed rows: row R + s*T + t.
      float4 v = *reinterpret_cast<const float4*>(yexp + ((size_t)R + (size_t)s * T + t) * H + h);
      acc.x = fmaf(ss, v.x, acc.x);
      acc.y = fmaf(ss, v.y, acc.y);
      acc.z = fmaf(ss, v.z, acc.z);
      acc.w = fmaf(ss, v.w, acc.w);
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 out;
    out.x = *reinterpret_cast<uint32_t*>(&lo);
    out.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(y + (size_t)t * H + h) = out;
  }
}

}  // namespace

cudaError_t launch_combine(const float* yexp, const int32_t* pos, const float* topk_w, int T, int H,
                           int k, int R, int n_shared, const float* shared_scale,
                           __nv_bfloat16* y, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (k > kMaxTopK) return cudaErrorInvalidValue;
  combine_kernel<<<T, kCombineThreads, 0, s>>>(yexp, pos, topk_w, T, H, k, R, n_shared, shared_scale, y);
  return cudaGetLastError();
}

}  // namespace pm
