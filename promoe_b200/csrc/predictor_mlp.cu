// K5: next-layer expert predictor, an MLP hidden -> d -> num_expert with ReLU,
// evaluated for every sequence of the batch and summed over the batch:
//   scores[e] = sum_b ( W2 . relu(W1 . x_b + b1) + b2 )[e]
//
// The reference runs a TorchScript module on the CPU in fp32 after a device-to-host
// copy of the hidden states and sums the output over the batch
// (src/cpp_worker/predictor.cpp:558-607, :638-683); here the hidden states never
// leave the GPU and only the num_expert scores go back to the host for ranking.
#include "pm_common.cuh"

namespace pm {
namespace {

constexpr int kWarpsPerCta = 8;

__device__ __forceinline__ float dot_bf16_row(const uint4* __restrict__ w, const uint4* __restrict__ x,
                                              int nvec, int lane) {
  float acc = 0.f;
  for (int v = lane; v < nvec; v += 32) {
    uint4 wv = __ldg(w + v);
    uint4 xv = __ldg(x + v);
    const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 wf = __bfloat1622float2(wp[i]);
      float2 xf = __bfloat1622float2(xp[i]);
      acc = fmaf(wf.x, xf.x, acc);
      acc = fmaf(wf.y, xf.y, acc);
    }
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
  return acc;
}

// hidden[b, j] = relu(W1[j, :] . x[b, :] + b1[j]); one warp per hidden unit j.
__global__ void __launch_bounds__(kWarpsPerCta * 32)
predictor_fc1_kernel(const __nv_bfloat16* __restrict__ x, int B, int H,
                     const __nv_bfloat16* __restrict__ w1, const float* __restrict__ b1, int D,
                     float* __restrict__ hidden) {
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (j >= D) return;
  const uint4* wrow = reinterpret_cast<const uint4*>(w1 + (size_t)j * H);
  const float bias = (b1 != nullptr) ? b1[j] : 0.f;
  for (int b = 0; b < B; ++b) {
    float d = dot_bf16_row(wrow, reinterpret_cast<const uint4*>(x + (size_t)b * H), H / 8, lane);
    if (lane == 0) hidden[(size_t)b * D + j] = fmaxf(d + bias, 0.f);
  }
}

// scores[e] = sum_b sum_j W2[e, j] * hidden[b, j] + B * b2[e]; one warp per expert.
__global__ void __launch_bounds__(kWarpsPerCta * 32)
predictor_fc2_kernel(const float* __restrict__ hidden, int B, int D,
                     const __nv_bfloat16* __restrict__ w2, const float* __restrict__ b2, int E,
                     float* __restrict__ scores) {
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (e >= E) return;
  float acc = 0.f;
  for (int j = lane; j < D; j += 32) {
    float hs = 0.f;
    for (int b = 0; b < B; ++b) hs += hidden[(size_t)b * D + j];
    acc = fmaf(__bfloat162float(w2[(size_t)e * D + j]), hs, acc);
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
  if (lane == 0) scores[e] = acc + (b2 != nullptr ? (float)B * b2[e] : 0.f);
}

}  // namespace

cudaError_t launch_predictor_mlp(const __nv_bfloat16* x, int B, int H, const __nv_bfloat16* w1,
                                 const float* b1, int D, const __nv_bfloat16* w2, const float* b2,
                                 int E, float* hidden_scratch, float* scores, cudaStream_t s) {
  if (B <= 0) return cudaSuccess;
  predictor_fc1_kernel<<<(D + kWarpsPerCta - 1) / kWarpsPerCta, kWarpsPerCta * 32, 0, s>>>(
      x, B, H, w1, b1, D, hidden_scratch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  predictor_fc2_kernel<<<(E + kWarpsPerCta - 1) / kWarpsPerCta, kWarpsPerCta * 32, 0, s>>>(
      hidden_scratch, B, D, w2, b2, E, scores);
  return cudaGetLastError();
}

}  // namespace pm
