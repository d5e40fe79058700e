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

// hidden[b, j] = relu(W1[j, :] . x[b, :] + b1[j]); one warp per hidden unit j. Up to 8 token rows
// are staged in shared memory per pass, so a unit's weight row is read once per 8 sequences and
// every inner load is a shared-memory read.
constexpr int kFc1Tok = 8;

__global__ void __launch_bounds__(kWarpsPerCta * 32)
predictor_fc1_kernel(const __nv_bfloat16* __restrict__ x, int B, int H,
                     const __nv_bfloat16* __restrict__ w1, const float* __restrict__ b1, int D,
                     float* __restrict__ hidden) {
  extern __shared__ __align__(16) unsigned char fc1_smem[];
  uint4* xs = reinterpret_cast<uint4*>(fc1_smem);  // [kFc1Tok][H / 8]
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const int nvec = H / 8;
  const uint4* wrow = reinterpret_cast<const uint4*>(w1 + (size_t)min(j, D - 1) * H);
  const float bias = (b1 != nullptr && j < D) ? b1[j] : 0.f;
  for (int b0 = 0; b0 < B; b0 += kFc1Tok) {
    const int nb = min(kFc1Tok, B - b0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nb * nvec; idx += blockDim.x)
      xs[idx] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)b0 * H) + idx);
    __syncthreads();
    float acc[kFc1Tok];
#pragma unroll
    for (int bb = 0; bb < kFc1Tok; ++bb) acc[bb] = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 wv = __ldg(wrow + v);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
      for (int bb = 0; bb < kFc1Tok; ++bb) {
        if (bb < nb) {
          const uint4 xv = xs[bb * nvec + v];
          const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 wf = __bfloat1622float2(wp[i]);
            float2 xf = __bfloat1622float2(xp[i]);
            acc[bb] = fmaf(wf.x, xf.x, acc[bb]);
            acc[bb] = fmaf(wf.y, xf.y, acc[bb]);
          }
        }
      }
    }
#pragma unroll
    for (int bb = 0; bb < kFc1Tok; ++bb) {
      float d = acc[bb];
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) d += __shfl_xor_sync(0xffffffffu, d, m);
      if (lane == 0 && bb < nb && j < D) hidden[(size_t)(b0 + bb) * D + j] = fmaxf(d + bias, 0.f);
    }
  }
}

// scores[e] = sum_b sum_j W2[e, j] * hidden[b, j] + B * b2[e]. Every CTA first sums the hidden
// activations over the batch into shared memory, then one warp per expert takes the dot product.
__global__ void __launch_bounds__(kWarpsPerCta * 32)
predictor_fc2_kernel(const float* __restrict__ hidden, int B, int D,
                     const __nv_bfloat16* __restrict__ w2, const float* __restrict__ b2, int E,
                     float* __restrict__ scores) {
  extern __shared__ float hsum[];  // [D]
  for (int j = threadIdx.x; j < D; j += blockDim.x) {
    float s = 0.f;
    for (int b = 0; b < B; ++b) s += hidden[(size_t)b * D + j];
    hsum[j] = s;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (e >= E) return;
  float acc = 0.f;
  for (int j = lane; j < D; j += 32) acc = fmaf(__bfloat162float(w2[(size_t)e * D + j]), hsum[j], acc);
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
  if (lane == 0) scores[e] = acc + (b2 != nullptr ? (float)B * b2[e] : 0.f);
}

// The n best of `width` scores in rank order (descending score, ties to the lower id: what a stable
// descending sort gives, predictor.hpp:24-28 of the reference). One warp: every round each lane
// scans its strided share of the scores that are still in, the warp agrees on the best, lane 0
// writes it and takes it out.
__global__ void __launch_bounds__(32)
rank_topn_kernel(const float* __restrict__ scores, int width, int n, int32_t* __restrict__ out) {
  extern __shared__ float sc[];  // [width] scores, then [width] taken flags as floats' bytes
  unsigned char* taken = reinterpret_cast<unsigned char*>(sc + width);
  const int lane = threadIdx.x;
  for (int i = lane; i < width; i += 32) {
    sc[i] = scores[i];
    taken[i] = 0;
  }
  __syncwarp();
  for (int r = 0; r < n; ++r) {
    float best = 0.f;
    int arg = -1;
    for (int i = lane; i < width; i += 32) {
      if (!taken[i] && (arg < 0 || sc[i] > best)) {  // ascending i: the first of equal scores stays
        best = sc[i];
        arg = i;
      }
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, m);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, m);
      if (oa >= 0 && (arg < 0 || ob > best || (ob == best && oa < arg))) {
        best = ob;
        arg = oa;
      }
    }
    if (lane == 0) {
      out[r] = arg;
      if (arg >= 0) taken[arg] = 1;
    }
    __syncwarp();
  }
}

}  // namespace

cudaError_t launch_rank_topn(const float* scores, int width, int n, int32_t* out, cudaStream_t s) {
  if (n <= 0 || width <= 0) return cudaSuccess;
  if (n > width) n = width;
  const size_t smem = (size_t)width * 5;
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  rank_topn_kernel<<<1, 32, smem, s>>>(scores, width, n, out);
  return cudaGetLastError();
}

cudaError_t launch_predictor_mlp(const __nv_bfloat16* x, int B, int H, const __nv_bfloat16* w1,
                                 const float* b1, int D, const __nv_bfloat16* w2, const float* b2,
                                 int E, float* hidden_scratch, float* scores, cudaStream_t s) {
  if (B <= 0) return cudaSuccess;
  const size_t fc1_smem = (size_t)kFc1Tok * H * 2;
  if (fc1_smem > 48 * 1024) {
    cudaError_t ae = cudaFuncSetAttribute(predictor_fc1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fc1_smem);
    if (ae != cudaSuccess) return ae;
  }
  predictor_fc1_kernel<<<(D + kWarpsPerCta - 1) / kWarpsPerCta, kWarpsPerCta * 32, fc1_smem, s>>>(
      x, B, H, w1, b1, D, hidden_scratch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  predictor_fc2_kernel<<<(E + kWarpsPerCta - 1) / kWarpsPerCta, kWarpsPerCta * 32, (size_t)D * 4, s>>>(
      hidden_scratch, B, D, w2, b2, E, scores);
  return cudaGetLastError();
}

}  // namespace pm
