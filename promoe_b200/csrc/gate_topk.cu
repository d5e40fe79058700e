// K1: router. One CTA per token computes the gate logits of every expert, selects
// the top-k experts, turns the selection into combine weights and looks the
// selected experts up in the layer's expert -> cache-slot table.
//
// This replaces the first half of the MoE block forward that the reference
// delegates to its patched transformers fork (gate linear -> softmax -> top-k ->
// optional renormalisation; contract: src/sparse_llm_cache/utils/__init__.py:82-89,
// eval/demo-simulate/transformers-deepseek-moe.py:36-49).
//
// Selection is done on the logits (softmax is monotonic), ties go to the lower
// expert id, and the dot product uses a fixed summation order so that a host
// restatement in float32 reproduces the logits bit for bit:
//   lane j of a warp accumulates the 8-element vectors v with v % 32 == j in
//   ascending v, elements 0..7 in order, acc = acc + w*x (the product of two
//   bf16 values is exact in float32, so fused and unfused multiply-add agree);
//   lanes are then combined by a butterfly over lane ^ 16, 8, 4, 2, 1.
#include "pm_common.cuh"

namespace pm {
namespace {

constexpr int kGateThreads = 512;
constexpr int kMaxExperts = 256;

// Logits of one expert row for TOK tokens at once: the weight vectors are fetched once (four at a
// time, for memory-level parallelism) and applied to every token's staged row. Each (token,
// expert) sum still runs over ascending v inside a lane, so the documented order is unchanged.
template <int TOK>
__device__ __forceinline__ void canonical_dot(const uint4* __restrict__ w, const uint4* xs, int nvec, int lane,
                                              float (&out)[TOK]) {
#pragma unroll
  for (int tt = 0; tt < TOK; ++tt) out[tt] = 0.f;
  for (int v0 = lane; v0 < nvec; v0 += 128) {
    uint4 wv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (v0 + 32 * u < nvec) wv[u] = __ldg(w + v0 + 32 * u);
#pragma unroll
    for (int tt = 0; tt < TOK; ++tt) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (v0 + 32 * u < nvec) {
          uint4 xv = xs[(size_t)tt * nvec + v0 + 32 * u];
          const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv[u]);
          const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 wf = __bfloat1622float2(wp[i]);
            float2 xf = __bfloat1622float2(xp[i]);
            out[tt] = __fmaf_rn(wf.x, xf.x, out[tt]);
            out[tt] = __fmaf_rn(wf.y, xf.y, out[tt]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int tt = 0; tt < TOK; ++tt)
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) out[tt] += __shfl_xor_sync(0xffffffffu, out[tt], m);
}

// TOK tokens per CTA: 1 for decode batches (most CTAs in flight), 8 for prefill batches (the
// router matrix is then read from L2 once per 8 tokens instead of once per token).
template <int TOK>
__global__ void __launch_bounds__(kGateThreads)
gate_topk_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w_gate,
                 const float* __restrict__ bias, const __nv_bfloat16* __restrict__ w_shared_gate,
                 int T, int H, int E, int k, int norm_topk, float routed_scale,
                 const int32_t* __restrict__ expert_slot, int32_t* __restrict__ topk_ids,
                 float* __restrict__ topk_w, int32_t* __restrict__ topk_slot,
                 float* __restrict__ shared_scale, float* __restrict__ logits_out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* xs = reinterpret_cast<uint4*>(smem_raw);                       // TOK rows of H bf16
  float* logit_all = reinterpret_cast<float*>(xs + (size_t)TOK * (H / 8));  // TOK x (E + 1)

  const int t0 = blockIdx.x * TOK;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarp = kGateThreads / 32;
  const int nvec = H / 8;
  const int n_tok = min(TOK, T - t0);

  for (int idx = threadIdx.x; idx < TOK * nvec; idx += kGateThreads) {
    const int tt = idx / nvec, v = idx - tt * nvec;
    xs[idx] = (tt < n_tok) ? __ldg(reinterpret_cast<const uint4*>(x + (size_t)(t0 + tt) * H) + v) : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();

  const int n_rows = E + (w_shared_gate != nullptr ? 1 : 0);
  for (int e = warp; e < n_rows; e += nwarp) {
    const uint4* wrow = (e < E) ? reinterpret_cast<const uint4*>(w_gate + (size_t)e * H)
                                : reinterpret_cast<const uint4*>(w_shared_gate);
    float d[TOK];
    canonical_dot<TOK>(wrow, xs, nvec, lane, d);
    if (lane == 0) {
      const float bv = (e < E && bias != nullptr) ? bias[e] : 0.f;
#pragma unroll
      for (int tt = 0; tt < TOK; ++tt) logit_all[tt * (E + 1) + e] = (e < E && bias != nullptr) ? d[tt] + bv : d[tt];
    }
  }
  __syncthreads();

  if (warp >= n_tok) return;  // warp tt finishes token t0 + tt
  const int t = t0 + warp;
  const float* logit_s = logit_all + warp * (E + 1);

  if (logits_out != nullptr)
    for (int e = lane; e < E; e += 32) logits_out[(size_t)t * E + e] = logit_s[e];
  if (w_shared_gate != nullptr && lane == 0 && shared_scale != nullptr)
    shared_scale[t] = 1.f / (1.f + __expf(-logit_s[E]));

  // Each lane owns experts lane, lane+32, ...
  constexpr int kPerLane = kMaxExperts / 32;
  float v[kPerLane];
  float vmax = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    int e = lane + 32 * i;
    v[i] = (e < E) ? logit_s[e] : -INFINITY;
    vmax = fmaxf(vmax, v[i]);
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, m));
  float denom = 0.f;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i)
    if (lane + 32 * i < E) denom += __expf(v[i] - vmax);
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, m);

  float sel_p = 0.f;   // lane j keeps the probability of the j-th selected expert
  int sel_e = -1;
  float sel_sum = 0.f;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      int e = lane + 32 * i;
      if (e < E && (v[i] > best)) {  // ascending e per lane: strict > keeps the lower id on ties
        best = v[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, m);
      int oe = __shfl_xor_sync(0xffffffffu, best_e, m);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    float p = __expf(best - vmax) / denom;
    sel_sum += p;
    if (lane == j) {
      sel_p = p;
      sel_e = best_e;
    }
#pragma unroll
    for (int i = 0; i < kPerLane; ++i)
      if (lane + 32 * i == best_e) v[i] = -INFINITY;
  }
  if (lane < k) {
    float w = sel_p;
    if (norm_topk) w = w / (sel_sum + 1e-20f);
    w *= routed_scale;
    topk_ids[(size_t)t * k + lane] = sel_e;
    topk_w[(size_t)t * k + lane] = w;
    if (topk_slot != nullptr)
      topk_slot[(size_t)t * k + lane] = (expert_slot != nullptr) ? expert_slot[sel_e] : -1;
  }
}

template <int TOK>
cudaError_t launch_gate(const __nv_bfloat16* x, const __nv_bfloat16* w_gate, const float* bias,
                        const __nv_bfloat16* w_shared_gate, int T, int H, int E, int k, int norm_topk,
                        float routed_scale, const int32_t* expert_slot, int32_t* topk_ids, float* topk_w,
                        int32_t* topk_slot, float* shared_scale, float* logits_out, cudaStream_t s) {
  const size_t smem = (size_t)TOK * H * 2 + (size_t)TOK * (E + 1) * 4;
  auto kern = gate_topk_kernel<TOK>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  kern<<<(T + TOK - 1) / TOK, kGateThreads, smem, s>>>(x, w_gate, bias, w_shared_gate, T, H, E, k, norm_topk,
                                                       routed_scale, expert_slot, topk_ids, topk_w, topk_slot,
                                                       shared_scale, logits_out);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gate_topk(const __nv_bfloat16* x, const __nv_bfloat16* w_gate, const float* bias,
                             const __nv_bfloat16* w_shared_gate, int T, int H, int E, int k, int norm_topk,
                             float routed_scale, const int32_t* expert_slot, int32_t* topk_ids, float* topk_w,
                             int32_t* topk_slot, float* shared_scale, float* logits_out, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (T >= 256 && (size_t)8 * H * 2 <= 160 * 1024)
    return launch_gate<8>(x, w_gate, bias, w_shared_gate, T, H, E, k, norm_topk, routed_scale, expert_slot, topk_ids,
                          topk_w, topk_slot, shared_scale, logits_out, s);
  return launch_gate<1>(x, w_gate, bias, w_shared_gate, T, H, E, k, norm_topk, routed_scale, expert_slot, topk_ids,
                        topk_w, topk_slot, shared_scale, logits_out, s);
}

}  // namespace pm
