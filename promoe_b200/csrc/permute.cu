// K2: token permutation. Turns the [T, k] routing table into per-expert
// contiguous row ranges: counts[E], offsets[E+1], row_token[R] (the token each
// permuted row reads) and pos[R] (where routed pair (t, j) landed). The order
// inside one expert is ascending in t*k + j, so the result is deterministic.
//
// The reference has no such step: its patched MoE block loops over experts in
// Python and indexes the hidden states per expert (contract:
// eval/demo-simulate/transformers-deepseek-moe.py:41-48). counts[] is also what
// the host reads back to form the unique expert list it reports to the cache
// (src/cpp_worker/prefetcher.cpp:188-202).
#include "pm_common.cuh"

namespace pm {
namespace {

constexpr int kPermThreads = 1024;
constexpr int kMaxExperts = 256;

__global__ void __launch_bounds__(kPermThreads)
permute_kernel(const int32_t* __restrict__ topk_ids, int R, int k, int E, int32_t* __restrict__ counts,
               int32_t* __restrict__ offsets, int32_t* __restrict__ row_token,
               int32_t* __restrict__ pos, int32_t* __restrict__ err_flag, int tail_rows, int T,
               int32_t* __restrict__ zero_words, int zero_n) {
  __shared__ int cnt[kMaxExperts];
  __shared__ int off[kMaxExperts + 1];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  for (int e = tid; e < E; e += kPermThreads) cnt[e] = 0;
  for (int i = tid; i < zero_n; i += kPermThreads) zero_words[i] = 0;
  // Rows after the R routed ones belong to the shared experts: every token once per shared expert.
  for (int i = tid; i < tail_rows; i += kPermThreads) row_token[R + i] = i % T;
  __syncthreads();
  for (int i = tid; i < R; i += kPermThreads) {
    int e = topk_ids[i];
    if (e >= 0 && e < E) {
      atomicAdd(&cnt[e], 1);
    } else {  // -1 = padding, dropped silently; any other id outside [0, E) is dropped and flagged.
      pos[i] = -1;  // either way the position must not keep an old value
      if (e != -1 && err_flag != nullptr) atomicExch(err_flag, 1);
    }
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      run += cnt[e];
    }
    off[E] = run;
  }
  __syncthreads();
  for (int e = tid; e < E; e += kPermThreads) counts[e] = cnt[e];
  for (int e = tid; e <= E; e += kPermThreads) offsets[e] = off[e];

  // Stable placement: warp w places experts w, w+32, ... by scanning the pairs in order.
  const unsigned lt_mask = (1u << lane) - 1u;
  for (int e = warp; e < E; e += kPermThreads / 32) {
    if (cnt[e] == 0) continue;
    int base = off[e];
    for (int c = 0; c < R; c += 32) {
      int i = c + lane;
      int id = (i < R) ? topk_ids[i] : -1;
      unsigned m = __ballot_sync(0xffffffffu, id == e);
      if (id == e) {
        int p = base + __popc(m & lt_mask);
        row_token[p] = i / k;
        pos[i] = p;
      }
      base += __popc(m);
    }
  }
}

// ---- multi-CTA variant for prefill-size batches: same result, three short launches ---------------
// Pairs are cut into chunks of kChunk; chunk c counts its pairs per expert, a scan turns the
// counts into each chunk's first position per expert, and every chunk places its own pairs in
// order. Chunks are ordered, so the placement stays ascending in t*k + j inside an expert.
constexpr int kChunk = 4096;

__global__ void __launch_bounds__(256)
permute_count_kernel(const int32_t* __restrict__ topk_ids, int R, int E, int32_t* __restrict__ chunk_cnt,
                     int32_t* __restrict__ err_flag, int32_t* __restrict__ pos) {
  __shared__ int cnt[kMaxExperts];
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  const int c0 = blockIdx.x * kChunk, c1 = min(R, c0 + kChunk);
  for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e >= 0 && e < E) {
      atomicAdd(&cnt[e], 1);
    } else {
      pos[i] = -1;
      if (e != -1 && err_flag != nullptr) atomicExch(err_flag, 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) chunk_cnt[(size_t)blockIdx.x * E + e] = cnt[e];
}

// One CTA: counts[e], offsets[e], and chunk_cnt[c][e] := first position of chunk c's pairs of expert e.
__global__ void __launch_bounds__(256)
permute_scan_kernel(int32_t* __restrict__ chunk_cnt, int n_chunks, int E, int32_t* __restrict__ counts,
                    int32_t* __restrict__ offsets, int32_t* __restrict__ row_token, int R, int tail_rows, int T) {
  __shared__ int tot[kMaxExperts];
  __shared__ int off[kMaxExperts + 1];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int s = 0;
    for (int c = 0; c < n_chunks; ++c) s += chunk_cnt[(size_t)c * E + e];
    tot[e] = s;
  }
  for (int i = threadIdx.x; i < tail_rows; i += blockDim.x) row_token[R + i] = i % T;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      run += tot[e];
    }
    off[E] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    counts[e] = tot[e];
    int run = off[e];
    for (int c = 0; c < n_chunks; ++c) {
      const int n = chunk_cnt[(size_t)c * E + e];
      chunk_cnt[(size_t)c * E + e] = run;
      run += n;
    }
  }
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
}

__global__ void __launch_bounds__(1024)
permute_place_kernel(const int32_t* __restrict__ topk_ids, int R, int k, int E,
                     const int32_t* __restrict__ chunk_base, int32_t* __restrict__ row_token,
                     int32_t* __restrict__ pos) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned lt_mask = (1u << lane) - 1u;
  const int c0 = blockIdx.x * kChunk, c1 = min(R, c0 + kChunk);
  for (int e = warp; e < E; e += 32) {
    int base = chunk_base[(size_t)blockIdx.x * E + e];
    for (int c = c0; c < c1; c += 32) {
      const int i = c + lane;
      const int id = (i < c1) ? topk_ids[i] : -1;
      const unsigned m = __ballot_sync(0xffffffffu, id == e);
      if (id == e) {
        const int p = base + __popc(m & lt_mask);
        row_token[p] = i / k;
        pos[i] = p;
      }
      base += __popc(m);
    }
  }
}

// dst row r = src row index[r]; rows are row_vec 16-byte vectors long. A negative index (a pair the
// permutation dropped) yields a row of zeros.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ index, int n_rows, int row_vec,
                   uint4* __restrict__ dst) {
  for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
    const int from = index[r];
    const uint4* s = src + (size_t)(from < 0 ? 0 : from) * row_vec;
    uint4* d = dst + (size_t)r * row_vec;
    for (int v = threadIdx.x; v < row_vec; v += blockDim.x) d[v] = from < 0 ? make_uint4(0, 0, 0, 0) : s[v];
  }
}

}  // namespace

cudaError_t launch_gather_rows(const void* src, const int32_t* index, int n_rows, size_t row_bytes, void* dst,
                               cudaStream_t s) {
  if (n_rows <= 0) return cudaSuccess;
  const int grid = n_rows < 1184 ? n_rows : 1184;  // 8 x 148 SMs
  gather_rows_kernel<<<grid, 256, 0, s>>>((const uint4*)src, index, n_rows, (int)(row_bytes / 16), (uint4*)dst);
  return cudaGetLastError();
}

cudaError_t launch_permute(const int32_t* topk_ids, int R, int k, int E, int32_t* counts,
                           int32_t* offsets, int32_t* row_token, int32_t* pos, int32_t* err_flag,
                           int tail_rows, int T, cudaStream_t s, int32_t* scratch, size_t scratch_ints,
                           int32_t* zero_words, int zero_n) {
  const int n_chunks = (R + kChunk - 1) / kChunk;
  if (zero_words == nullptr) zero_n = 0;
  if (R > 2 * kChunk && scratch != nullptr && scratch_ints >= (size_t)n_chunks * E) {
    permute_count_kernel<<<n_chunks, 256, 0, s>>>(topk_ids, R, E, scratch, err_flag, pos);
    permute_scan_kernel<<<1, 256, 0, s>>>(scratch, n_chunks, E, counts, offsets, row_token, R, tail_rows, T > 0 ? T : 1);
    permute_place_kernel<<<n_chunks, 1024, 0, s>>>(topk_ids, R, k, E, scratch, row_token, pos);
    if (zero_n > 0) {
      cudaError_t e = cudaMemsetAsync(zero_words, 0, (size_t)zero_n * 4, s);
      if (e != cudaSuccess) return e;
    }
    return cudaGetLastError();
  }
  permute_kernel<<<1, kPermThreads, 0, s>>>(topk_ids, R, k, E, counts, offsets, row_token, pos, err_flag,
                                            tail_rows, T > 0 ? T : 1, zero_words, zero_n);
  return cudaGetLastError();
}

}  // namespace pm
