// K3a: grouped SwiGLU expert FFN for decode-size batches, weights read by cache-slot
// indirection. Two launches per layer:
//   gate/up : h[r, i] = silu(x_r . Wg[i, :]) * (x_r . Wu[i, :])
//   down    : y[r, n] = h_r . Wd[n, :]
// Every CTA tile streams 64 weight rows (4 warps x 16 rows) exactly once from HBM
// and applies them to all token rows of its chunk (up to 64) with warp-level
// bf16 MMAs, fp32 accumulation. The kernel is HBM-bound: the weight bytes of each
// activated expert are the algorithmic traffic.
//
// It replaces the per-expert Python loop over torch linears that the reference
// drives through ExpertHook (src/sparse_llm_cache/utils/hooks.py:187-198) after
// report_experts (src/sparse_llm_cache/utils/__init__.py:82-89); the weights it
// reads are the cache lines the reference re-points module parameters to
// (src/sparse_llm_cache/utils/__init__.py:58-69).
//
// Operand layout trick: a dot product does not care about the order of k, so each
// lane loads 16 contiguous bytes (8 bf16) of a weight row and of a token row at
// the same k offset and feeds pairs {0,1} and {2,3} to one m16n8k16 MMA and pairs
// {4,5}, {6,7} to a second one. Both operands therefore use full 128-bit loads.
#include <cooperative_groups.h>

#include <cstdlib>

#include "pm_common.cuh"

namespace pm {
namespace {

constexpr int kThreads = 128;
constexpr int kPadElems = 32;  // 64 B of padding per staged token row: conflict-free 128-bit reads
constexpr int kDepth = 4;      // k-steps of weight loads issued back to back per lane

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float silu(float v) { return v / (1.f + __expf(-v)); }

// NT = number of 8-row n-tiles of tokens a chunk may hold (rows <= 8*NT).
// NMAT = 2 for the gate/up pass (two weight streams, SwiGLU epilogue), 1 for down.
template <int NT, int NMAT>
__global__ void __launch_bounds__(kThreads)
grouped_ffn_kernel(const GroupDesc* __restrict__ groups, const int32_t* __restrict__ tile_group,
                   const __nv_bfloat16* __restrict__ bsrc, int ldb,
                   const int32_t* __restrict__ row_token, int hidden, int kc_cap,
                   __nv_bfloat16* __restrict__ hbuf, int ld_h, float* __restrict__ yexp) {
  constexpr bool GATEUP = (NMAT == 2);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* xs = reinterpret_cast<uint4*>(smem_raw);

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int g = lane >> 2;
  const int q = lane & 3;

  const GroupDesc grp = groups[tile_group[blockIdx.x]];
  const int tile_local = blockIdx.x - (GATEUP ? grp.tile_start_gu : grp.tile_start_dn);
  const int K = GATEUP ? hidden : grp.inter;       // reduction length
  const int M = GATEUP ? grp.inter : hidden;       // weight rows
  const int m0 = tile_local * kTileRows + warp * 16;
  const bool active = (m0 + 16 <= M);
  const int rows = grp.row_count;

  const int kc = min(K, kc_cap);
  const int xs_stride = (kc_cap + kPadElems) / 8;  // in uint4

  const unsigned char* a_ptr[NMAT][2];
  {
    const size_t row_bytes = (size_t)K * 2;
    const unsigned char* w0 = reinterpret_cast<const unsigned char*>(GATEUP ? grp.w_gate : grp.w_down);
    const int mr = active ? m0 : 0;
    a_ptr[0][0] = w0 + (size_t)(mr + g) * row_bytes + q * 16;
    a_ptr[0][1] = w0 + (size_t)(mr + g + 8) * row_bytes + q * 16;
    if (GATEUP) {
      const unsigned char* w1 = reinterpret_cast<const unsigned char*>(grp.w_up);
      a_ptr[NMAT - 1][0] = w1 + (size_t)(mr + g) * row_bytes + q * 16;
      a_ptr[NMAT - 1][1] = w1 + (size_t)(mr + g + 8) * row_bytes + q * 16;
    }
  }

  float acc[NMAT][NT][4];
#pragma unroll
  for (int m = 0; m < NMAT; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][nt][i] = 0.f;

  for (int kc0 = 0; kc0 < K; kc0 += kc) {
    const int kc_len = min(kc, K - kc0);
    const int vec_per_row = kc_len / 8;
    __syncthreads();
    // Stage this k-chunk of the chunk's token rows (zero rows beyond row_count).
    for (int idx = threadIdx.x; idx < 8 * NT * vec_per_row; idx += kThreads) {
      int n = idx / vec_per_row;
      int c = idx - n * vec_per_row;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (n < rows) {
        const __nv_bfloat16* src =
            GATEUP ? bsrc + (size_t)row_token[grp.row_start + n] * ldb
                   : bsrc + (size_t)(grp.row_start + n) * ldb;
        v = *reinterpret_cast<const uint4*>(src + kc0 + c * 8);
      }
      xs[n * xs_stride + c] = v;
    }
    __syncthreads();
    if (!active) continue;

    const int steps = kc_len / 32;
    const size_t a_off = (size_t)kc0 * 2;
    for (int s0 = 0; s0 < steps; s0 += kDepth) {
      uint4 a[kDepth][NMAT][2];
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        if (s0 + d < steps) {
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            a[d][m][0] = ldg_stream(a_ptr[m][0] + a_off + (size_t)(s0 + d) * 64);
            a[d][m][1] = ldg_stream(a_ptr[m][1] + a_off + (size_t)(s0 + d) * 64);
          }
        }
      }
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        if (s0 + d < steps) {
          const int kb_vec = (s0 + d) * 4 + q;  // uint4 index inside the staged row
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            uint4 b = xs[(nt * 8 + g) * xs_stride + kb_vec];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
              mma_bf16(acc[m][nt], a[d][m][0].x, a[d][m][1].x, a[d][m][0].y, a[d][m][1].y, b.x, b.y);
              mma_bf16(acc[m][nt], a[d][m][0].z, a[d][m][1].z, a[d][m][0].w, a[d][m][1].w, b.z, b.w);
            }
          }
        }
      }
    }
  }

  if (!active) return;
  // acc[..][nt][0..3] = (row m0+g, token n0), (m0+g, n0+1), (m0+g+8, n0), (m0+g+8, n0+1)
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int n = nt * 8 + 2 * q + (i & 1);
      const int m = m0 + g + ((i & 2) ? 8 : 0);
      if (n < rows) {
        const size_t r = (size_t)(grp.row_start + n);
        if (GATEUP) {
          float h = silu(acc[0][nt][i]) * acc[NMAT - 1][nt][i];
          hbuf[r * ld_h + m] = __float2bfloat16_rn(h);
        } else {
          yexp[r * hidden + m] = acc[0][nt][i];
        }
      }
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Decode variant for chunks of at most 16 token rows (the common case: a handful of tokens per
// expert). A CTA owns one m-tile (16 gate rows + the same 16 up rows, or 32 down rows) and its
// 8 warps split the reduction dimension, so every warp issues its whole share of weight loads
// in one or two batches and a tile lives for a couple of DRAM round trips. Token rows are
// read straight from global memory (they are tiny and stay in L1/L2) into MMA B fragments,
// so there is no shared-memory staging and no barrier before the final cross-warp reduction.
// ---------------------------------------------------------------------------------------------
constexpr int kSplitWarps = 8;
constexpr int kSplitThreads = kSplitWarps * 32;

// Token-row fragment load. Rows written earlier in the same kernel (the fused variant reads the
// intermediate rows other CTAs produced before the grid barrier) must not go through the
// non-coherent path.
template <bool COHERENT>
__device__ __forceinline__ uint4 load_b(const unsigned char* p) {
  uint4 r;
  if (COHERENT) {
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  } else {
    r = __ldg(reinterpret_cast<const uint4*>(p));
  }
  return r;
}

// One split-K tile: 16 gate + 16 up rows (GATEUP) or 32 down rows of one chunk, all 8 warps of
// the CTA. `red` is the CTA's reduction buffer; the caller separates consecutive tiles by a barrier.
template <int NT, bool GATEUP, int DEPTH, bool COHERENT_B>
__device__ __forceinline__ void splitk_tile(const GroupDesc& grp, int tile_local,
                                            const __nv_bfloat16* __restrict__ bsrc, int ldb,
                                            const int32_t* __restrict__ row_token, int hidden,
                                            __nv_bfloat16* __restrict__ hbuf, int ld_h,
                                            float* __restrict__ yexp, float (*red)[2 * NT * 4][32]) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int g = lane >> 2;
  const int q = lane & 3;
  const int K = GATEUP ? hidden : grp.inter;
  const int rows = grp.row_count;
  const int m0 = tile_local * (GATEUP ? 16 : 32);
  const size_t row_bytes = (size_t)K * 2;

  // Four weight-row streams per lane: gate rows g / g+8 and up rows g / g+8, or down rows
  // g, g+8, g+16, g+24 of the tile.
  const unsigned char* a_ptr[4];
  if (GATEUP) {
    const unsigned char* w0 = reinterpret_cast<const unsigned char*>(grp.w_gate);
    const unsigned char* w1 = reinterpret_cast<const unsigned char*>(grp.w_up);
    a_ptr[0] = w0 + (size_t)(m0 + g) * row_bytes + q * 16;
    a_ptr[1] = w0 + (size_t)(m0 + g + 8) * row_bytes + q * 16;
    a_ptr[2] = w1 + (size_t)(m0 + g) * row_bytes + q * 16;
    a_ptr[3] = w1 + (size_t)(m0 + g + 8) * row_bytes + q * 16;
  } else {
    const unsigned char* w0 = reinterpret_cast<const unsigned char*>(grp.w_down);
#pragma unroll
    for (int j = 0; j < 4; ++j) a_ptr[j] = w0 + (size_t)(m0 + g + 8 * j) * row_bytes + q * 16;
  }
  const unsigned char* b_ptr[NT];
  bool b_ok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + g;
    b_ok[nt] = n < rows;
    const int src_row = b_ok[nt] ? (GATEUP ? row_token[grp.row_start + n] : grp.row_start + n) : 0;
    b_ptr[nt] = reinterpret_cast<const unsigned char*>(bsrc + (size_t)src_row * ldb) + q * 16;
  }

  float acc[2][NT][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][nt][i] = 0.f;

  const int steps = K / 32;
  const int s_begin = (warp * steps) / kSplitWarps;
  const int s_end = ((warp + 1) * steps) / kSplitWarps;
  for (int s0 = s_begin; s0 < s_end; s0 += DEPTH) {
    uint4 a[DEPTH][4];
    uint4 b[DEPTH][NT];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      if (s0 + d < s_end) {
        const size_t off = (size_t)(s0 + d) * 64;
#pragma unroll
        for (int j = 0; j < 4; ++j) a[d][j] = ldg_stream(a_ptr[j] + off);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          b[d][nt] = b_ok[nt] ? load_b<COHERENT_B>(b_ptr[nt] + off) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      if (s0 + d < s_end) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            const uint4& lo = a[d][2 * m];
            const uint4& hi = a[d][2 * m + 1];
            mma_bf16(acc[m][nt], lo.x, hi.x, lo.y, hi.y, b[d][nt].x, b[d][nt].y);
            mma_bf16(acc[m][nt], lo.z, hi.z, lo.w, hi.w, b[d][nt].z, b[d][nt].w);
          }
        }
      }
    }
  }

  // Cross-warp reduction of the split-K partial sums, then the epilogue.
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[warp][(m * NT + nt) * 4 + i][lane] = acc[m][nt][i];
  __syncthreads();
  for (int idx = threadIdx.x; idx < NT * 4 * 32; idx += kSplitThreads) {
    const int l = idx & 31;
    const int v = idx >> 5;  // nt * 4 + i
    const int nt = v >> 2, i = v & 3;
    float s0v = 0.f, s1v = 0.f;
#pragma unroll
    for (int w = 0; w < kSplitWarps; ++w) {
      s0v += red[w][v][l];
      s1v += red[w][NT * 4 + v][l];
    }
    const int lg = l >> 2, lq = l & 3;
    const int n = nt * 8 + 2 * lq + (i & 1);
    if (n >= rows) continue;
    const int m = m0 + lg + ((i & 2) ? 8 : 0);
    const size_t r = (size_t)(grp.row_start + n);
    if (GATEUP) {
      hbuf[r * ld_h + m] = __float2bfloat16_rn(silu(s0v) * s1v);
    } else {
      yexp[r * hidden + m] = s0v;
      yexp[r * hidden + m + 16] = s1v;
    }
  }
}


// ---------------------------------------------------------------------------------------------
// uint4 group-128 experts (asymmetric: w = (q - zero) * scale, fp16 scale and zero per 128
// weights of a row). Dequantisation is fused into the load path without touching the weights
// one by one: a 32-bit word holds 8 weights of one row, the even-k nibbles in its low half and
// the odd-k nibbles in its high half, so `((word >> 4j) & 0x000F000F) | 0x43004300` is the bf16
// pair (128 + q[2j], 128 + q[2j+1]) ready to be an MMA A register. One lane load of 16 bytes
// covers 32 weights, the four lanes of a row cover exactly one quantisation group, and per group
//     sum_k (q_k - z) s x_k = s * ( sum_k (128 + q_k) x_k  -  (128 + z) * sum_k x_k ),
// where both sums come out of the tensor core (the second from an all-ones A fragment).
// Layout of the metadata: per matrix an array [rows, K/128] of {scale, zero} fp16 pairs.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t q4_pair(uint32_t word, int j) {
  return ((word >> (4 * j)) & 0x000F000Fu) | 0x43004300u;
}

template <int NT, bool GATEUP, int DEPTH, bool COHERENT_B>
__device__ __forceinline__ void splitk_tile_q4(const GroupDesc& grp, int tile_local,
                                               const __nv_bfloat16* __restrict__ bsrc, int ldb,
                                               const int32_t* __restrict__ row_token, int hidden,
                                               __nv_bfloat16* __restrict__ hbuf, int ld_h,
                                               float* __restrict__ yexp, float (*red)[2 * NT * 4][32]) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int g = lane >> 2;
  const int q = lane & 3;
  const int K = GATEUP ? hidden : grp.inter;
  const int rows = grp.row_count;
  const int m0 = tile_local * (GATEUP ? 16 : 32);
  const size_t row_bytes = (size_t)K / 2;   // packed nibbles
  const int n_grp = K / 128;                // quantisation groups per row = k-steps

  const unsigned char* a_ptr[4];
  const uint32_t* sz_ptr[4];  // {scale, zero} fp16 pairs of the same four rows
  {
    const unsigned char* w0 = reinterpret_cast<const unsigned char*>(GATEUP ? grp.w_gate : grp.w_down);
    const unsigned char* w1 = reinterpret_cast<const unsigned char*>(GATEUP ? grp.w_up : grp.w_down);
    const uint32_t* z0 = reinterpret_cast<const uint32_t*>(GATEUP ? grp.q_gate : grp.q_down);
    const uint32_t* z1 = reinterpret_cast<const uint32_t*>(GATEUP ? grp.q_up : grp.q_down);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = GATEUP ? (m0 + g + 8 * (j & 1)) : (m0 + g + 8 * j);
      const unsigned char* w = (GATEUP && j >= 2) ? w1 : w0;
      const uint32_t* z = (GATEUP && j >= 2) ? z1 : z0;
      a_ptr[j] = w + (size_t)row * row_bytes + q * 16;
      sz_ptr[j] = z + (size_t)row * n_grp;
    }
  }
  const unsigned char* b_ptr[NT];
  bool b_ok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + g;
    b_ok[nt] = n < rows;
    const int src_row = b_ok[nt] ? (GATEUP ? row_token[grp.row_start + n] : grp.row_start + n) : 0;
    b_ptr[nt] = reinterpret_cast<const unsigned char*>(bsrc + (size_t)src_row * ldb) + q * 64;
  }

  float acc[2][NT][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][nt][i] = 0.f;

  const int s_begin = (warp * n_grp) / kSplitWarps;
  const int s_end = ((warp + 1) * n_grp) / kSplitWarps;
  constexpr uint32_t kOnes = 0x3F803F80u;  // bf16 (1, 1)
  for (int s0 = s_begin; s0 < s_end; s0 += DEPTH) {
    uint4 a[DEPTH][4];
    uint32_t sz[DEPTH][4];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      if (s0 + d < s_end) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          a[d][j] = ldg_stream(a_ptr[j] + (size_t)(s0 + d) * 64);
          sz[d][j] = __ldg(sz_ptr[j] + (s0 + d));
        }
      }
    }
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      if (s0 + d < s_end) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          float raw[2][4], xs[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) raw[0][i] = raw[1][i] = xs[i] = 0.f;
          // this lane's 32 token values of the group: four 16-byte vectors
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint4 b = b_ok[nt] ? load_b<COHERENT_B>(b_ptr[nt] + (size_t)(s0 + d) * 256 + v * 16)
                                     : make_uint4(0, 0, 0, 0);
            const uint32_t w00 = (&a[d][0].x)[v], w01 = (&a[d][1].x)[v];  // matrix 0: rows g, g+8
            const uint32_t w10 = (&a[d][2].x)[v], w11 = (&a[d][3].x)[v];  // matrix 1
            mma_bf16(raw[0], q4_pair(w00, 0), q4_pair(w01, 0), q4_pair(w00, 1), q4_pair(w01, 1), b.x, b.y);
            mma_bf16(raw[0], q4_pair(w00, 2), q4_pair(w01, 2), q4_pair(w00, 3), q4_pair(w01, 3), b.z, b.w);
            mma_bf16(raw[1], q4_pair(w10, 0), q4_pair(w11, 0), q4_pair(w10, 1), q4_pair(w11, 1), b.x, b.y);
            mma_bf16(raw[1], q4_pair(w10, 2), q4_pair(w11, 2), q4_pair(w10, 3), q4_pair(w11, 3), b.z, b.w);
            mma_bf16(xs, kOnes, kOnes, kOnes, kOnes, b.x, b.y);
            mma_bf16(xs, kOnes, kOnes, kOnes, kOnes, b.z, b.w);
          }
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&sz[d][2 * m]));      // row g
            const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&sz[d][2 * m + 1]));  // row g+8
            acc[m][nt][0] += lo.x * (raw[m][0] - (128.f + lo.y) * xs[0]);
            acc[m][nt][1] += lo.x * (raw[m][1] - (128.f + lo.y) * xs[1]);
            acc[m][nt][2] += hi.x * (raw[m][2] - (128.f + hi.y) * xs[0]);
            acc[m][nt][3] += hi.x * (raw[m][3] - (128.f + hi.y) * xs[1]);
          }
        }
      }
    }
  }

#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[warp][(m * NT + nt) * 4 + i][lane] = acc[m][nt][i];
  __syncthreads();
  for (int idx = threadIdx.x; idx < NT * 4 * 32; idx += kSplitThreads) {
    const int l = idx & 31;
    const int v = idx >> 5;
    const int nt = v >> 2, i = v & 3;
    float s0v = 0.f, s1v = 0.f;
#pragma unroll
    for (int w = 0; w < kSplitWarps; ++w) {
      s0v += red[w][v][l];
      s1v += red[w][NT * 4 + v][l];
    }
    const int lg = l >> 2, lq = l & 3;
    const int n = nt * 8 + 2 * lq + (i & 1);
    if (n >= rows) continue;
    const int m = m0 + lg + ((i & 2) ? 8 : 0);
    const size_t r = (size_t)(grp.row_start + n);
    if (GATEUP) {
      hbuf[r * ld_h + m] = __float2bfloat16_rn(silu(s0v) * s1v);
    } else {
      yexp[r * hidden + m] = s0v;
      yexp[r * hidden + m + 16] = s1v;
    }
  }
}

template <int NT, int NMAT, int DEPTH>
__global__ void __launch_bounds__(kSplitThreads, 2)
grouped_ffn_q4_kernel(const GroupDesc* __restrict__ groups, const int32_t* __restrict__ tile_group,
                      const __nv_bfloat16* __restrict__ bsrc, int ldb,
                      const int32_t* __restrict__ row_token, int hidden,
                      __nv_bfloat16* __restrict__ hbuf, int ld_h, float* __restrict__ yexp) {
  constexpr bool GATEUP = (NMAT == 2);
  __shared__ float red[kSplitWarps][2 * NT * 4][32];
  const GroupDesc grp = groups[tile_group[blockIdx.x]];
  const int tile_local = blockIdx.x - (GATEUP ? grp.tile_start_gu : grp.tile_start_dn);
  splitk_tile_q4<NT, GATEUP, DEPTH, false>(grp, tile_local, bsrc, ldb, row_token, hidden, hbuf, ld_h, yexp, red);
}

template <int NT, int NMAT>
cudaError_t launch_q4(const GroupDesc* groups, const int32_t* tile_group, int tiles, const __nv_bfloat16* bsrc,
                      int ldb, const int32_t* row_token, int hidden, __nv_bfloat16* hbuf, int ld_h, float* yexp,
                      cudaStream_t s) {
  grouped_ffn_q4_kernel<NT, NMAT, 2><<<tiles, kSplitThreads, 0, s>>>(groups, tile_group, bsrc, ldb, row_token,
                                                                     hidden, hbuf, ld_h, yexp);
  return cudaGetLastError();
}

template <int NT, int NMAT, int DEPTH>
__global__ void __launch_bounds__(kSplitThreads, 2)
grouped_ffn_splitk_kernel(const GroupDesc* __restrict__ groups, const int32_t* __restrict__ tile_group,
                          const __nv_bfloat16* __restrict__ bsrc, int ldb,
                          const int32_t* __restrict__ row_token, int hidden,
                          __nv_bfloat16* __restrict__ hbuf, int ld_h, float* __restrict__ yexp) {
  constexpr bool GATEUP = (NMAT == 2);
  __shared__ float red[kSplitWarps][2 * NT * 4][32];
  const GroupDesc grp = groups[tile_group[blockIdx.x]];
  const int tile_local = blockIdx.x - (GATEUP ? grp.tile_start_gu : grp.tile_start_dn);
  splitk_tile<NT, GATEUP, DEPTH, false>(grp, tile_local, bsrc, ldb, row_token, hidden, hbuf, ld_h, yexp, red);
}

// ---------------------------------------------------------------------------------------------
// Fused decode variant: ONE cooperative launch per segment. A fixed grid of resident CTAs strides
// over the gate/up tiles, meets at a grid barrier (the intermediate rows must be complete before
// any down tile reads them), then strides over the down tiles. Compared with two launches this
// removes one launch gap and one tail per segment.
// ---------------------------------------------------------------------------------------------
// The same split-K tile cut into stages, so that a resident CTA can have the first loads of its
// NEXT tile in flight while it reduces and stores the current one.
template <int NT>
struct TileCtx {
  const unsigned char* a_ptr[4];
  const unsigned char* b_ptr[NT];
  bool b_ok[NT];
  int rows, m0, row_start, s_begin, s_end;  // s_* count this warp's k-steps: 0 .. s_end
  int step_bytes;                            // distance between two of them
};

// What a tile needs from its chunk descriptor and the row table. It is fetched one tile ahead, so
// that the two dependent loads (descriptor, then token row numbers) never stall the load stream.
template <int NT>
struct TileMeta {
  const unsigned char* w0;
  const unsigned char* w1;
  int row_start, rows, inter, tile_start;
  int src_row[NT];
};

template <int NT, bool GATEUP>
__device__ __forceinline__ void meta_load_desc(TileMeta<NT>& m, const GroupDesc* __restrict__ groups, int gi) {
  const GroupDesc* d = groups + gi;
  m.w0 = reinterpret_cast<const unsigned char*>(GATEUP ? d->w_gate : d->w_down);
  m.w1 = reinterpret_cast<const unsigned char*>(GATEUP ? d->w_up : d->w_down);
  m.row_start = d->row_start;
  m.rows = d->row_count;
  m.inter = d->inter;
  m.tile_start = GATEUP ? d->tile_start_gu : d->tile_start_dn;
}

template <int NT, bool GATEUP>
__device__ __forceinline__ void meta_load_rows(TileMeta<NT>& m, const int32_t* __restrict__ row_token) {
  const int g = (threadIdx.x & 31) >> 2;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + g;
    m.src_row[nt] = (n < m.rows) ? (GATEUP ? row_token[m.row_start + n] : m.row_start + n) : -1;
  }
}

template <int NT, bool GATEUP, int WARPS>
__device__ __forceinline__ void tile_setup(TileCtx<NT>& t, const TileMeta<NT>& m, int tile,
                                           const __nv_bfloat16* bsrc, int ldb, int hidden) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, q = lane & 3;
  const int tile_local = tile - m.tile_start;
  const int K = GATEUP ? hidden : m.inter;
  const size_t row_bytes = (size_t)K * 2;
  t.rows = m.rows;
  t.row_start = m.row_start;
  t.m0 = tile_local * (GATEUP ? 16 : 32);
  // Every warp takes a contiguous range of k-steps (interleaving them across warps, w, w+8, ...,
  // measured 6 % slower: longer contiguous runs per warp suit DRAM better).
  const int steps = K / 32;
  const int first = (warp * steps) / WARPS;
  t.s_end = ((warp + 1) * steps) / WARPS - first;
  t.s_begin = 0;
  t.step_bytes = 64;
  const size_t col = (size_t)first * 64 + q * 16;
  if (GATEUP) {
    t.a_ptr[0] = m.w0 + (size_t)(t.m0 + g) * row_bytes + col;
    t.a_ptr[1] = m.w0 + (size_t)(t.m0 + g + 8) * row_bytes + col;
    t.a_ptr[2] = m.w1 + (size_t)(t.m0 + g) * row_bytes + col;
    t.a_ptr[3] = m.w1 + (size_t)(t.m0 + g + 8) * row_bytes + col;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) t.a_ptr[j] = m.w0 + (size_t)(t.m0 + g + 8 * j) * row_bytes + col;
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    t.b_ok[nt] = m.src_row[nt] >= 0;
    t.b_ptr[nt] = reinterpret_cast<const unsigned char*>(bsrc + (size_t)max(m.src_row[nt], 0) * ldb) + col;
  }
}

template <int NT, int DEPTH, bool COHERENT_B>
__device__ __forceinline__ void tile_issue(const TileCtx<NT>& t, int s0, uint4 (&a)[DEPTH][4], uint4 (&b)[DEPTH][NT]) {
#pragma unroll
  for (int d = 0; d < DEPTH; ++d) {
    if (s0 + d < t.s_end) {
      const size_t off = (size_t)(s0 + d) * t.step_bytes;
#pragma unroll
      for (int j = 0; j < 4; ++j) a[d][j] = ldg_stream(t.a_ptr[j] + off);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        b[d][nt] = t.b_ok[nt] ? load_b<COHERENT_B>(t.b_ptr[nt] + off) : make_uint4(0, 0, 0, 0);
    }
  }
}

// First batch of a tile in two halves: the weight loads can go out before the token rows exist.
template <int NT, int DEPTH>
__device__ __forceinline__ void tile_issue_a(const TileCtx<NT>& t, int s0, uint4 (&a)[DEPTH][4]) {
#pragma unroll
  for (int d = 0; d < DEPTH; ++d) {
    if (s0 + d < t.s_end) {
      const size_t off = (size_t)(s0 + d) * t.step_bytes;
#pragma unroll
      for (int j = 0; j < 4; ++j) a[d][j] = ldg_stream(t.a_ptr[j] + off);
    }
  }
}

template <int NT, int DEPTH, bool COHERENT_B>
__device__ __forceinline__ void tile_issue_b(const TileCtx<NT>& t, int s0, uint4 (&b)[DEPTH][NT]) {
#pragma unroll
  for (int d = 0; d < DEPTH; ++d) {
    if (s0 + d < t.s_end) {
      const size_t off = (size_t)(s0 + d) * t.step_bytes;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        b[d][nt] = t.b_ok[nt] ? load_b<COHERENT_B>(t.b_ptr[nt] + off) : make_uint4(0, 0, 0, 0);
    }
  }
}

template <int NT, int DEPTH>
__device__ __forceinline__ void tile_compute(const TileCtx<NT>& t, int s0, const uint4 (&a)[DEPTH][4],
                                             const uint4 (&b)[DEPTH][NT], float (&acc)[2][NT][4]) {
#pragma unroll
  for (int d = 0; d < DEPTH; ++d) {
    if (s0 + d < t.s_end) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const uint4& lo = a[d][2 * m];
          const uint4& hi = a[d][2 * m + 1];
          mma_bf16(acc[m][nt], lo.x, hi.x, lo.y, hi.y, b[d][nt].x, b[d][nt].y);
          mma_bf16(acc[m][nt], lo.z, hi.z, lo.w, hi.w, b[d][nt].z, b[d][nt].w);
        }
      }
    }
  }
}

template <int NT, bool GATEUP, int WARPS>
__device__ __forceinline__ void tile_finish(int rows, int m0, int row_start, float (&acc)[2][NT][4],
                                            float (*red)[2 * NT * 4][32], __nv_bfloat16* __restrict__ hbuf, int ld_h,
                                            float* __restrict__ yexp, int hidden) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        red[warp][(m * NT + nt) * 4 + i][lane] = acc[m][nt][i];
        acc[m][nt][i] = 0.f;
      }
  __syncthreads();
  for (int idx = threadIdx.x; idx < NT * 4 * 32; idx += WARPS * 32) {
    const int l = idx & 31, v = idx >> 5;
    const int nt = v >> 2, i = v & 3;
    float s0v = 0.f, s1v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      s0v += red[w][v][l];
      s1v += red[w][NT * 4 + v][l];
    }
    const int lg = l >> 2, lq = l & 3;
    const int n = nt * 8 + 2 * lq + (i & 1);
    if (n >= rows) continue;
    const int m = m0 + lg + ((i & 2) ? 8 : 0);
    const size_t r = (size_t)(row_start + n);
    if (GATEUP) {
      hbuf[r * ld_h + m] = __float2bfloat16_rn(silu(s0v) * s1v);
    } else {
      yexp[r * hidden + m] = s0v;
      yexp[r * hidden + m + 16] = s1v;
    }
  }
  // no trailing barrier: the caller alternates between two reduction buffers, and the barrier above of
  // the NEXT tile orders this tile's reads before the writes of the tile after it
}

// Tiles blockIdx.x, blockIdx.x + gridDim.x, ... of one phase. The assignment is static, so the
// next tile is known early: its descriptor is fetched one tile ahead and its first batch of loads
// is issued before the current tile is reduced, which keeps DRAM requests in flight across tile
// boundaries. The phase is cut in two calls so that the fused kernel can start the down phase's
// first weight loads (which do not depend on the intermediate rows) BEFORE the grid barrier.
template <int NT, int DEPTH>
struct StreamState {
  TileCtx<NT> t;
  TileMeta<NT> m;
  uint4 a[DEPTH][4];
  uint4 b[DEPTH][NT];
  int tile;
  bool active;
};

// Sets the CTA's first tile up and issues its weight loads. Reads only the plan and the weights.
template <int NT, bool GATEUP, int DEPTH, int WARPS>
__device__ __forceinline__ void stream_begin(StreamState<NT, DEPTH>& st, const GroupDesc* __restrict__ groups,
                                             const int32_t* __restrict__ tile_group, int n_tiles,
                                             const __nv_bfloat16* bsrc, int ldb,
                                             const int32_t* __restrict__ row_token, int hidden) {
  st.tile = blockIdx.x;
  st.active = st.tile < n_tiles;
  if (!st.active) return;
  meta_load_desc<NT, GATEUP>(st.m, groups, tile_group[st.tile]);  // only the first tile pays for these round trips
  meta_load_rows<NT, GATEUP>(st.m, row_token);
  tile_setup<NT, GATEUP, WARPS>(st.t, st.m, st.tile, bsrc, ldb, hidden);
  tile_issue_a<NT, DEPTH>(st.t, st.t.s_begin, st.a);
}

template <int NT, bool GATEUP, int DEPTH, int WARPS>
__device__ __forceinline__ void stream_run(StreamState<NT, DEPTH>& st, const GroupDesc* __restrict__ groups,
                                           const int32_t* __restrict__ tile_group, int n_tiles,
                                           const __nv_bfloat16* bsrc, int ldb,
                                           const int32_t* __restrict__ row_token, int hidden,
                                           __nv_bfloat16* __restrict__ hbuf, int ld_h, float* __restrict__ yexp,
                                           float (*red2)[WARPS][2 * NT * 4][32]) {
  constexpr bool COH = !GATEUP;  // the down phase reads rows other CTAs wrote in this kernel
  if (!st.active) return;
  TileCtx<NT>& t = st.t;
  TileMeta<NT>& m = st.m;
  int buf = 0;
  float acc[2][NT][4];
#pragma unroll
  for (int mm = 0; mm < 2; ++mm)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mm][nt][i] = 0.f;
  tile_issue_b<NT, DEPTH, COH>(t, t.s_begin, st.b);
  const int stride = gridDim.x;
  int tile = st.tile;
  int next = tile + stride;
  int gi_next = (next < n_tiles) ? tile_group[next] : 0;
  while (true) {
    const bool has_next = next < n_tiles;
    if (has_next) meta_load_desc<NT, GATEUP>(m, groups, gi_next);  // arrives while this tile streams
    const int next2 = next + stride;
    const int gi_next2 = (next2 < n_tiles) ? tile_group[next2] : 0;
    bool rows_loaded = false;
    for (int s0 = t.s_begin; s0 < t.s_end;) {
      tile_compute<NT, DEPTH>(t, s0, st.a, st.b, acc);
      if (has_next && !rows_loaded) {  // the descriptor is here by now: fetch the token row numbers
        meta_load_rows<NT, GATEUP>(m, row_token);
        rows_loaded = true;
      }
      s0 += DEPTH;
      if (s0 < t.s_end) tile_issue<NT, DEPTH, COH>(t, s0, st.a, st.b);
    }
    if (has_next && !rows_loaded) meta_load_rows<NT, GATEUP>(m, row_token);
    const int rows = t.rows, m0 = t.m0, row_start = t.row_start;
    if (has_next) {
      tile_setup<NT, GATEUP, WARPS>(t, m, next, bsrc, ldb, hidden);
      tile_issue<NT, DEPTH, COH>(t, t.s_begin, st.a, st.b);
    }
    tile_finish<NT, GATEUP, WARPS>(rows, m0, row_start, acc, red2[buf], hbuf, ld_h, yexp, hidden);
    buf ^= 1;
    if (!has_next) break;
    tile = next;
    next = next2;
    gi_next = gi_next2;
  }
}

template <int NT, int DEPTH, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 16 / WARPS)
grouped_ffn_fused_kernel(const GroupDesc* __restrict__ groups, const int32_t* __restrict__ tile_gu,
                         const int32_t* __restrict__ tile_dn, int tiles_gu, int tiles_dn, int* counters,
                         const __nv_bfloat16* __restrict__ x, int hidden,
                         const int32_t* __restrict__ row_token, __nv_bfloat16* hbuf, int ld_h,
                         float* __restrict__ yexp, const int32_t* __restrict__ dev_tiles) {
  __shared__ float red[2][WARPS][2 * NT * 4][32];  // two reduction buffers, used alternately
  (void)counters;
  if (dev_tiles != nullptr) {  // plan built on the device: the tile counts live there too
    tiles_gu = dev_tiles[0];
    tiles_dn = dev_tiles[1];
  }
  StreamState<NT, DEPTH> st;
  stream_begin<NT, true, DEPTH, WARPS>(st, groups, tile_gu, tiles_gu, x, hidden, row_token, hidden);
  stream_run<NT, true, DEPTH, WARPS>(st, groups, tile_gu, tiles_gu, x, hidden, row_token, hidden, hbuf, ld_h, yexp, red);
  // The first down tile's descriptor and weight loads do not depend on the intermediate rows: they go
  // out before the barrier, so their DRAM latency is hidden behind it.
  stream_begin<NT, false, DEPTH, WARPS>(st, groups, tile_dn, tiles_dn, hbuf, ld_h, row_token, hidden);
  __threadfence();
  cooperative_groups::this_grid().sync();
  stream_run<NT, false, DEPTH, WARPS>(st, groups, tile_dn, tiles_dn, hbuf, ld_h, row_token, hidden, nullptr, ld_h, yexp,
                                      red);
}

// Resident grid of the fused kernel on the current device (0 if cooperative launch is unavailable).
template <int NT, int DEPTH, int WARPS>
int fused_grid_size() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] != 0) return cached[dev] < 0 ? 0 : cached[dev];
  int coop = 0, sms = 0, per_sm = 0;
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (!coop || sms <= 0 ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, grouped_ffn_fused_kernel<NT, DEPTH, WARPS>, WARPS * 32, 0) !=
          cudaSuccess ||
      per_sm <= 0) {
    cached[dev] = -1;
    return 0;
  }
  cached[dev] = sms * per_sm;
  return cached[dev];
}

template <int NT, int DEPTH, int WARPS>
cudaError_t launch_fused_w(const GroupDesc* groups, const int32_t* t_gu, const int32_t* t_dn, int tiles_gu,
                         int tiles_dn, int* counters, const __nv_bfloat16* x, int hidden,
                         const int32_t* row_token, __nv_bfloat16* hbuf, int ld_h, float* yexp, cudaStream_t s,
                         const int32_t* dev_tiles = nullptr) {
  int grid = fused_grid_size<NT, DEPTH, WARPS>();
  if (grid <= 0) return cudaErrorNotSupported;
  if (dev_tiles == nullptr) grid = min(grid, max(tiles_gu, tiles_dn));
  void* args[] = {(void*)&groups, (void*)&t_gu, (void*)&t_dn, (void*)&tiles_gu, (void*)&tiles_dn, (void*)&counters,
                  (void*)&x, (void*)&hidden, (void*)&row_token, (void*)&hbuf, (void*)&ld_h, (void*)&yexp,
                  (void*)&dev_tiles};
  return cudaLaunchCooperativeKernel((const void*)grouped_ffn_fused_kernel<NT, DEPTH, WARPS>, dim3(grid),
                                     dim3(WARPS * 32), args, 0, s);
}

// 8 warps x 2 CTAs per SM. (16 warps x 1 CTA, one batch of loads per tile, measured 28 % slower at
// 60 experts: with a single CTA per SM nothing overlaps the reduction and the barrier.)
constexpr int kFusedWarps = 8;

template <int NT, int DEPTH>
cudaError_t launch_fused(const GroupDesc* groups, const int32_t* t_gu, const int32_t* t_dn, int tiles_gu,
                         int tiles_dn, int* counters, const __nv_bfloat16* x, int hidden,
                         const int32_t* row_token, __nv_bfloat16* hbuf, int ld_h, float* yexp, cudaStream_t s,
                         const int32_t* dev_tiles = nullptr) {
  return launch_fused_w<NT, DEPTH, kFusedWarps>(groups, t_gu, t_dn, tiles_gu, tiles_dn, counters, x, hidden, row_token,
                                                hbuf, ld_h, yexp, s, dev_tiles);
}

template <int NT, int DEPTH>
int fused_grid_size_any() {
  return fused_grid_size<NT, DEPTH, kFusedWarps>();
}

template <int NT, int NMAT>
cudaError_t launch_splitk(const GroupDesc* groups, const int32_t* tile_group, int tiles, const __nv_bfloat16* bsrc, int ldb,
                          const int32_t* row_token, int hidden, __nv_bfloat16* hbuf, int ld_h, float* yexp,
                          cudaStream_t s) {
  constexpr int kDepthSplit = (NT == 1) ? 4 : 2;
  grouped_ffn_splitk_kernel<NT, NMAT, kDepthSplit><<<tiles, kSplitThreads, 0, s>>>(
      groups, tile_group, bsrc, ldb, row_token, hidden, hbuf, ld_h, yexp);
  return cudaGetLastError();
}

int kc_cap_for(int nt, int maxK) {
  // Keep the staged token rows near 33 KB per CTA so several CTAs share an SM.
  int cap = (nt == 1) ? 2048 : (nt == 2) ? 1024 : (nt == 4) ? 512 : 256;
  if (cap > maxK) cap = maxK;
  return cap;
}

template <int NT, int NMAT>
cudaError_t launch_one(const GroupDesc* groups, const int32_t* tile_group, int tiles, const __nv_bfloat16* bsrc,
                       int ldb, const int32_t* row_token, int hidden, int maxK,
                       __nv_bfloat16* hbuf, int ld_h, float* yexp, cudaStream_t s) {
  const int cap = kc_cap_for(NT, maxK);
  const size_t smem = (size_t)8 * NT * (cap + kPadElems) * 2;
  auto kern = grouped_ffn_kernel<NT, NMAT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  kern<<<tiles, kThreads, smem, s>>>(groups, tile_group, bsrc, ldb, row_token, hidden, cap, hbuf, ld_h, yexp);
  return cudaGetLastError();
}

template <int NMAT>
cudaError_t dispatch_nt(int max_rows, const GroupDesc* groups, const int32_t* tile_group, int tiles,
                        const __nv_bfloat16* bsrc, int ldb, const int32_t* row_token, int hidden,
                        int maxK, __nv_bfloat16* hbuf, int ld_h, float* yexp, cudaStream_t s) {
  if (max_rows <= 8)
    return launch_one<1, NMAT>(groups, tile_group, tiles, bsrc, ldb, row_token, hidden, maxK, hbuf, ld_h, yexp, s);
  if (max_rows <= 16)
    return launch_one<2, NMAT>(groups, tile_group, tiles, bsrc, ldb, row_token, hidden, maxK, hbuf, ld_h, yexp, s);
  if (max_rows <= 32)
    return launch_one<4, NMAT>(groups, tile_group, tiles, bsrc, ldb, row_token, hidden, maxK, hbuf, ld_h, yexp, s);
  return launch_one<8, NMAT>(groups, tile_group, tiles, bsrc, ldb, row_token, hidden, maxK, hbuf, ld_h, yexp, s);
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Device-side planner for the experts that are already resident. It turns the router's per-expert
// row counts and the layer's expert -> slot table into a launch plan (descriptors, tile tables,
// zeroed counters) without a host round trip, so the fused kernel for the resident experts and
// the shared expert can be enqueued right behind the router while the host is still reading the
// counts back to decide about the misses.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
plan_resident_kernel(const int32_t* __restrict__ counts, const int32_t* __restrict__ offsets,
                     const int32_t* __restrict__ slot_table, ResidentPlanArgs a, unsigned char* blob) {
  __shared__ int s_n, s_tg, s_td;
  __shared__ int s_cnt[256], s_off[256], s_slot[256];  // staged so that the serial pass reads no global memory
  for (int e = threadIdx.x; e < a.num_expert; e += blockDim.x) {
    s_cnt[e] = counts[e];
    s_off[e] = offsets[e];
    s_slot[e] = slot_table[e];
  }
  __syncthreads();
  GroupDesc* desc = reinterpret_cast<GroupDesc*>(blob + a.off_desc);
  int32_t* t_gu = reinterpret_cast<int32_t*>(blob + a.off_tile_gu);
  int32_t* t_dn = reinterpret_cast<int32_t*>(blob + a.off_tile_dn);
  int32_t* header = reinterpret_cast<int32_t*>(blob);  // [tiles_gu, tiles_dn, counter_gu, counter_dn, n_desc]
  if (threadIdx.x == 0) {
    int n = 0, tg = 0, td = 0;
    const int dn_tiles = a.hidden / kSplitTileDn;
    if (a.shared_inter > 0) {  // heaviest tiles first
      GroupDesc d{};
      d.w_gate = a.shared_w_gate; d.w_up = a.shared_w_up; d.w_down = a.shared_w_down;
      d.row_start = a.n_routed_rows; d.row_count = a.tokens; d.inter = a.shared_inter;
      d.tile_start_gu = tg; d.tile_start_dn = td;
      desc[n++] = d;
      tg += a.shared_inter / kSplitTileGu;
      td += dn_tiles;
    }
    for (int e = 0; e < a.num_expert; ++e) {
      const int slot = s_slot[e];
      if (s_cnt[e] <= 0 || slot < 0) continue;
      const unsigned char* line = a.pool_base + (size_t)slot * a.line_stride;
      GroupDesc d{};
      d.w_gate = line + a.off_gate; d.w_up = line + a.off_up; d.w_down = line + a.off_down;
      d.row_start = s_off[e]; d.row_count = s_cnt[e]; d.inter = a.inter;
      d.tile_start_gu = tg; d.tile_start_dn = td;
      desc[n++] = d;
      tg += a.inter / kSplitTileGu;
      td += dn_tiles;
    }
    s_n = n; s_tg = tg; s_td = td;
    header[0] = tg; header[1] = td; header[2] = 0; header[3] = 0; header[4] = n;
  }
  __syncthreads();
  for (int d = 0; d < s_n; ++d) {
    const int g0 = desc[d].tile_start_gu, g1 = (d + 1 < s_n) ? desc[d + 1].tile_start_gu : s_tg;
    const int d0 = desc[d].tile_start_dn, d1 = (d + 1 < s_n) ? desc[d + 1].tile_start_dn : s_td;
    for (int t = g0 + threadIdx.x; t < g1; t += blockDim.x) t_gu[t] = d;
    for (int t = d0 + threadIdx.x; t < d1; t += blockDim.x) t_dn[t] = d;
  }
}

cudaError_t launch_resident_ffn(const int32_t* counts, const int32_t* offsets, const int32_t* slot_table,
                                const ResidentPlanArgs& a, unsigned char* blob_dev, int max_rows,
                                const __nv_bfloat16* x, const int32_t* row_token, __nv_bfloat16* hbuf, int ld_h,
                                float* yexp, cudaStream_t s, cudaEvent_t start_event) {
  if (max_rows > kSplitMaxRows) return cudaErrorNotSupported;
  plan_resident_kernel<<<1, 256, 0, s>>>(counts, offsets, slot_table, a, blob_dev);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (start_event != nullptr) {
    e = cudaEventRecord(start_event, s);
    if (e != cudaSuccess) return e;
  }
  const GroupDesc* groups = reinterpret_cast<const GroupDesc*>(blob_dev + a.off_desc);
  const int32_t* t_gu = reinterpret_cast<const int32_t*>(blob_dev + a.off_tile_gu);
  const int32_t* t_dn = reinterpret_cast<const int32_t*>(blob_dev + a.off_tile_dn);
  int32_t* header = reinterpret_cast<int32_t*>(blob_dev);
  if (max_rows <= 8)
    return launch_fused<1, 4>(groups, t_gu, t_dn, 0, 0, header + 2, x, a.hidden, row_token, hbuf, ld_h, yexp, s, header);
  return launch_fused<2, 2>(groups, t_gu, t_dn, 0, 0, header + 2, x, a.hidden, row_token, hbuf, ld_h, yexp, s, header);
}

bool resident_ffn_available(int max_rows) {
  if (max_rows > kSplitMaxRows) return false;
  return (max_rows <= 8 ? fused_grid_size_any<1, 4>() : fused_grid_size_any<2, 2>()) > 0;
}

cudaError_t launch_swiglu_ffn(const unsigned char* blob_dev, const FfnPlanInfo& info, int quant4,
                              const __nv_bfloat16* x, int H, const int32_t* row_token,
                              __nv_bfloat16* hbuf, int ld_h, float* yexp, cudaStream_t s,
                              cudaEvent_t mid_event, bool fused) {
  if (info.n_desc <= 0) return cudaSuccess;
  const GroupDesc* groups = reinterpret_cast<const GroupDesc*>(blob_dev);
  const int32_t* t_gu = reinterpret_cast<const int32_t*>(blob_dev + info.off_tile_gu());
  const int32_t* t_dn = reinterpret_cast<const int32_t*>(blob_dev + info.off_tile_dn());
  const int max_rows = info.max_rows;
  cudaError_t e;
  if (quant4) {
    // uint4 experts: split-K decode tiles only (the planner keeps chunks at kSplitMaxRows rows)
    if (max_rows > kSplitMaxRows) return cudaErrorNotSupported;
    e = (max_rows <= 8) ? launch_q4<1, 2>(groups, t_gu, info.tiles_gu, x, H, row_token, H, hbuf, ld_h, yexp, s)
                        : launch_q4<2, 2>(groups, t_gu, info.tiles_gu, x, H, row_token, H, hbuf, ld_h, yexp, s);
    if (e != cudaSuccess) return e;
    if (mid_event != nullptr) {
      e = cudaEventRecord(mid_event, s);
      if (e != cudaSuccess) return e;
    }
    return (max_rows <= 8)
               ? launch_q4<1, 1>(groups, t_dn, info.tiles_dn, hbuf, ld_h, row_token, H, nullptr, ld_h, yexp, s)
               : launch_q4<2, 1>(groups, t_dn, info.tiles_dn, hbuf, ld_h, row_token, H, nullptr, ld_h, yexp, s);
  }
  if (fused && max_rows <= kSplitMaxRows && mid_event == nullptr) {
    int* counters = reinterpret_cast<int*>(const_cast<unsigned char*>(blob_dev) + info.off_counters());
    e = (max_rows <= 8)
            ? launch_fused<1, 4>(groups, t_gu, t_dn, info.tiles_gu, info.tiles_dn, counters, x, H, row_token, hbuf, ld_h, yexp, s)
            : launch_fused<2, 2>(groups, t_gu, t_dn, info.tiles_gu, info.tiles_dn, counters, x, H, row_token, hbuf, ld_h, yexp, s);
    if (e != cudaErrorNotSupported) return e;
    (void)cudaGetLastError();  // cooperative launch unavailable: fall through to the two-launch path
  }
  if (max_rows <= 8) {
    e = launch_splitk<1, 2>(groups, t_gu, info.tiles_gu, x, H, row_token, H, hbuf, ld_h, yexp, s);
  } else if (max_rows <= kSplitMaxRows) {
    e = launch_splitk<2, 2>(groups, t_gu, info.tiles_gu, x, H, row_token, H, hbuf, ld_h, yexp, s);
  } else {
    e = dispatch_nt<2>(max_rows, groups, t_gu, info.tiles_gu, x, H, row_token, H, H, hbuf, ld_h, yexp, s);
  }
  if (e != cudaSuccess) return e;
  if (mid_event != nullptr) {
    e = cudaEventRecord(mid_event, s);
    if (e != cudaSuccess) return e;
  }
  if (max_rows <= 8)
    return launch_splitk<1, 1>(groups, t_dn, info.tiles_dn, hbuf, ld_h, row_token, H, nullptr, ld_h, yexp, s);
  if (max_rows <= kSplitMaxRows)
    return launch_splitk<2, 1>(groups, t_dn, info.tiles_dn, hbuf, ld_h, row_token, H, nullptr, ld_h, yexp, s);
  return dispatch_nt<1>(max_rows, groups, t_dn, info.tiles_dn, hbuf, ld_h, row_token, H, ld_h, nullptr, ld_h,
                        yexp, s);
}

}  // namespace pm
