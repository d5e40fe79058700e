// K3a: grouped SwiGLU expert FFN for decode-size batches, weights read by cache-slot
// indirection:
//   gate/up : h[r, i] = silu(x_r . Wg[i, :]) * (x_r . Wu[i, :])
//   down    : y[r, n] = h_r . Wd[n, :]
// Three kernels share the arithmetic: the fused decode kernel (chunks of at most 16 token rows,
// bf16 or uint4 weights, one cooperative launch for both passes), the two-launch uint4 kernel
// (launches with more chunks than the fused kernel's table holds) and the staged kernel for chunks
// of up to 64 rows (two launches; every CTA tile streams 64 weight rows, 4 warps x 16 rows, and
// applies them to all token rows of its chunk; used where the tensor-core path cannot tile the
// shapes and by the stateless entry point). Every weight byte of an activated expert is read once
// from HBM per chunk with warp-level bf16 MMAs and fp32 accumulation: the bf16 kernels are
// HBM-bound and the weight bytes are the algorithmic traffic.
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
#include <algorithm>
#include <cstdlib>
#include <type_traits>

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

__device__ __forceinline__ uint32_t ldg_stream_u32(const uint32_t* p) {
  uint32_t r;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(r) : "l"(p));
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
// Decode tiles (chunks of at most 16 token rows): a CTA owns one m-tile and its 8 warps split the
// reduction dimension. Shared by the uint4 kernel and the fused bf16 kernel below.
// ---------------------------------------------------------------------------------------------
constexpr int kSplitWarps = 8;
constexpr int kSplitThreads = kSplitWarps * 32;

// Token-row fragment load. Rows written earlier in the same kernel (the fused kernel's down tiles
// read the intermediate rows other CTAs produced) must not go through the non-coherent path.
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

// ---------------------------------------------------------------------------------------------
// Fused decode kernel: ONE cooperative launch per segment, chunks of at most 16 token rows (the
// common case: a handful of tokens per expert). A tile is 16 gate rows + the same 16 up rows, or
// 32 down rows, of one chunk; the 8 warps of a CTA split the reduction dimension, so every warp
// issues its share of weight loads in one or two batches. Token rows come straight from global
// memory (they are tiny and stay in L1/L2) into MMA B fragments.
//
// All tiles of the launch form one sequence, gate/up tiles first, then down tiles, dealt round
// robin to a fixed grid of resident CTAs. There is no grid barrier: a gate/up tile bumps its
// chunk's counter when its intermediate rows are stored, and a down tile waits (bounded) until
// its chunk's counter shows every gate/up tile of the chunk. Because every CTA runs all its
// gate/up tiles before its first down tile and the grid is co-resident (cooperative launch), the
// wait cannot deadlock; it is bounded anyway and reports a give-up through `err`.
//
// Every CTA first builds the launch's chunk table in shared memory, either from descriptors the
// host uploaded or, for the device-planned launch, from the router's per-expert row counts and
// the layer's expert -> slot table. The shared expert enters as slices of its intermediate
// dimension (a chunk per slice: rows of W_gate / W_up, columns of W_down), so its tiles weigh the
// same as a routed expert's and the round-robin deal stays balanced.
// ---------------------------------------------------------------------------------------------
struct FusedGroup {  // shared-memory record of one chunk
  const unsigned char* w_gate;
  const unsigned char* w_up;
  const unsigned char* w_down;
  int32_t row_start, rows, inter, ld_down;
  int32_t tile_gu, tile_dn;  // first gate/up tile, first down tile
};
struct FusedGroupQ4 : FusedGroup {  // uint4 experts: {scale, zero} fp16 pairs per (row, 128-group)
  const uint32_t* q_gate;
  const uint32_t* q_up;
  const uint32_t* q_down;
};
template <bool Q4>
struct GroupOf {
  using type = FusedGroup;
};
template <>
struct GroupOf<true> {
  using type = FusedGroupQ4;
};

struct FusedLaunch {
  const GroupDesc* groups;  // host-planned launch: n_groups descriptors; nullptr = device-planned
  int32_t n_groups, tiles_gu, tiles_dn;
  ResidentArgs res;         // device-planned launch
  int32_t* counters;        // one per chunk, zero at launch
  int32_t* total;           // arrivals of the whole launch, zero at launch
  int32_t* err;             // may be nullptr
  const __nv_bfloat16* x;
  const int32_t* row_token;
  __nv_bfloat16* hbuf;
  float* yexp;
  int32_t hidden, ld_h;
};

// The split-K tile cut into stages, so that a resident CTA can have the first loads of its NEXT
// tile in flight while it reduces and stores the current one. Only what the load stream needs
// lives in registers; everything else is re-read from the shared-memory chunk table.
template <int NT>
struct TileCtx {
  const unsigned char* a_ptr[4];
  const unsigned char* b_ptr[NT];
  const uint32_t* sz_ptr[4];  // uint4 experts only
  int s_end;  // this warp's k-steps
  int gi;     // chunk index
  int m0;     // first weight row of the tile
};

// First chunk at or after `from` whose tile range holds `tile` (tiles only move forward).
template <bool GATEUP, class G>
__device__ __forceinline__ int find_group(const G* sg, int n, int from, int tile) {
  int gi = from;
  while (gi + 1 < n && (GATEUP ? sg[gi + 1].tile_gu : sg[gi + 1].tile_dn) <= tile) ++gi;
  return gi;
}

// Source rows of the tile's token fragments (this lane's n-tile rows): the one global round trip
// a tile needs before its token loads, fetched one tile ahead.
template <int NT, bool GATEUP>
__device__ __forceinline__ void load_src_rows(int (&src_row)[NT], const FusedGroup& d,
                                              const int32_t* __restrict__ row_token) {
  const int g = (threadIdx.x & 31) >> 2;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int n = nt * 8 + g;
    // n-tile slots past the chunk's last row repeat that row: their output columns are never stored,
    // and a valid address spares every token load a null check
    const int nn = min(n, d.rows - 1);
    src_row[nt] = GATEUP ? row_token[d.row_start + nn] : d.row_start + nn;
  }
}

template <int NT, bool GATEUP, int WARPS, class G>
__device__ __forceinline__ void tile_setup(TileCtx<NT>& t, const G& d, int gi, int tile,
                                           const int (&src_row)[NT], const __nv_bfloat16* bsrc, int ldb, int hidden) {
  constexpr bool Q4 = std::is_same<G, FusedGroupQ4>::value;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, q = lane & 3;
  const int tile_local = tile - (GATEUP ? d.tile_gu : d.tile_dn);
  const int K = GATEUP ? hidden : d.inter;
  // bf16: a k-step is 32 elements of a row (4 lanes x 16 bytes); uint4: one 128-weight quantisation
  // group, also 4 lanes x 16 bytes of packed nibbles, against 4 x 64 bytes of token values
  const size_t row_bytes = Q4 ? (size_t)K / 2 : (size_t)(GATEUP ? hidden : d.ld_down) * 2;
  t.gi = gi;
  t.m0 = tile_local * (GATEUP ? 16 : 32);
  // Every warp takes a contiguous range of k-steps (interleaving them across warps, w, w+8, ...,
  // measured 6 % slower: longer contiguous runs per warp suit DRAM better).
  const int steps = Q4 ? K / 128 : K / 32;
  const int first = (warp * steps) / WARPS;
  t.s_end = ((warp + 1) * steps) / WARPS - first;
  const size_t col = (size_t)first * 64 + q * 16;
  int row[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) row[j] = GATEUP ? t.m0 + g + 8 * (j & 1) : t.m0 + g + 8 * j;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const unsigned char* w = GATEUP ? (j < 2 ? d.w_gate : d.w_up) : d.w_down;
    t.a_ptr[j] = w + (size_t)row[j] * row_bytes + col;
  }
  if constexpr (Q4) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t* z = GATEUP ? (j < 2 ? d.q_gate : d.q_up) : d.q_down;
      t.sz_ptr[j] = z + (size_t)row[j] * steps + first;
    }
  }
  const size_t col_b = Q4 ? (size_t)first * 256 + q * 64 : col;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
    t.b_ptr[nt] = reinterpret_cast<const unsigned char*>(bsrc + (size_t)src_row[nt] * ldb) + col_b;
}

// The DEPTH register slots of a lane hold the k-steps s0 .. s0 + DEPTH - 1 of the tile; the helpers
// below work on the slots [FIRST, FIRST + COUNT), so that the two halves can be refilled separately.
template <int NT, int DEPTH, bool Q4, int FIRST = 0, int COUNT = DEPTH>
__device__ __forceinline__ void tile_issue_a(const TileCtx<NT>& t, int s0, uint4 (&a)[DEPTH][4],
                                             uint32_t (&sz)[DEPTH][4]) {
#pragma unroll
  for (int d = FIRST; d < FIRST + COUNT; ++d) {
    if (s0 + d < t.s_end) {
      const size_t off = (size_t)(s0 + d) * 64;
#pragma unroll
      for (int j = 0; j < 4; ++j) a[d][j] = ldg_stream(t.a_ptr[j] + off);
      if constexpr (Q4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) sz[d][j] = __ldg(t.sz_ptr[j] + (s0 + d));
      }
    }
  }
}

template <int NT, int DEPTH, bool COHERENT_B, bool Q4, int FIRST = 0, int COUNT = DEPTH>
__device__ __forceinline__ void tile_issue_b(const TileCtx<NT>& t, int s0, uint4 (&b)[DEPTH][NT]) {
  if constexpr (!Q4) {  // uint4 tiles fetch their token values (L1/L2 hits) inside tile_compute_q4
#pragma unroll
    for (int d = FIRST; d < FIRST + COUNT; ++d) {
      if (s0 + d < t.s_end) {
        const size_t off = (size_t)(s0 + d) * 64;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          b[d][nt] = load_b<COHERENT_B>(t.b_ptr[nt] + off);
      }
    }
  }
}

template <int NT, int DEPTH, int FIRST = 0, int COUNT = DEPTH>
__device__ __forceinline__ void tile_compute(const TileCtx<NT>& t, int s0, const uint4 (&a)[DEPTH][4],
                                             const uint4 (&b)[DEPTH][NT], float (&acc)[2][NT][4]) {
#pragma unroll
  for (int d = FIRST; d < FIRST + COUNT; ++d) {
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

// uint4 k-step: four 16-byte vectors of token values against the four packed words of each weight row
// (see the layout note above q4_pair), then the per-group scale / zero fix-up.
template <int NT, int DEPTH, bool COHERENT_B, int FIRST = 0, int COUNT = DEPTH>
__device__ __forceinline__ void tile_compute_q4(const TileCtx<NT>& t, int s0, const uint4 (&a)[DEPTH][4],
                                                const uint32_t (&sz)[DEPTH][4], float (&acc)[2][NT][4]) {
  constexpr uint32_t kOnes = 0x3F803F80u;  // bf16 (1, 1)
#pragma unroll
  for (int d = FIRST; d < FIRST + COUNT; ++d) {
    if (s0 + d < t.s_end) {
      float raw[NT][2][4], xs[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) raw[nt][0][i] = raw[nt][1][i] = xs[nt][i] = 0.f;
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const uint32_t w00 = (&a[d][0].x)[v], w01 = (&a[d][1].x)[v];  // first pair of rows
        const uint32_t w10 = (&a[d][2].x)[v], w11 = (&a[d][3].x)[v];  // second pair
        uint4 bv[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          bv[nt] = load_b<COHERENT_B>(t.b_ptr[nt] + (size_t)(s0 + d) * 256 + v * 16);
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // nibble pairs {0,1} go with b.x, b.y; pairs {2,3} with b.z, b.w
          // each word is unpacked once and used for every n-tile
          const uint32_t a0 = q4_pair(w00, 2 * h), a1 = q4_pair(w01, 2 * h), a2 = q4_pair(w00, 2 * h + 1),
                         a3 = q4_pair(w01, 2 * h + 1);
          const uint32_t c0 = q4_pair(w10, 2 * h), c1 = q4_pair(w11, 2 * h), c2 = q4_pair(w10, 2 * h + 1),
                         c3 = q4_pair(w11, 2 * h + 1);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint32_t b0 = h ? bv[nt].z : bv[nt].x, b1 = h ? bv[nt].w : bv[nt].y;
            mma_bf16(raw[nt][0], a0, a1, a2, a3, b0, b1);
            mma_bf16(raw[nt][1], c0, c1, c2, c3, b0, b1);
            mma_bf16(xs[nt], kOnes, kOnes, kOnes, kOnes, b0, b1);
          }
        }
      }
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&sz[d][2 * m]));      // row g (+16)
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&sz[d][2 * m + 1]));  // row g + 8 (+16)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          acc[m][nt][0] += lo.x * (raw[nt][m][0] - (128.f + lo.y) * xs[nt][0]);
          acc[m][nt][1] += lo.x * (raw[nt][m][1] - (128.f + lo.y) * xs[nt][1]);
          acc[m][nt][2] += hi.x * (raw[nt][m][2] - (128.f + hi.y) * xs[nt][0]);
          acc[m][nt][3] += hi.x * (raw[nt][m][3] - (128.f + hi.y) * xs[nt][1]);
        }
      }
    }
  }
}

__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

__device__ __forceinline__ int load_relaxed(const int32_t* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Dependency of a down tile on its chunk's gate/up tiles. counters[gi] counts the arrivals of
// chunk gi, *total all arrivals of the launch. Once the launch total shows every
// gate/up tile, `all_done` latches and later tiles skip the check. The poll is a relaxed load; the
// fence that follows a successful poll orders this thread's token-row loads behind it (it runs
// when the thread has no load in flight, so it is cheap). Bounded: after about a quarter of a
// second without progress the wait gives up, records code 4 in *err and lets the tile run on.
__device__ __forceinline__ void wait_rows_ready(const int32_t* counters, const int32_t* total, int gi, int target,
                                                int total_target, bool& all_done, int32_t* err) {
  if (all_done) return;
  if (load_relaxed(total) >= total_target) {
    all_done = true;
  } else {
    bool ok = false;
    for (int i = 0; i < (1 << 21); ++i) {
      if (load_relaxed(counters + gi) >= target) {
        ok = true;
        break;
      }
      __nanosleep(100);
    }
    if (!ok && err != nullptr) atomicExch(err, 4);
  }
  fence_acq_rel_gpu();
}

// Arrival of one gate/up tile of chunk `gi`: called by ONE thread after a CTA barrier that follows
// the tile's stores (the barrier orders them before this thread's fence, the fence publishes them).
__device__ __forceinline__ void arrive_rows(int32_t* counters, int32_t* total, int gi) {
  fence_acq_rel_gpu();
  atomicAdd(counters + gi, 1);
  atomicAdd(total, 1);
}

// Cross-warp reduction of the split-K partial sums and the epilogue. The barrier in here also lies
// behind the stores of the PREVIOUS tile, so one thread signals that tile's arrival (chunk
// `pending`, -1 = none) right after it: it is the last thread of the CTA, whose warp has nothing
// else to do until its next loads land.
template <int NT, bool GATEUP, int WARPS>
__device__ __forceinline__ void tile_finish(const FusedGroup& d, int m0, float (&acc)[2][NT][4],
                                            float (*red)[2 * NT * 4][32], __nv_bfloat16* __restrict__ hbuf, int ld_h,
                                            float* __restrict__ yexp, int hidden, int32_t* counters, int32_t* total,
                                            int pending) {
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
  static_assert(NT * 4 <= WARPS, "one pass of the epilogue, NT * 4 storing warps");
  if (GATEUP && pending >= 0 && threadIdx.x == WARPS * 32 - 1) arrive_rows(counters, total, pending);
  if (warp < NT * 4) {
    const int v = warp;  // nt * 4 + i
    const int nt = v >> 2, i = v & 3;
    float s0v = 0.f, s1v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      s0v += red[w][v][lane];
      s1v += red[w][NT * 4 + v][lane];
    }
    const int lg = lane >> 2, lq = lane & 3;
    const int n = nt * 8 + 2 * lq + (i & 1);
    if (n < d.rows) {
      const int m = m0 + lg + ((i & 2) ? 8 : 0);
      const size_t r = (size_t)(d.row_start + n);
      if (GATEUP) {
        hbuf[r * ld_h + m] = __float2bfloat16_rn(silu(s0v) * s1v);
      } else {
        yexp[r * hidden + m] = s0v;
        yexp[r * hidden + m + 16] = s1v;
      }
    }
  }
  // no trailing barrier: the caller alternates between two reduction buffers, and the barrier above of
  // the NEXT tile orders this tile's reads before the writes of the tile after it
}

template <int NT, int DEPTH>
struct StreamState {
  TileCtx<NT> t;
  uint4 a[DEPTH][4];
  uint4 b[DEPTH][NT];      // bf16 tiles only
  uint32_t sz[DEPTH][4];   // uint4 tiles only
  int tile, buf;
  bool active, all_done;
};

// Sets the CTA's first tile of a phase up and issues its weight loads. Reads only the chunk table,
// the row table and the weights: for the down phase nothing here depends on the gate/up tiles.
template <int NT, bool GATEUP, int DEPTH, int WARPS, class G>
__device__ __forceinline__ void stream_begin(StreamState<NT, DEPTH>& st, const G* sg, int n_groups,
                                             int first_tile, int n_tiles, const __nv_bfloat16* bsrc, int ldb,
                                             const int32_t* __restrict__ row_token, int hidden) {
  st.tile = first_tile;
  st.active = first_tile < n_tiles;
  if (!st.active) return;
  const int gi = find_group<GATEUP>(sg, n_groups, 0, first_tile);
  int src_row[NT];
  load_src_rows<NT, GATEUP>(src_row, sg[gi], row_token);
  tile_setup<NT, GATEUP, WARPS>(st.t, sg[gi], gi, first_tile, src_row, bsrc, ldb, hidden);
  tile_issue_a<NT, DEPTH, std::is_same<G, FusedGroupQ4>::value>(st.t, 0, st.a, st.sz);
}

// Tiles st.tile, st.tile + gridDim.x, ... of one phase. The next tile is known early: its token row
// numbers are fetched one tile ahead and its first batch of loads is issued before the current
// tile is reduced, which keeps DRAM requests in flight across tile boundaries. A gate/up tile's
// arrival is signalled one tile late, behind the next tile's reduction barrier (see tile_finish).
template <int NT, bool GATEUP, int DEPTH, int WARPS, class G>
__device__ __forceinline__ void stream_run(StreamState<NT, DEPTH>& st, const G* sg, int n_groups, int n_tiles,
                                           const __nv_bfloat16* bsrc, int ldb,
                                           const int32_t* __restrict__ row_token, int hidden,
                                           __nv_bfloat16* __restrict__ hbuf, int ld_h, float* __restrict__ yexp,
                                           float (*red2)[WARPS][2 * NT * 4][32], int32_t* counters, int32_t* total,
                                           int total_target, int32_t* err) {
  constexpr bool COH = !GATEUP;  // the down phase reads rows other CTAs wrote in this kernel
  constexpr bool Q4 = std::is_same<G, FusedGroupQ4>::value;
  if (!st.active) return;
  TileCtx<NT>& t = st.t;
  float acc[2][NT][4];
#pragma unroll
  for (int mm = 0; mm < 2; ++mm)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mm][nt][i] = 0.f;
  // arrivals a chunk's counter shows when its intermediate rows are complete
  auto target_of = [&](int gi) { return sg[gi].inter / kSplitTileGu; };
  if (!GATEUP) wait_rows_ready(counters, total, t.gi, target_of(t.gi), total_target, st.all_done, err);
  tile_issue_b<NT, DEPTH, COH, Q4>(t, 0, st.b);
  const int stride = gridDim.x;
  int next = st.tile + stride;
  int pending = -1;  // chunk of the gate/up tile whose arrival is still to be signalled
  while (true) {
    const bool has_next = next < n_tiles;
    const int gi_next = has_next ? find_group<GATEUP>(sg, n_groups, t.gi, next) : 0;
    int src_row[NT];
    bool rows_loaded = false;
    // Two half-batches of k-steps are in flight per lane; whenever one has been consumed it is refilled
    // with the steps DEPTH further on, so a warp always has loads outstanding while it waits.
    constexpr int HALF = DEPTH / 2;
    for (int s0 = 0; s0 < t.s_end; s0 += DEPTH) {
      if constexpr (Q4) tile_compute_q4<NT, DEPTH, COH, 0, HALF>(t, s0, st.a, st.sz, acc);
      else tile_compute<NT, DEPTH, 0, HALF>(t, s0, st.a, st.b, acc);
      if (s0 + DEPTH < t.s_end) {
        tile_issue_a<NT, DEPTH, Q4, 0, HALF>(t, s0 + DEPTH, st.a, st.sz);
        tile_issue_b<NT, DEPTH, COH, Q4, 0, HALF>(t, s0 + DEPTH, st.b);
      }
      if (has_next && !rows_loaded) {  // fetch the next tile's token row numbers under this tile's loads
        load_src_rows<NT, GATEUP>(src_row, sg[gi_next], row_token);
        rows_loaded = true;
      }
      if (s0 + HALF < t.s_end) {
        if constexpr (Q4) tile_compute_q4<NT, DEPTH, COH, HALF, HALF>(t, s0, st.a, st.sz, acc);
        else tile_compute<NT, DEPTH, HALF, HALF>(t, s0, st.a, st.b, acc);
        if (s0 + DEPTH + HALF < t.s_end) {
          tile_issue_a<NT, DEPTH, Q4, HALF, HALF>(t, s0 + DEPTH, st.a, st.sz);
          tile_issue_b<NT, DEPTH, COH, Q4, HALF, HALF>(t, s0 + DEPTH, st.b);
        }
      }
    }
    if (has_next && !rows_loaded) load_src_rows<NT, GATEUP>(src_row, sg[gi_next], row_token);
    const int gi = t.gi, m0 = t.m0;
    if (has_next) {
      if (!GATEUP) wait_rows_ready(counters, total, gi_next, target_of(gi_next), total_target, st.all_done, err);
      tile_setup<NT, GATEUP, WARPS>(t, sg[gi_next], gi_next, next, src_row, bsrc, ldb, hidden);
      tile_issue_a<NT, DEPTH, Q4>(t, 0, st.a, st.sz);
      tile_issue_b<NT, DEPTH, COH, Q4>(t, 0, st.b);
    }
    tile_finish<NT, GATEUP, WARPS>(sg[gi], m0, acc, red2[st.buf], hbuf, ld_h, yexp, hidden, counters, total, pending);
    pending = gi;
    st.buf ^= 1;
    if (!has_next) break;
    next += stride;
  }
  if (GATEUP) {  // the last tile's arrival: once per CTA
    __syncthreads();
    if (threadIdx.x == WARPS * 32 - 1) arrive_rows(counters, total, pending);
  }
}

// Chunk table of the launch in shared memory; meta = {chunks, gate/up tiles, down tiles}.
template <class G>
__device__ __forceinline__ void build_chunk_table(const FusedLaunch& a, G* sg, int* meta) {
  constexpr bool Q4 = std::is_same<G, FusedGroupQ4>::value;
  if (a.groups != nullptr) {
    for (int i = threadIdx.x; i < a.n_groups; i += blockDim.x) {
      const GroupDesc& d = a.groups[i];
      G g;
      if constexpr (Q4) {
        g.q_gate = reinterpret_cast<const uint32_t*>(d.q_gate);
        g.q_up = reinterpret_cast<const uint32_t*>(d.q_up);
        g.q_down = reinterpret_cast<const uint32_t*>(d.q_down);
      }
      g.w_gate = reinterpret_cast<const unsigned char*>(d.w_gate);
      g.w_up = reinterpret_cast<const unsigned char*>(d.w_up);
      g.w_down = reinterpret_cast<const unsigned char*>(d.w_down);
      g.row_start = d.row_start;
      g.rows = d.row_count;
      g.inter = d.inter;
      g.ld_down = d.ld_down > 0 ? d.ld_down : d.inter;
      g.tile_gu = d.tile_start_gu;
      g.tile_dn = d.tile_start_dn;
      sg[i] = g;
    }
    if (threadIdx.x == 0) {
      meta[0] = a.n_groups;
      meta[1] = a.tiles_gu;
      meta[2] = a.tiles_dn;
    }
    return;
  }
  if constexpr (Q4) {  // uint4 launches are always host-planned
    if (threadIdx.x == 0) meta[0] = meta[1] = meta[2] = 0;
    return;
  }
  const ResidentArgs& r = a.res;
  const int dn_tiles = a.hidden / kSplitTileDn;
  const int slice = r.shared_slice;
  const int n_sh = r.shared_inter > 0 ? (r.shared_inter + slice - 1) / slice : 0;
  const int sh_tiles = r.shared_inter / kSplitTileGu;
  if ((int)threadIdx.x < n_sh) {  // heaviest rows first: the slices of the shared expert
    const int j = threadIdx.x;
    G g{};
    g.w_gate = reinterpret_cast<const unsigned char*>(r.shared_w_gate) + (size_t)j * slice * a.hidden * 2;
    g.w_up = reinterpret_cast<const unsigned char*>(r.shared_w_up) + (size_t)j * slice * a.hidden * 2;
    g.w_down = reinterpret_cast<const unsigned char*>(r.shared_w_down) + (size_t)j * slice * 2;
    g.row_start = r.n_routed_rows + j * r.tokens;
    g.rows = r.tokens;
    g.inter = min(slice, r.shared_inter - j * slice);
    g.ld_down = r.shared_inter;
    g.tile_gu = j * (slice / kSplitTileGu);
    g.tile_dn = j * dn_tiles;
    sg[j] = g;
  }
  if (threadIdx.x < 32) {  // one warp compacts the activated resident experts in ascending id order
    const int lane = threadIdx.x;
    const unsigned lt = (1u << lane) - 1u;
    const int gu_tiles = r.inter / kSplitTileGu;
    int base = n_sh;
    for (int c = 0; c < r.num_expert; c += 32) {
      const int e = c + lane;
      int cnt = 0, slot = -1, off = 0;
      if (e < r.num_expert) {
        cnt = r.counts[e];
        slot = r.slot_table[e];
        off = r.offsets[e];
      }
      const bool act = cnt > 0 && slot >= 0;
      const unsigned mask = __ballot_sync(0xffffffffu, act);
      if (act) {
        const int idx = base + __popc(mask & lt);
        const unsigned char* line = r.pool_base + (size_t)slot * r.line_stride;
        G g{};
        g.w_gate = line + r.off_gate;
        g.w_up = line + r.off_up;
        g.w_down = line + r.off_down;
        g.row_start = off;
        g.rows = cnt;
        g.inter = r.inter;
        g.ld_down = r.inter;
        g.tile_gu = sh_tiles + (idx - n_sh) * gu_tiles;
        g.tile_dn = idx * dn_tiles;
        sg[idx] = g;
      }
      base += __popc(mask);
    }
    if (lane == 0) {
      meta[0] = base;
      meta[1] = sh_tiles + (base - n_sh) * gu_tiles;
      meta[2] = base * dn_tiles;
    }
  }
}

template <int NT, int DEPTH, int WARPS, bool Q4>
__global__ void __launch_bounds__(WARPS * 32, 16 / WARPS)
grouped_ffn_fused_kernel(const __grid_constant__ FusedLaunch a) {
  __shared__ float red[2][WARPS][2 * NT * 4][32];  // two reduction buffers, used alternately
  __shared__ typename GroupOf<Q4>::type sg[Q4 ? kMaxFusedGroupsQ4 : kMaxFusedGroups];
  __shared__ int meta[3];
  build_chunk_table(a, sg, meta);
  __syncthreads();
  const int n = meta[0], tiles_gu = meta[1], tiles_dn = meta[2];
  const int total_target = tiles_gu;  // arrivals of the whole launch: one per gate/up tile
  const int b = blockIdx.x, grid = gridDim.x;
  StreamState<NT, DEPTH> st;
  st.buf = 0;
  st.all_done = false;
  stream_begin<NT, true, DEPTH, WARPS>(st, sg, n, b, tiles_gu, a.x, a.hidden, a.row_token, a.hidden);
  stream_run<NT, true, DEPTH, WARPS>(st, sg, n, tiles_gu, a.x, a.hidden, a.row_token, a.hidden, a.hbuf, a.ld_h, a.yexp,
                                     red, a.counters, a.total, total_target, a.err);
  // This CTA's place in the one round-robin sequence continues into the down tiles, so the CTAs
  // that had one gate/up tile fewer take the first down tiles.
  const int n1 = b < tiles_gu ? (tiles_gu - b + grid - 1) / grid : 0;
  const int first_dn = b + n1 * grid - tiles_gu;
  stream_begin<NT, false, DEPTH, WARPS>(st, sg, n, first_dn, tiles_dn, a.hbuf, a.ld_h, a.row_token, a.hidden);
  stream_run<NT, false, DEPTH, WARPS>(st, sg, n, tiles_dn, a.hbuf, a.ld_h, a.row_token, a.hidden, nullptr, a.ld_h,
                                      a.yexp, red, a.counters, a.total, total_target, a.err);
}

// 8 warps x 2 CTAs per SM. (16 warps x 1 CTA, one batch of loads per tile, measured 28 % slower at
// 60 experts: with a single CTA per SM nothing overlaps the reduction.)
constexpr int kFusedWarps = 8;

// Resident grid of the fused kernel on the current device (0 if cooperative launch is unavailable).
template <int NT, int DEPTH, bool Q4>
int fused_grid_size() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] != 0) return cached[dev] < 0 ? 0 : cached[dev];
  int coop = 0, sms = 0, per_sm = 0;
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (!coop || sms <= 0 ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, grouped_ffn_fused_kernel<NT, DEPTH, kFusedWarps, Q4>,
                                                    kFusedWarps * 32, 0) != cudaSuccess ||
      per_sm <= 0) {
    cached[dev] = -1;
    return 0;
  }
  cached[dev] = sms * per_sm;
  return cached[dev];
}

template <int NT, int DEPTH, bool Q4 = false>
cudaError_t launch_fused(const FusedLaunch& a, int total_tiles, cudaStream_t s) {
  int grid = fused_grid_size<NT, DEPTH, Q4>();
  if (grid <= 0) return cudaErrorNotSupported;
  if (total_tiles > 0) grid = min(grid, total_tiles);
  void* args[] = {(void*)&a};
  return cudaLaunchCooperativeKernel((const void*)grouped_ffn_fused_kernel<NT, DEPTH, kFusedWarps, Q4>, dim3(grid),
                                     dim3(kFusedWarps * 32), args, 0, s);
}

cudaError_t launch_fused_rows(const FusedLaunch& a, int max_rows, int total_tiles, cudaStream_t s) {
  return max_rows <= 8 ? launch_fused<1, 4>(a, total_tiles, s) : launch_fused<2, 2>(a, total_tiles, s);
}

// uint4 experts: a k-step is a whole 128-weight group, so two steps per lane are in flight
cudaError_t launch_fused_rows_q4(const FusedLaunch& a, int max_rows, int total_tiles, cudaStream_t s) {
  return max_rows <= 8 ? launch_fused<1, 2, true>(a, total_tiles, s) : launch_fused<2, 2, true>(a, total_tiles, s);
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

// Expands one uint4 group-128 matrix [rows, K] into bf16 (for the prefill path, which reads bf16 tiles
// by TMA): a thread turns one 32-bit word (8 weights: even-k nibbles in the low half, odd-k nibbles in
// the high half) into 16 bytes of bf16, w = (q - zero) * scale in float32, rounded once.
__global__ void __launch_bounds__(256)
dequant_q4_kernel(const uint32_t* __restrict__ packed, const uint32_t* __restrict__ sz, size_t n_words,
                  int words_per_row, uint4* __restrict__ out) {
  const int groups_per_row = words_per_row / 16;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t w = ldg_stream_u32(packed + i);
    const size_t row = i / words_per_row;
    const int wc = (int)(i - row * words_per_row);
    const uint32_t m = __ldg(sz + row * groups_per_row + wc / 16);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&m));  // x = scale, y = zero
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float even = ((float)((w >> (4 * j)) & 0xFu) - f.y) * f.x;
      const float odd = ((float)((w >> (16 + 4 * j)) & 0xFu) - f.y) * f.x;
      const __nv_bfloat162 pair = __floats2bfloat162_rn(even, odd);
      o[j] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace

cudaError_t launch_resident_ffn(const ResidentArgs& r, int32_t* counters, int32_t* err, int max_rows,
                                const __nv_bfloat16* x, int hidden, const int32_t* row_token,
                                __nv_bfloat16* hbuf, int ld_h, float* yexp, cudaStream_t s) {
  if (max_rows > kSplitMaxRows) return cudaErrorNotSupported;
  FusedLaunch a{};
  a.groups = nullptr;
  a.res = r;
  a.counters = counters;
  a.total = counters + kMaxFusedGroups;
  a.err = err;
  a.x = x;
  a.row_token = row_token;
  a.hbuf = hbuf;
  a.yexp = yexp;
  a.hidden = hidden;
  a.ld_h = ld_h;
  return launch_fused_rows(a, max_rows, 0, s);  // the tile count is only known on the device: full grid
}

bool resident_ffn_available(int max_rows) {
  if (max_rows > kSplitMaxRows) return false;
  return (max_rows <= 8 ? fused_grid_size<1, 4, false>() : fused_grid_size<2, 2, false>()) > 0;
}

cudaError_t launch_swiglu_ffn(const unsigned char* blob_dev, const FfnPlanInfo& info, int quant4,
                              const __nv_bfloat16* x, int H, const int32_t* row_token,
                              __nv_bfloat16* hbuf, int ld_h, float* yexp, cudaStream_t s,
                              cudaEvent_t mid_event, int32_t* err) {
  if (info.n_desc <= 0) return cudaSuccess;
  const GroupDesc* groups = reinterpret_cast<const GroupDesc*>(blob_dev);
  const int32_t* t_gu = reinterpret_cast<const int32_t*>(blob_dev + info.off_tile_gu());
  const int32_t* t_dn = reinterpret_cast<const int32_t*>(blob_dev + info.off_tile_dn());
  const int max_rows = info.max_rows;
  cudaError_t e;
  if (ffn_launch_is_fused(info, quant4)) {
    FusedLaunch a{};
    a.groups = groups;
    a.n_groups = info.n_desc;
    a.tiles_gu = info.tiles_gu;
    a.tiles_dn = info.tiles_dn;
    int32_t* counters = reinterpret_cast<int32_t*>(const_cast<unsigned char*>(blob_dev) + info.off_counters());
    a.counters = counters;
    a.total = counters + info.n_desc;
    a.err = err != nullptr ? err : counters + info.n_desc + 1;  // default: the blob's error word
    a.x = x;
    a.row_token = row_token;
    a.hbuf = hbuf;
    a.yexp = yexp;
    a.hidden = H;
    a.ld_h = ld_h;
    const int tiles = info.tiles_gu + info.tiles_dn;
    return quant4 ? launch_fused_rows_q4(a, max_rows, tiles, s) : launch_fused_rows(a, max_rows, tiles, s);
  }
  if (quant4) {
    // more uint4 chunks than the fused kernel's table holds: split-K decode tiles in two launches
    // (the planner keeps uint4 chunks at kSplitMaxRows rows)
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
  e = dispatch_nt<2>(max_rows, groups, t_gu, info.tiles_gu, x, H, row_token, H, H, hbuf, ld_h, yexp, s);
  if (e != cudaSuccess) return e;
  if (mid_event != nullptr) {
    e = cudaEventRecord(mid_event, s);
    if (e != cudaSuccess) return e;
  }
  return dispatch_nt<1>(max_rows, groups, t_dn, info.tiles_dn, hbuf, ld_h, row_token, H, ld_h, nullptr, ld_h,
                        yexp, s);
}

cudaError_t launch_dequant_q4(const void* packed, const void* scale_zero, int rows, int K, __nv_bfloat16* out,
                              cudaStream_t s) {
  if (rows <= 0 || K <= 0 || K % 128 != 0) return cudaErrorInvalidValue;
  const size_t n_words = (size_t)rows * (K / 8);
  const unsigned blocks = (unsigned)std::min<size_t>((n_words + 255) / 256, 148 * 16);
  dequant_q4_kernel<<<blocks, 256, 0, s>>>((const uint32_t*)packed, (const uint32_t*)scale_zero, n_words, K / 8,
                                           (uint4*)out);
  return cudaGetLastError();
}

}  // namespace pm
