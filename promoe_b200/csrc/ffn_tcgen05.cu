// K3b: grouped SwiGLU expert FFN for prefill-size batches on the 5th-generation tensor cores.
// One CTA computes a 128-row x 128-column tile of one expert's gate AND up projections (two f32
// accumulators in tensor memory), or of its down projection, with tcgen05.mma issued by one
// thread, operands staged in shared memory by TMA (128-byte swizzle, 2- or 3-stage mbarrier ring) and
// the accumulators read back with tcgen05.ld for the epilogue (SwiGLU -> bf16, or f32 rows).
//
// Rows are the expert-sorted token rows (gathered once per layer call), so an expert's rows are
// contiguous; a tile may run past the expert's last row into its neighbour's rows or past the
// end of the buffer (TMA zero fill): those rows are computed and never stored. Expert weights
// are addressed by cache line through ONE 3-D tensor map per projection over the whole slab
// (k, weight row, line); the shared expert has 2-D maps of its own. No multicast is used.
//
// It replaces, for batches of more than 16 rows per expert, the per-expert torch linears the
// reference runs in its Python expert loop (src/sparse_llm_cache/utils/hooks.py:187-198).
//
// Every mbarrier wait is bounded; on a give-up the kernel records a code in *err, skips the
// epilogue, frees its tensor memory and returns.
#include "pm_common.cuh"
#include "sm100_ptx.cuh"

namespace pm {

namespace {

using namespace sm100;

constexpr int kTcThreads = 128;
constexpr int kBM = 128, kBK = 64;  // tile rows, k per stage (128 bytes of bf16)
// Tile columns: 128 for gate/up (two accumulators = 256 TMEM columns), 256 for down (one).
template <bool GATEUP>
constexpr int tc_bn() { return GATEUP ? 128 : 256; }
constexpr int kTileBytes = kBM * kBK * 2;  // 16 KB: one operand tile of one stage

// Two CTAs share an SM (96 KB of operand stages and 256 / 128 TMEM columns each), so that one CTA's
// epilogue overlaps the other's main loop: 2 stages of 3 tiles for gate/up, 3 stages of 2 for down.
// Both passes stage 3 x 16 KB per k-step (token tile + two 128-row weight tiles) in 2 stages.
template <bool GATEUP>
constexpr int tc_stages() { return 2; }

template <bool GATEUP>
constexpr size_t tc_smem_bytes() {
  return 1024 /*alignment slack*/ + (size_t)tc_stages<GATEUP>() * 3 * kTileBytes + 256;
}

template <bool GATEUP>
__global__ void __launch_bounds__(kTcThreads, 2)
prefill_ffn_kernel(const __grid_constant__ TcMaps maps, const TcGroup* __restrict__ groups,
                   const TcTile* __restrict__ tiles, int hidden, __nv_bfloat16* __restrict__ hbuf, int ld_h,
                   float* __restrict__ yexp, int32_t* __restrict__ err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kOperands = 3;  // token tile, then gate + up tiles or the two halves of a 256-row down tile
  constexpr int kStages = tc_stages<GATEUP>();
  constexpr int kBN = tc_bn<GATEUP>();
  unsigned char* stage_base = smem;  // [stage][operand][16 KB]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * kOperands * kTileBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_bar = empty_bar + kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TcTile tile = tiles[blockIdx.x];
  const TcGroup grp = groups[tile.group];
  const int K = GATEUP ? hidden : grp.inter;
  const int n_total = GATEUP ? grp.inter : hidden;
  const int k_tiles = K / kBK;
  constexpr uint32_t kCols = 256;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
    *s_abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const bool shared_expert = grp.line < 0;
  const CUtensorMap* map_a = GATEUP ? &maps.a_x : &maps.a_h;
  const CUtensorMap* map_b0 = GATEUP ? (shared_expert ? &maps.sh_gate : &maps.slab_gate)
                                     : (shared_expert ? &maps.sh_down : &maps.slab_down);
  const CUtensorMap* map_b1 = shared_expert ? &maps.sh_up : &maps.slab_up;

  if (warp == 0 && lane == 0) {
    // ---- producer: TMA loads into the stage ring ------------------------------------------
    prefetch_tmap(map_a);
    prefetch_tmap(map_b0);
    if (GATEUP) prefetch_tmap(map_b1);
    const int row0 = grp.row_start + tile.m0;
    for (int kt = 0; kt < k_tiles; ++kt) {
      const int s = kt % kStages;
      if (kt >= kStages && !mbar_wait(&empty_bar[s], ((kt / kStages) - 1) & 1, 1u << 20)) {
        atomicExch(err, 1);
        *s_abort = 1;
        break;
      }
      if (*s_abort) break;
      unsigned char* st = stage_base + (size_t)s * kOperands * kTileBytes;
      mbar_arrive_expect_tx(&full_bar[s], kOperands * kTileBytes);
      const int k0 = kt * kBK;
      tma_load_2d(st, map_a, &full_bar[s], k0, row0);
      // second weight tile: the up projection, or rows n0+128.. of the same down tile
      const CUtensorMap* map_b_second = GATEUP ? map_b1 : map_b0;
      const int n_second = GATEUP ? tile.n0 : tile.n0 + 128;
      if (shared_expert) {
        tma_load_2d(st + kTileBytes, map_b0, &full_bar[s], k0, tile.n0);
        tma_load_2d(st + 2 * kTileBytes, map_b_second, &full_bar[s], k0, n_second);
      } else {
        tma_load_3d(st + kTileBytes, map_b0, &full_bar[s], k0, tile.n0, grp.line);
        tma_load_3d(st + 2 * kTileBytes, map_b_second, &full_bar[s], k0, n_second, grp.line);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ------------------------------------------------------------------------
    constexpr uint32_t idesc = umma_idesc_bf16(kBM, kBN);
    bool ok = true;
    for (int kt = 0; kt < k_tiles && ok; ++kt) {
      const int s = kt % kStages;
      if (!mbar_wait(&full_bar[s], (kt / kStages) & 1, 1u << 20)) {
        atomicExch(err, 2);
        *s_abort = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t a_addr = smem_u32(stage_base + (size_t)s * kOperands * kTileBytes);
#pragma unroll
      for (int k = 0; k < kBK / 16; ++k) {  // UMMA K = 16 bf16 = 32 bytes inside the swizzled row
        const uint64_t da = umma_desc_k_sw128(a_addr + k * 32);
        const uint64_t db0 = umma_desc_k_sw128(a_addr + kTileBytes + k * 32);
        const uint32_t accumulate = (kt > 0 || k > 0) ? 1u : 0u;
        umma_bf16(tmem_base, da, db0, idesc, accumulate);  // down: one N = 256 MMA over both weight tiles
        if (GATEUP) {
          const uint64_t db1 = umma_desc_k_sw128(a_addr + 2 * kTileBytes + k * 32);
          umma_bf16(tmem_base + kBN, da, db1, idesc, accumulate);
        }
      }
      umma_commit(&empty_bar[s]);  // the stage may be refilled once these MMAs have read it
    }
    if (ok) umma_commit(acc_bar);  // accumulators complete
  }

  // ---- epilogue: all four warps, warp w owns accumulator rows 32w .. 32w+31 ---------------------
  __syncwarp();
  bool have_acc = mbar_wait(acc_bar, 0, 1u << 21);
  if (!have_acc && threadIdx.x == 0) atomicExch(err, 3);
  tc_fence_after();
  if (have_acc && !*s_abort) {
    const int r_in_tile = 32 * warp + lane;
    const int row_in_group = tile.m0 + r_in_tile;
    const bool row_ok = row_in_group < grp.row_count;
    const size_t out_row = (size_t)(grp.row_start + row_in_group);
    const uint32_t lane_base = tmem_base + ((uint32_t)(32 * warp) << 16);
#pragma unroll 1
    for (int c = 0; c < kBN / 32; ++c) {
      uint32_t g[32];
      tmem_ld32(lane_base + c * 32, g);
      const int col0 = tile.n0 + c * 32;
      if (GATEUP) {
        uint32_t u[32];
        tmem_ld32(lane_base + kBN + c * 32, u);
        tmem_ld_wait();
        if (row_ok && col0 < n_total) {
          uint32_t packed[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
            const float h0 = g0 / (1.f + __expf(-g0)) * __uint_as_float(u[2 * j]);
            const float h1 = g1 / (1.f + __expf(-g1)) * __uint_as_float(u[2 * j + 1]);
            __nv_bfloat162 p = __floats2bfloat162_rn(h0, h1);
            packed[j] = *reinterpret_cast<uint32_t*>(&p);
          }
          __nv_bfloat16* dst = hbuf + out_row * ld_h + col0;
          if (col0 + 32 <= n_total) {
#pragma unroll
            for (int v = 0; v < 4; ++v)
              reinterpret_cast<uint4*>(dst)[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
          } else {
            for (int j = 0; j < 32 && col0 + j < n_total; ++j)
              dst[j] = reinterpret_cast<__nv_bfloat16*>(packed)[j];
          }
        }
      } else {
        tmem_ld_wait();
        if (row_ok && col0 < n_total) {
          float* dst = yexp + out_row * hidden + col0;
          if (col0 + 32 <= n_total) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
              reinterpret_cast<uint4*>(dst)[v] = make_uint4(g[4 * v], g[4 * v + 1], g[4 * v + 2], g[4 * v + 3]);
          } else {
            for (int j = 0; j < 32 && col0 + j < n_total; ++j) dst[j] = __uint_as_float(g[j]);
          }
        }
      }
    }
  } else if (*s_abort) {
    // give loads that are still in flight time to land before the shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kCols);
}

}  // namespace

cudaError_t launch_prefill_ffn(const TcMaps& maps, const TcGroup* groups_dev, const TcTile* tiles_gu_dev, int n_gu,
                               const TcTile* tiles_dn_dev, int n_dn, int hidden, __nv_bfloat16* hbuf, int ld_h,
                               float* yexp, int32_t* err_dev, cudaStream_t s, cudaEvent_t mid_event) {
  // the attribute is per device: a process that drives several GPUs opts in on each of them
  static bool configured_dev[64] = {};
  int dev = 0;
  cudaError_t e0 = cudaGetDevice(&dev);
  if (e0 != cudaSuccess) return e0;
  const bool known = dev >= 0 && dev < 64;
  if (!known || !configured_dev[dev]) {
    cudaError_t e = cudaFuncSetAttribute(prefill_ffn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)tc_smem_bytes<true>());
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(prefill_ffn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)tc_smem_bytes<false>());
    if (e != cudaSuccess) return e;
    if (known) configured_dev[dev] = true;
  }
  if (n_gu > 0)
    prefill_ffn_kernel<true><<<n_gu, kTcThreads, tc_smem_bytes<true>(), s>>>(maps, groups_dev, tiles_gu_dev, hidden,
                                                                              hbuf, ld_h, yexp, err_dev);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (mid_event != nullptr) {
    e = cudaEventRecord(mid_event, s);
    if (e != cudaSuccess) return e;
  }
  if (n_dn > 0)
    prefill_ffn_kernel<false><<<n_dn, kTcThreads, tc_smem_bytes<false>(), s>>>(maps, groups_dev, tiles_dn_dev, hidden,
                                                                                hbuf, ld_h, yexp, err_dev);
  return cudaGetLastError();
}

}  // namespace pm
