// Host side of the prefill (tcgen05) path: tensor-map encoding and tile planning for one segment.
#include <algorithm>
#include <cstring>

#include "runtime.hpp"

namespace pm {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    cudaDriverEntryPointQueryResult q;
    void* p = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// bf16 tensor, innermost dimension k: box = 64 k x 128 rows (x 1 line), 128-byte swizzle, zero fill.
int encode(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(PM_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides_bytes,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
  return PM_OK;
}

int encode_2d(CUtensorMap* map, const void* base, uint64_t k, uint64_t rows, uint64_t pitch_elems) {
  cuuint64_t dims[2] = {k, rows};
  cuuint64_t strides[1] = {pitch_elems * 2};
  return encode(map, base, 2, dims, strides);
}

}  // namespace

bool tc_prefill_usable(const pm_ctx* c, const pm_layer_weights& w) {
  if (!c->tc_prefill || w.quant4 || encode_fn() == nullptr) return false;
  if (w.hidden % 64 != 0 || w.inter % 64 != 0 || w.shared_inter % 64 != 0) return false;
  return true;
}

bool tc_prefill_usable_q4(const pm_ctx* c, const pm_layer_weights& w) {
  if (!c->tc_prefill || !w.quant4 || encode_fn() == nullptr) return false;
  return w.hidden % 128 == 0 && w.inter % 128 == 0 && w.shared_inter % 64 == 0;
}

namespace {

// Maps of the token rows, of a slab of bf16 expert lines (`lines` lines `stride` bytes apart, the
// three matrices at the given addresses of line 0) and of the layer's shared expert.
int build_maps(pm_ctx* c, const pm_layer_weights& w, int rows_cap, const unsigned char* gate0,
               const unsigned char* up0, const unsigned char* down0, uint64_t stride, uint64_t lines, TcMaps* m) {
  const uint64_t H = w.hidden, I = w.inter;
  int rc = encode_2d(&m->a_x, c->d_xperm, H, (uint64_t)rows_cap, H);
  if (rc != PM_OK) return rc;
  rc = encode_2d(&m->a_h, c->d_hbuf, (uint64_t)c->ws_inter, (uint64_t)rows_cap, (uint64_t)c->ws_inter);
  if (rc != PM_OK) return rc;
  {
    cuuint64_t dims[3] = {H, I, lines};
    cuuint64_t strides[2] = {H * 2, (cuuint64_t)stride};
    rc = encode(&m->slab_gate, gate0, 3, dims, strides);
    if (rc != PM_OK) return rc;
    rc = encode(&m->slab_up, up0, 3, dims, strides);
    if (rc != PM_OK) return rc;
  }
  {
    cuuint64_t dims[3] = {I, H, lines};
    cuuint64_t strides[2] = {I * 2, (cuuint64_t)stride};
    rc = encode(&m->slab_down, down0, 3, dims, strides);
    if (rc != PM_OK) return rc;
  }
  if (w.shared_inter > 0) {
    const uint64_t Is = w.shared_inter;
    rc = encode_2d(&m->sh_gate, w.shared_w_gate, H, Is, H);
    if (rc != PM_OK) return rc;
    rc = encode_2d(&m->sh_up, w.shared_w_up, H, Is, H);
    if (rc != PM_OK) return rc;
    rc = encode_2d(&m->sh_down, w.shared_w_down, Is, H, Is);
    if (rc != PM_OK) return rc;
  } else {  // never dereferenced: any valid map keeps the parameter well formed
    m->sh_gate = m->slab_gate;
    m->sh_up = m->slab_up;
    m->sh_down = m->slab_down;
  }
  return PM_OK;
}

}  // namespace

int tc_build_maps(pm_ctx* c, const pm_layer_weights& w, int rows_cap, TcMaps* m) {
  return build_maps(c, w, rows_cap, c->slab + c->param_offset[c->role_gate], c->slab + c->param_offset[c->role_up],
                    c->slab + c->param_offset[c->role_down], (uint64_t)c->line_stride, (uint64_t)c->n_lines, m);
}

int tc_build_maps_q4(pm_ctx* c, const pm_layer_weights& w, int rows_cap, TcMaps* m) {
  const size_t mat = (size_t)w.inter * w.hidden * 2;
  return build_maps(c, w, rows_cap, c->q4_scratch, c->q4_scratch + mat, c->q4_scratch + 2 * mat,
                    (uint64_t)c->q4_scratch_stride, (uint64_t)c->q4_scratch_lines, m);
}

// Tiles of one segment: every 128-row block of every group times every 128-column block of the
// gate/up projections and every 256-column block of the down projection.
void tc_plan(const std::vector<TcGroup>& groups, int hidden, std::vector<TcTile>* gu, std::vector<TcTile>* dn) {
  gu->clear();
  dn->clear();
  for (int g = 0; g < (int)groups.size(); ++g) {
    const TcGroup& grp = groups[g];
    for (int m0 = 0; m0 < grp.row_count; m0 += 128) {
      for (int n0 = 0; n0 < grp.inter; n0 += 128) gu->push_back(TcTile{g, m0, n0, 0});
      for (int n0 = 0; n0 < hidden; n0 += 256) dn->push_back(TcTile{g, m0, n0, 0});
    }
  }
}

}  // namespace pm
