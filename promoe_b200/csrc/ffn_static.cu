// pm_k_swiglu_ffn_static: the grouped SwiGLU FFN for callers that cannot give it scratch memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need the FFN: a
// serving engine that sized its own pools to all remaining HBM at start-up has nothing left to
// hand out, and a latency-critical decode loop cannot afford an allocation, which synchronises
// the whole device. For them the launch plan and the bf16 intermediate rows live in a fixed
// array that is part of the library image: every GPU that loads the library holds
// kStaticScratchBytes of it until the process exits.
//
// The array's name is only a host-side handle. Its device address is looked up once per device
// (with that device current) through cudaGetSymbolAddress, and that address is what the kernels
// receive. The first call on a device performs this look-up. A call on a stream that is being
// captured is refused (PM_ERR_UNSUPPORTED): the plan is uploaded from the host stack. All calls share the one array and it keeps the previous call's bytes: every
// byte a launch reads (plan, intermediate rows of its own groups) is written by the same call
// first, so nothing needs clearing, but two calls that overlap on the GPU (different streams,
// or different threads) would overwrite each other's plan and rows -- serialise them.
#include <cstdio>
#include <mutex>

#include "pm_common.cuh"

namespace pm {
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB per GPU
constexpr size_t kStaticPlanBytes = 64u << 10;    // largest launch plan it accepts (host stack buffer)
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_ffn_scratch[kStaticScratchBytes];

std::mutex g_addr_mutex;
unsigned char* g_scratch_addr[kMaxDevices] = {};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Device address of g_ffn_scratch on the current device; resolved on first use.
int scratch_address(unsigned char** out) {
  int dev = -1;
  PM_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(PM_ERR_UNSUPPORTED, "swiglu_ffn_static: device index above 63");
  std::lock_guard<std::mutex> lock(g_addr_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_ffn_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(g_ffn_scratch)");
    if (p == nullptr) return fail(PM_ERR_CUDA, "swiglu_ffn_static: the scratch array has no device address");
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_addr[dev];
  return PM_OK;
}

}  // namespace
}  // namespace pm

using namespace pm;

extern "C" {

size_t pm_k_swiglu_ffn_static_capacity(void) { return kStaticScratchBytes; }

int pm_k_swiglu_ffn_static(const pm_ffn_group* groups, int n_groups, const void* x, int hidden,
                           const int32_t* row_token, int n_rows, float* yexp, void* stream) {
  if (n_groups < 0 || n_rows < 0) return fail(PM_ERR_INVALID, "swiglu_ffn_static: negative size");
  if (n_groups == 0 || n_rows == 0) return PM_OK;
  if (!groups || !x || !row_token || !yexp) return fail(PM_ERR_INVALID, "swiglu_ffn_static: null pointer");
  if (hidden <= 0) return fail(PM_ERR_INVALID, "swiglu_ffn_static: hidden must be positive");
  int rc = refuse_if_capturing((cudaStream_t)stream, "swiglu_ffn_static");
  if (rc != PM_OK) return rc;
  for (int i = 0; i < n_groups; ++i) {
    if (groups[i].row_count <= 0) continue;
    if (groups[i].row_start < 0 || groups[i].row_start + groups[i].row_count > n_rows)
      return fail(PM_ERR_INVALID, "swiglu_ffn_static: group rows outside [0, n_rows)");
    if (groups[i].q_gate || groups[i].q_up || groups[i].q_down)
      return fail(PM_ERR_INVALID, "swiglu_ffn_static: bf16 experts only (a group carries scale/zero tensors)");
  }
  FfnPlanInfo info;
  rc = plan_groups_size(groups, n_groups, hidden, &info);
  if (rc != PM_OK) return rc;
  if (info.n_desc == 0) return PM_OK;
  const size_t plan_bytes = align_up(info.blob_bytes(), 256);
  const size_t rows_bytes = align_up((size_t)n_rows * info.max_inter * 2, 256);
  if (info.blob_bytes() > kStaticPlanBytes || plan_bytes + rows_bytes > kStaticScratchBytes) {
    char msg[256];
    std::snprintf(msg, sizeof(msg),
                  "swiglu_ffn_static: this launch needs %zu bytes of scratch (plan %zu), the built-in array holds %zu "
                  "(plan at most %zu); use pm_k_swiglu_ffn with caller scratch",
                  plan_bytes + rows_bytes, info.blob_bytes(), kStaticScratchBytes, kStaticPlanBytes);
    return fail(PM_ERR_INVALID, msg);
  }
  unsigned char* scratch = nullptr;
  rc = scratch_address(&scratch);
  if (rc != PM_OK) return rc;
  alignas(16) unsigned char plan[kStaticPlanBytes];  // host stack: no device allocation on this path
  rc = plan_groups_into(groups, n_groups, hidden, plan, sizeof(plan), &info);
  if (rc != PM_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  // Pageable source: the bytes are staged before the call returns, so `plan` may leave scope.
  PM_CUDA(cudaMemcpyAsync(scratch, plan, info.blob_bytes(), cudaMemcpyHostToDevice, s));
  __nv_bfloat16* hbuf = reinterpret_cast<__nv_bfloat16*>(scratch + plan_bytes);
  PM_CUDA(launch_swiglu_ffn(scratch, info, 0, (const __nv_bfloat16*)x, hidden, row_token, hbuf, info.max_inter,
                            yexp, s));
  return PM_OK;
}

}  // extern "C"
