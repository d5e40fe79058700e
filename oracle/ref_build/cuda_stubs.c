/* Host-only stand-ins for the CUDA runtime / driver entry points that the reference's
 * cpp_worker sources reference. TEST INFRASTRUCTURE ONLY: they let the reference's cache,
 * policy and scheduler classes be driven on a machine without a GPU. Every call "succeeds";
 * device memory is ordinary host memory that is never read. Nothing here is part of the
 * product library. */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

typedef int cudaError_t;
typedef int CUresult;
typedef unsigned long long CUdeviceptr;
typedef unsigned long long CUmemGenericAllocationHandle;

cudaError_t cudaSetDevice(int d) { (void)d; return 0; }
cudaError_t cudaGetDevice(int* d) { *d = 0; return 0; }
cudaError_t cudaEventCreateWithFlags(void** e, unsigned f) { (void)f; *e = malloc(8); return 0; }
cudaError_t cudaEventCreate(void** e) { *e = malloc(8); return 0; }
cudaError_t cudaEventRecord(void* e, void* s) { (void)e; (void)s; return 0; }
cudaError_t cudaEventSynchronize(void* e) { (void)e; return 0; }
cudaError_t cudaEventDestroy(void* e) { free(e); return 0; }
cudaError_t cudaStreamCreateWithFlags(void** s, unsigned f) { (void)f; *s = malloc(8); return 0; }
cudaError_t cudaStreamSynchronize(void* s) { (void)s; return 0; }
cudaError_t cudaMalloc(void** p, size_t n) { *p = malloc(n ? n : 1); return 0; }
cudaError_t cudaFree(void* p) { free(p); return 0; }
cudaError_t cudaMemset(void* p, int v, size_t n) { (void)p; (void)v; (void)n; return 0; }
cudaError_t cudaMemcpyAsync(void* d, const void* s, size_t n, int k, void* st) { (void)d; (void)s; (void)n; (void)k; (void)st; return 0; }
cudaError_t cudaMemcpy(void* d, const void* s, size_t n, int k) { (void)d; (void)s; (void)n; (void)k; return 0; }
cudaError_t cudaMallocManaged(void** p, size_t n, unsigned f) { (void)f; *p = malloc(n ? n : 1); return 0; }
cudaError_t cudaMemAdvise(const void* p, size_t n, int a, int d) { (void)p; (void)n; (void)a; (void)d; return 0; }
cudaError_t cudaMemGetInfo(size_t* f, size_t* t) { *f = *t = (size_t)1 << 34; return 0; }
cudaError_t cudaDeviceSynchronize(void) { return 0; }
cudaError_t cudaGetLastError(void) { return 0; }
const char* cudaGetErrorString(cudaError_t e) { (void)e; return "stub"; }

CUresult cuGetErrorString(CUresult e, const char** s) { (void)e; if (s) *s = "stub"; return 0; }
CUresult cuMemGetAllocationGranularity(size_t* g, const void* prop, int opt) { (void)prop; (void)opt; *g = 2u << 20; return 0; }
CUresult cuMemCreate(CUmemGenericAllocationHandle* h, size_t n, const void* p, unsigned long long f) { (void)n; (void)p; (void)f; *h = 1; return 0; }
CUresult cuMemAddressReserve(CUdeviceptr* p, size_t n, size_t a, CUdeviceptr addr, unsigned long long f) { (void)a; (void)addr; (void)f; *p = (CUdeviceptr)(size_t)malloc(n ? n : 1); return 0; }
CUresult cuMemMap(CUdeviceptr p, size_t n, size_t o, CUmemGenericAllocationHandle h, unsigned long long f) { (void)p; (void)n; (void)o; (void)h; (void)f; return 0; }
CUresult cuMemSetAccess(CUdeviceptr p, size_t n, const void* d, size_t c) { (void)p; (void)n; (void)d; (void)c; return 0; }
CUresult cuMemUnmap(CUdeviceptr p, size_t n) { (void)p; (void)n; return 0; }
CUresult cuMemRelease(CUmemGenericAllocationHandle h) { (void)h; return 0; }
CUresult cuMemAddressFree(CUdeviceptr p, size_t n) { (void)p; (void)n; return 0; }

/* cuBLAS: referenced once by the reference's PrefetchMngr constructor, which the harness never runs. */
int cublasSetStream_v2(void* handle, void* stream) { (void)handle; (void)stream; return 0; }
