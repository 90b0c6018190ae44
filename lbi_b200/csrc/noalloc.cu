// RMSNorm weight gradient with a library-owned workspace (see noalloc.h for the contract).
#include "noalloc.h"

#include "api.h"

namespace {

// File-scope device array: in host code this name is only a handle for the runtime, not a device address, so it is
// never passed to a kernel directly; setup() asks the runtime for the address that is valid on the current device.
static __device__ __align__(256) float g_workspace[LBI_NOALLOC_BLOCKS * LBI_NOALLOC_MAX_DIM];

constexpr int MAX_DEVICES = 64;
float* g_workspace_ptr[MAX_DEVICES] = {nullptr};

// Once per device, with that device current.
int workspace_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return (int)cudaErrorInvalidDevice;
  if (g_workspace_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_workspace);
    if (e != cudaSuccess) return (int)e;
    g_workspace_ptr[dev] = ptr;
  }
  *out = g_workspace_ptr[dev];
  return 0;
}

}  // namespace

extern "C" int lbi_rmsnorm_wgrad_noalloc(const void* d_normed_bf16, const float* x_stream, const float* rstd, float* dw,
                                         int64_t rows, int dim, cudaStream_t stream) {
  if (dim <= 0 || dim % 8 != 0 || dim > LBI_NOALLOC_MAX_DIM || rows < 0) return (int)cudaErrorInvalidValue;
  if (d_normed_bf16 == nullptr || x_stream == nullptr || rstd == nullptr || dw == nullptr)
    return (int)cudaErrorInvalidValue;
  float* workspace = nullptr;
  int rc = workspace_for_current_device(&workspace);
  if (rc != 0) return rc;
  int nblocks = LBI_NOALLOC_BLOCKS;
  if (rows < nblocks) nblocks = rows > 0 ? (int)rows : 1;
  // Stage 1 writes partials[0 .. nblocks) x [0 .. dim) in full before stage 2 reads exactly that range.
  return lbi_rmsnorm_wgrad(d_normed_bf16, x_stream, rstd, workspace, dw, rows, dim, nblocks, stream);
}
