// Allocation-free variant of the Lp-norm reduction: same kernels as mk::lp_norms, scratch in a static device array.
#include "no_alloc.h"

#include <mutex>
#include <stdio.h>

#include "fused_ops.cuh"

namespace {

// Partial sums (planes * chunks * 2 floats) followed by one completion counter per plane.  Zero-initialised when the
// module is loaded on a device; every GPU that loads the library holds its own copy until the process exits.
static __device__ __align__(256) float g_noalloc_scratch[MK_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};   // device addresses, looked up once per device
std::mutex g_setup_mutex;
thread_local char g_msg[256] = {0};

int fail(int code, const char* what, cudaError_t e = cudaSuccess) {
  if (e != cudaSuccess) snprintf(g_msg, sizeof(g_msg), "%s: %s", what, cudaGetErrorString(e));
  else snprintf(g_msg, sizeof(g_msg), "%s", what);
  return code;
}

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address: the address a kernel can
// use has to be asked for, per device, with that device current.
int scratch_for_current_device(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(-3, "cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail(-1, "device index out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return fail(-3, "cudaGetSymbolAddress(scratch)", e);
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *ptr = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" const char* mk_noalloc_last_error(void) { return g_msg; }

extern "C" int mk_lp_norms_noalloc(const void* pred, const void* tgt, int is_f32, const float* qlat, float* out, int planes,
                                   int H, int W, int P, cudaStream_t stream) {
  g_msg[0] = 0;
  if (!pred || !tgt || !qlat || !out) return fail(-1, "null pointer argument");
  if (planes <= 0 || H <= 0 || W <= 0) return fail(-1, "planes, H and W must be positive");
  if (P != 1 && P != 2) return fail(-1, "P must be 1 or 2");
  const long long hw = static_cast<long long>(H) * W;
  const long long chunks = mk::lp_norms_chunks(hw);
  const long long need = static_cast<long long>(planes) * chunks * 2 + planes;
  if (need > MK_NOALLOC_SCRATCH_FLOATS) {
    snprintf(g_msg, sizeof(g_msg),
             "problem needs %lld scratch floats (planes %d x chunks %lld x 2 + planes) but the built-in scratch holds %d; "
             "split the call over fewer planes",
             need, planes, chunks, MK_NOALLOC_SCRATCH_FLOATS);
    return -2;
  }
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // the completion counters must start at zero whatever an earlier (possibly interrupted) call left behind
  cudaError_t e = cudaMemsetAsync(scratch + static_cast<long long>(planes) * chunks * 2, 0, sizeof(int) * planes, stream);
  if (e != cudaSuccess) return fail(-3, "cudaMemsetAsync(counters)", e);
  e = mk::lp_norms(pred, tgt, is_f32, qlat, out, scratch, planes, H, W, P, stream);
  if (e != cudaSuccess) return fail(-3, "lp_norms launch", e);
  return 0;
}
