// Allocation-free C entry point for the quadrature-weighted Lp-norm reduction.
//
// This entry point has no counterpart in the reference implementation.  It exists for host programs that
// embed this library but own all device memory themselves: a serving process or a C/Fortran forecast driver
// that reserves the whole GPU for its own pools at start-up (so a later cudaMalloc from a library would fail
// or fragment their arena), or a latency-critical verification loop in which an allocator call - which may
// synchronise the device - is not acceptable.  Such callers pass finished device buffers for the inputs and
// the output; the reduction's scratch space lives in a fixed device array that is part of the library image.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch array in floats (256 KiB per GPU that loads the library, held until exit).
// A call needs planes * ceil(H*W / 65536) * 2 + planes floats.
#define MK_NOALLOC_SCRATCH_FLOATS 65536

// out[plane] = (sum_hw q[h] |pred - tgt|^P, sum_hw q[h] |tgt|^P) for planes = B*C contiguous [H, W] fields.
//   pred, tgt : device pointers, fp32 (is_f32 != 0) or bf16, each planes*H*W elements
//   qlat      : device pointer, H fp32 latitude weights (longitude element folded in)
//   out       : device pointer, planes*2 fp32
//   P         : 1 or 2
// Returns 0 on success, a negative code otherwise (see mk_noalloc_last_error()):
//   -1 bad argument, -2 the problem needs more scratch than MK_NOALLOC_SCRATCH_FLOATS, -3 CUDA error.
//
// Behaviour to know about:
//   * Nothing is allocated or freed, by this function or by anything it calls.
//   * The first call on each device looks up the device address of the scratch array (one
//     cudaGetSymbolAddress with that device current).  Make that first call outside any stream capture.
//   * All calls on a device share the one scratch array.  The completion counters in it are cleared on the
//     stream before every launch, so stale contents of an earlier call never matter, but two calls that
//     overlap on the GPU (different streams, no dependency) race on it: serialise them.
int mk_lp_norms_noalloc(const void* pred, const void* tgt, int is_f32, const float* qlat, float* out, int planes, int H,
                        int W, int P, cudaStream_t stream);

// Message describing the last failure of mk_lp_norms_noalloc on the calling thread ("" if none).
const char* mk_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
