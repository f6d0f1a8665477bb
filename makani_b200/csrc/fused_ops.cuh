// Launchers for the memory-bound fused kernels (normalisation, loss, optimiser, weight re-layout).
// All take raw device pointers and a stream; none allocates.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace mk {

// number of SMs of the current device
int sm_count();

// ---- instance norm over the last `hw` elements of each of `planes` = B*C rows (channel = plane % C) ----
// stats: [planes, 2] fp32 (mean, rstd) written by fwd, read by bwd.  act: 0 none, 1 GELU applied after the affine.
// If `ext_stats` is non-zero the forward skips the reduction and uses the (mean, rstd) already in `stats`
// (used by the spatially distributed norm after the cross-rank merge).
cudaError_t inorm_fwd(const __nv_bfloat16* x, __nv_bfloat16* y, const float* w, const float* b, float* stats,
                      int planes, int C, long long hw, float eps, int act, int ext_stats, cudaStream_t s);
// partial statistics only: sums[plane] = (sum, sum of squares) in fp32
cudaError_t inorm_partial_stats(const __nv_bfloat16* x, float* sums, int planes, long long hw, cudaStream_t s);
// bwd: dx, and atomically accumulated dw[C], db[C].  `sums_io` [planes,2]: when ext_sums == 0 the kernel
// computes (sum g, sum g*xhat) itself; when ext_sums == 1 it only computes them (phase 1) and returns;
// when ext_sums == 2 it reads merged sums from sums_io and does phase 2 with `count` = global element count.
cudaError_t inorm_bwd(const __nv_bfloat16* x, const __nv_bfloat16* dy, __nv_bfloat16* dx, const float* w,
                      const float* b, const float* stats, float* dw, float* db, float* sums_io, int planes, int C,
                      long long hw, double count, int act, int ext_sums, cudaStream_t s);

// ---- cross-device exchange of the partial sums of a spatially sharded instance norm (peer memory, one node) ----
// Producer side (sums kernel): the last CTA to finish waits (bounded) until `wait[p] >= *wait_exp + wait_off` for all
// peers, stores the [B, C, 2] sums into `dst[q]` (this rank's segment in every rank's buffer), bumps `bump` and
// increments `sig[p]` on every peer.  Consumer side (apply kernel): every CTA waits the same way, sums the `nsrc`
// segments found at `src + q * src_stride`, and the last CTA bumps / signals.  All counters are monotonic.
struct StatExchange {
  int npeers;                      // 0: no exchange (single device or host-side reduction)
  const unsigned int* wait;
  const unsigned int* wait_exp;
  int wait_off;
  unsigned int* bump;
  unsigned int* sig[8];
  unsigned int* done_ctr;
  int* err;
  float* dst[8];                   // producer: destinations (ndst)
  int ndst;
  const float* src;                // consumer: base of segment 0 in the local buffer
  long long src_stride;            // floats between segments
  int nsrc;
};

// ---- instance norm on channels-last data x[B, T, C] (C contiguous, C % 8 == 0, C <= 1024) ----
// sums: [B, C, 2] fp32, zero-initialised by the caller, accumulated atomically.
//   mode 0: (sum x, sum x^2);   mode 1: (sum g, sum g*xhat), also accumulated over B into dw / db.
cudaError_t inorm_cl_sums(const __nv_bfloat16* x, const __nv_bfloat16* dy, const float* w, const float* b, const float* stats,
                          float* sums, float* dw, float* db, int B, int C, long long T, int act, int mode, cudaStream_t s,
                          const StatExchange* xch = nullptr);
// mode 0: out = act(xhat * w + b) with statistics from `sums` over `count` elements (stats [B, C, 2] written);
// mode 1: out = dx from the merged backward sums.
cudaError_t inorm_cl_apply(const __nv_bfloat16* x, const __nv_bfloat16* dy, __nv_bfloat16* out, const float* w, const float* b,
                           const float* sums, float* stats, int B, int C, long long T, double count, float eps, int act, int mode,
                           cudaStream_t s, const StatExchange* xch = nullptr);

// ---- quadrature-weighted Lp norms on the sphere ----
// out[plane] = (sum_hw q[h] |p-t|^P, sum_hw q[h] |t|^P), P in {1,2}.  `scratch` holds
// planes*chunks*2 floats + planes ints (zero-initialised once; the kernel leaves the counters at zero).
int lp_norms_chunks(long long hw);
cudaError_t lp_norms(const void* pred, const void* tgt, int is_f32, const float* qlat, float* out, float* scratch,
                     int planes, int H, int W, int P, cudaStream_t s);
// grad[plane, h, w] = coef[plane] * q[h] * d|p-t|^P/dp   (written in the dtype of pred)
cudaError_t lp_norms_bwd(const void* pred, const void* tgt, int is_f32, const float* qlat, const float* coef,
                         void* grad, int planes, int H, int W, int P, cudaStream_t s);

// ---- fused multi-tensor AdamW ----
struct AdamEntry {
  float* p;
  const float* g;
  float* m;
  float* v;
  __nv_bfloat16* shadow;   // optional bf16 copy of the updated parameter (may be null)
  long long n;
  float wd_scale;          // 1 = apply weight decay, 0 = no decay for this tensor
  int pair_mode;           // 1: elements are (re, im) pairs sharing one second moment |g|^2
};
// hyper (device, fp32[8]): lr, beta1, beta2, eps, weight_decay, step, grad_scale, adamw(1)/adam-L2(0)
// err (optional): the device error word; the update is skipped while it is non-zero
cudaError_t adamw_step(const AdamEntry* table, const int* chunk_tensor, const long long* chunk_off, int nchunks,
                       long long chunk, const float* hyper, const int* err, cudaStream_t s);

// ---- spectral weight re-layout ----
// w: complex64 [Cin, Cout, L] (interleaved) -> wx: bf16 [L, 2*Cout, 2*Cin] real 2x2-block form
cudaError_t spectral_expand(const float* w, __nv_bfloat16* wx, int Cin, int Cout, int L, cudaStream_t s);
// dwx: fp32 [L, 2*Cout, 2*Cin] (two_block 0) or [2][L][Cout][Cin] = (dWr, dWi) (two_block 1)
//   -> dw (complex64 [Cin, Cout, L]) += fold(dwx), or = fold(dwx) when `assign`
cudaError_t spectral_fold(const float* dwx, float* dw, int Cin, int Cout, int L, cudaStream_t s, int two_block = 0,
                          int assign = 0);

// rows of (re[C], im[C]) -> (im[C], -re[C]) (bf16, C % 8 == 0): the operand of the imaginary-part weight gradient
cudaError_t swap_ri_bf16(const __nv_bfloat16* in, __nv_bfloat16* out, long long rows, int C, cudaStream_t s);

// ---- small elementwise helpers ----
cudaError_t cast_f32_bf16(const float* x, __nv_bfloat16* y, long long n, cudaStream_t s);
cudaError_t fill_normal_bf16(__nv_bfloat16* y, long long n, uint64_t seed, cudaStream_t s);

}  // namespace mk
