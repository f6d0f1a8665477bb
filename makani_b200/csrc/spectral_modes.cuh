// Mode-wise complex contractions ("diagonal" and "separable" spectral operators); complex64 tensors are passed as
// interleaved (re, im) floats.  See spectral_modes.cu.
#pragma once
#include <cuda_runtime.h>

namespace mk {

// a [B, I, S], w [I, O, S], out [B, O, S]
cudaError_t modes_diag_fwd(const float* a, const float* w, float* out, int B, int I, int O, long long S, cudaStream_t st);
// dy [B, O, S], w [I, O, S], da [B, I, S]
cudaError_t modes_diag_dgrad(const float* dy, const float* w, float* da, int B, int I, int O, long long S, cudaStream_t st);
// a [B, I, S], dy [B, O, S], dw [I, O, S]
cudaError_t modes_diag_wgrad(const float* a, const float* dy, float* dw, int B, int I, int O, long long S, cudaStream_t st);
// out[b, i, s] = a[b, i, s] * w[i, s / wdiv] (or * conj(w) when conj_w); w [I, S / wdiv]
cudaError_t modes_sep_mul(const float* a, const float* w, float* out, int B, int I, long long S, int wdiv, int conj_w, cudaStream_t st);
// dw[i, s'] = sum_b sum_{s / wdiv == s'} conj(a[b, i, s]) dy[b, i, s]
cudaError_t modes_sep_wgrad(const float* a, const float* dy, float* dw, int B, int I, long long S, int wdiv, cudaStream_t st);

}  // namespace mk
