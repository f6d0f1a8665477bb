// Mode-wise complex contractions of the spectral filters whose weights differ per (l, m) mode ("diagonal" operator)
// or act per channel ("separable"): for every mode a [B, Cin] x [Cin, Cout] complex product.  At batch sizes of one
// or two there is no tile shape for the tensor cores here; the work is streaming the weights once, so these are
// bandwidth kernels: threads run along the mode index (the contiguous one in activations and weights), every weight
// element is read exactly once per batch sample and the activations of a block of modes are re-read from L2.
//
//   diag fwd : out[b, o, s] = sum_i a[b, i, s] w[i, o, s]
//   diag dA  : da[b, i, s]  = sum_o dy[b, o, s] conj(w[i, o, s])
//   diag dW  : dw[i, o, s]  = sum_b conj(a[b, i, s]) dy[b, o, s]
//   separable: out[b, i, s] = a[b, i, s] w[i, s'] with s' = s ("diagonal") or s' = s / M (per degree, "dhconv")
#include "spectral_modes.cuh"

namespace mk {

namespace {

__device__ __forceinline__ float2 cmul(float2 a, float2 b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }
__device__ __forceinline__ float2 cmulc(float2 a, float2 b) {   // a * conj(b)
  return make_float2(a.x * b.x + a.y * b.y, a.y * b.x - a.x * b.y);
}
__device__ __forceinline__ void cfma(float2& acc, float2 a, float2 b) {
  acc.x = fmaf(a.x, b.x, fmaf(-a.y, b.y, acc.x));
  acc.y = fmaf(a.x, b.y, fmaf(a.y, b.x, acc.y));
}
__device__ __forceinline__ void cfmac(float2& acc, float2 a, float2 b) {   // acc += a * conj(b)
  acc.x = fmaf(a.x, b.x, fmaf(a.y, b.y, acc.x));
  acc.y = fmaf(a.y, b.x, fmaf(-a.x, b.y, acc.y));
}

constexpr int TS = 128;   // modes per CTA
constexpr int TO = 4;     // output channels per thread (the activations of a mode are loaded once for four outputs)

// grid (ceil(S / TS), ceil(O / TO), B)
__global__ void __launch_bounds__(TS) diag_fwd_kernel(const float2* __restrict__ a, const float2* __restrict__ w,
                                                      float2* __restrict__ out, int I, int O, long long S) {
  const long long s = static_cast<long long>(blockIdx.x) * TS + threadIdx.x;
  const int o0 = blockIdx.y * TO, b = blockIdx.z;
  if (s >= S) return;
  float2 acc[TO];
#pragma unroll
  for (int j = 0; j < TO; ++j) acc[j] = make_float2(0.f, 0.f);
  const float2* ap = a + static_cast<long long>(b) * I * S + s;
  for (int i = 0; i < I; ++i) {
    const float2 av = ap[static_cast<long long>(i) * S];
    const float2* wp = w + (static_cast<long long>(i) * O + o0) * S + s;
#pragma unroll
    for (int j = 0; j < TO; ++j)
      if (o0 + j < O) cfma(acc[j], av, __ldcs(wp + static_cast<long long>(j) * S));
  }
#pragma unroll
  for (int j = 0; j < TO; ++j)
    if (o0 + j < O) out[(static_cast<long long>(b) * O + o0 + j) * S + s] = acc[j];
}

// da[b, i, s] = sum_o dy[b, o, s] conj(w[i, o, s]); grid (ceil(S / TS), ceil(I / TO), B)
__global__ void __launch_bounds__(TS) diag_dgrad_kernel(const float2* __restrict__ dy, const float2* __restrict__ w,
                                                        float2* __restrict__ da, int I, int O, long long S) {
  const long long s = static_cast<long long>(blockIdx.x) * TS + threadIdx.x;
  const int i0 = blockIdx.y * TO, b = blockIdx.z;
  if (s >= S) return;
  float2 acc[TO];
#pragma unroll
  for (int j = 0; j < TO; ++j) acc[j] = make_float2(0.f, 0.f);
  const float2* gp = dy + static_cast<long long>(b) * O * S + s;
  for (int o = 0; o < O; ++o) {
    const float2 gv = gp[static_cast<long long>(o) * S];
#pragma unroll
    for (int j = 0; j < TO; ++j)
      if (i0 + j < I) cfmac(acc[j], gv, __ldcs(w + (static_cast<long long>(i0 + j) * O + o) * S + s));
  }
#pragma unroll
  for (int j = 0; j < TO; ++j)
    if (i0 + j < I) da[(static_cast<long long>(b) * I + i0 + j) * S + s] = acc[j];
}

// dw[i, o, s] = sum_b conj(a[b, i, s]) dy[b, o, s]; grid (ceil(S / TS), O, I)
__global__ void __launch_bounds__(TS) diag_wgrad_kernel(const float2* __restrict__ a, const float2* __restrict__ dy,
                                                        float2* __restrict__ dw, int B, int I, int O, long long S) {
  const long long s = static_cast<long long>(blockIdx.x) * TS + threadIdx.x;
  const int o = blockIdx.y, i = blockIdx.z;
  if (s >= S) return;
  float2 acc = make_float2(0.f, 0.f);
  for (int b = 0; b < B; ++b)
    cfmac(acc, dy[(static_cast<long long>(b) * O + o) * S + s], a[(static_cast<long long>(b) * I + i) * S + s]);
  __stcs(dw + (static_cast<long long>(i) * O + o) * S + s, acc);
}

// separable: grid (ceil(S / TS), I, B); wdiv = 1 (weight per mode) or M (weight per degree, s' = s / M)
__global__ void __launch_bounds__(TS) sep_mul_kernel(const float2* __restrict__ a, const float2* __restrict__ w,
                                                     float2* __restrict__ out, int I, long long S, int wdiv, int conj_w) {
  const long long s = static_cast<long long>(blockIdx.x) * TS + threadIdx.x;
  const int i = blockIdx.y, b = blockIdx.z;
  if (s >= S) return;
  const long long ws = S / wdiv;
  const float2 wv = w[static_cast<long long>(i) * ws + s / wdiv];
  const float2 av = a[(static_cast<long long>(b) * I + i) * S + s];
  out[(static_cast<long long>(b) * I + i) * S + s] = conj_w ? cmulc(av, wv) : cmul(av, wv);
}

// dw[i, s'] = sum_b sum_{s in s'} conj(a[b, i, s]) dy[b, i, s]; grid (ceil(S' / TS), I); one thread per weight element
__global__ void __launch_bounds__(TS) sep_wgrad_kernel(const float2* __restrict__ a, const float2* __restrict__ dy,
                                                       float2* __restrict__ dw, int B, int I, long long S, int wdiv) {
  const long long ws = S / wdiv;
  const long long sp = static_cast<long long>(blockIdx.x) * TS + threadIdx.x;
  const int i = blockIdx.y;
  if (sp >= ws) return;
  float2 acc = make_float2(0.f, 0.f);
  for (int b = 0; b < B; ++b) {
    const long long base = (static_cast<long long>(b) * I + i) * S + sp * wdiv;
    for (int k = 0; k < wdiv; ++k) cfmac(acc, dy[base + k], a[base + k]);
  }
  dw[static_cast<long long>(i) * ws + sp] = acc;
}

inline unsigned cdiv(long long a, long long b) { return static_cast<unsigned>((a + b - 1) / b); }

}  // namespace

cudaError_t modes_diag_fwd(const float* a, const float* w, float* out, int B, int I, int O, long long S, cudaStream_t st) {
  if (B <= 0 || I <= 0 || O <= 0 || S <= 0) return cudaSuccess;
  diag_fwd_kernel<<<dim3(cdiv(S, TS), cdiv(O, TO), B), TS, 0, st>>>(reinterpret_cast<const float2*>(a), reinterpret_cast<const float2*>(w),
                                                                     reinterpret_cast<float2*>(out), I, O, S);
  return cudaGetLastError();
}

cudaError_t modes_diag_dgrad(const float* dy, const float* w, float* da, int B, int I, int O, long long S, cudaStream_t st) {
  if (B <= 0 || I <= 0 || O <= 0 || S <= 0) return cudaSuccess;
  diag_dgrad_kernel<<<dim3(cdiv(S, TS), cdiv(I, TO), B), TS, 0, st>>>(reinterpret_cast<const float2*>(dy), reinterpret_cast<const float2*>(w),
                                                                       reinterpret_cast<float2*>(da), I, O, S);
  return cudaGetLastError();
}

cudaError_t modes_diag_wgrad(const float* a, const float* dy, float* dw, int B, int I, int O, long long S, cudaStream_t st) {
  if (I <= 0 || O <= 0 || S <= 0) return cudaSuccess;
  diag_wgrad_kernel<<<dim3(cdiv(S, TS), O, I), TS, 0, st>>>(reinterpret_cast<const float2*>(a), reinterpret_cast<const float2*>(dy),
                                                             reinterpret_cast<float2*>(dw), B, I, O, S);
  return cudaGetLastError();
}

cudaError_t modes_sep_mul(const float* a, const float* w, float* out, int B, int I, long long S, int wdiv, int conj_w, cudaStream_t st) {
  if (B <= 0 || I <= 0 || S <= 0) return cudaSuccess;
  sep_mul_kernel<<<dim3(cdiv(S, TS), I, B), TS, 0, st>>>(reinterpret_cast<const float2*>(a), reinterpret_cast<const float2*>(w),
                                                          reinterpret_cast<float2*>(out), I, S, wdiv, conj_w);
  return cudaGetLastError();
}

cudaError_t modes_sep_wgrad(const float* a, const float* dy, float* dw, int B, int I, long long S, int wdiv, cudaStream_t st) {
  if (I <= 0 || S <= 0) return cudaSuccess;
  sep_wgrad_kernel<<<dim3(cdiv(S / wdiv, TS), I), TS, 0, st>>>(reinterpret_cast<const float2*>(a), reinterpret_cast<const float2*>(dy),
                                                                reinterpret_cast<float2*>(dw), B, I, S, wdiv);
  return cudaGetLastError();
}

}  // namespace mk
