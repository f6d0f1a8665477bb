// GELU and its derivative for the fused epilogues and the normalisation kernels.
//
//   default ("erf form")  : 0.5 x (1 + erf(x / sqrt 2)), the definition of torch.nn.GELU().  These epilogues have a
//                           budget of about a dozen instructions per output element (a 128x256 tile with K = 384 is
//                           done by the tensor cores in 3072 cycles), so erf is not evaluated with erff() (that
//                           doubled the time of the GELU GEMMs) but through the identity
//                           erf(x / sqrt 2) ~= tanh(x (c0 + c1 x^2 + c2 x^4)), a minimax fit of the argument whose
//                           normal-CDF error is below 1.9e-5 everywhere (|GELU error| < 5.5e-5), on the hardware
//                           tanh.approx instruction (relative error 2^-11 on the tanh value).  Both terms are far
//                           below the 2^-8 relative spacing of the bf16 activations the result is rounded to.
//   tanh form (opt-in)    : 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), i.e. torch.nn.GELU(approximate="tanh"),
//                           which deviates from the erf form by up to 4.7e-4.
//
// The derivative is that of the function actually evaluated, so forward and backward are consistent.  Which form runs
// is a process-wide setting (mk::set_gelu_tanh) that every launcher reads and passes to its kernel.
#pragma once
#include <cuda_runtime.h>

namespace mk {

// 0: exact erf form, 1: tanh approximation
void set_gelu_tanh(int on);
int gelu_tanh();

__device__ __forceinline__ float gelu_tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Both forms are 0.5 x (1 + tanh(x q(x^2))) with q(u) = c0 + c1 u + c2 u^2; a launcher passes the coefficients of the
// selected form to its kernel, so the device code has no branch on the form.
struct GeluCoef {
  float c0, c1, c2;
};
inline GeluCoef gelu_coef(int tanh_form) {
  if (tanh_form) return GeluCoef{0.7978845608f, 0.0356774081f, 0.f};
  return GeluCoef{0.797717881f, 0.0367982429f, -3.15818913e-4f};
}

// x^2 is clamped at 36: beyond |x| = 6 the tanh is 1 to fp32 precision, and the fitted q (c2 < 0) must not be
// followed to where it turns negative (|x| > 11)
__device__ __forceinline__ float gelu_fwd(float x, const GeluCoef& c) {
  const float u = fminf(x * x, 36.f);
  const float q = fmaf(u, fmaf(u, c.c2, c.c1), c.c0);
  const float hx = 0.5f * x;
  return fmaf(hx, gelu_tanh_approx(x * q), hx);
}

__device__ __forceinline__ float gelu_bwd(float x, const GeluCoef& c) {
  const float u = fminf(x * x, 36.f);
  const float q = fmaf(u, fmaf(u, c.c2, c.c1), c.c0);
  const float dq = fmaf(u, fmaf(u, 5.f * c.c2, 3.f * c.c1), c.c0);   // d(x q(x^2))/dx
  const float t = gelu_tanh_approx(x * q);
  return fmaf(0.5f * x * fmaf(-t, t, 1.0f), dq, fmaf(0.5f, t, 0.5f));
}

// GELU and its derivative at the same point (shared polynomial and tanh): the forward epilogue that saves the
// derivative for the backward pass pays six more instructions than the plain forward.
__device__ __forceinline__ void gelu_fwd_bwd(float x, const GeluCoef& c, float& y, float& dy) {
  const float u = fminf(x * x, 36.f);
  const float q = fmaf(u, fmaf(u, c.c2, c.c1), c.c0);
  const float dq = fmaf(u, fmaf(u, 5.f * c.c2, 3.f * c.c1), c.c0);
  const float t = gelu_tanh_approx(x * q);
  const float hx = 0.5f * x;
  y = fmaf(hx, t, hx);
  dy = fmaf(hx * fmaf(-t, t, 1.0f), dq, fmaf(0.5f, t, 0.5f));
}

// Activation codes of the GEMM epilogue.  Odd codes act on the value itself (then an optional residual is added); even
// codes multiply the value by the derivative of the matching activation, evaluated at the epilogue operand:
//   1 GELU(x)               2 x * GELU'(aux)          aux = saved pre-activation
//   3 max(x, 0)             4 x * [aux > 0]           aux = saved OUTPUT of the ReLU
//   5 softshrink(x, param)  6 x * [aux != 0]          aux = saved OUTPUT of the soft shrinkage
//                           8 x * aux                 aux = derivative saved by the forward pass
__device__ __forceinline__ float act_fwd(float x, int act, float param, const GeluCoef& gc) {
  if (act == 1) return gelu_fwd(x, gc);
  if (act == 3) return fmaxf(x, 0.f);
  if (act == 5) return x > param ? x - param : (x < -param ? x + param : 0.f);
  return x;
}
__device__ __forceinline__ float act_bwd(float aux, int act, const GeluCoef& gc) {
  if (act == 2) return gelu_bwd(aux, gc);
  if (act == 4) return aux > 0.f ? 1.f : 0.f;
  if (act == 6) return aux != 0.f ? 1.f : 0.f;
  if (act == 8) return aux;
  return 1.f;
}

}  // namespace mk
