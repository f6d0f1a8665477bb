// GELU and its derivative for the fused epilogues and the normalisation kernels.
//   exact form (default)  : 0.5 x (1 + erf(x / sqrt 2)), the definition of torch.nn.GELU()
//   tanh form (opt-in)    : 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) on the hardware tanh.approx instruction,
//                           i.e. torch.nn.GELU(approximate="tanh"); about a third of the instructions
// Which one runs is a process-wide setting (mk::set_gelu_tanh) that every launcher reads and passes to its kernel, so
// forward and backward of one model always use the same function.
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

__device__ __forceinline__ float gelu_fwd(float x, int tanh_form) {
  const float hx = 0.5f * x;
  if (tanh_form) return fmaf(hx, gelu_tanh_approx(x * fmaf(x * x, 0.0356774081f, 0.7978845608f)), hx);
  return fmaf(hx, erff(x * 0.70710678118654752f), hx);
}

__device__ __forceinline__ float gelu_bwd(float x, int tanh_form) {
  const float x2 = x * x;
  if (tanh_form) {
    const float t = gelu_tanh_approx(x * fmaf(x2, 0.0356774081f, 0.7978845608f));
    return fmaf(0.5f * x * fmaf(-t, t, 1.0f), fmaf(x2, 0.1070322243f, 0.7978845608f), fmaf(0.5f, t, 0.5f));
  }
  // Phi(x) + x phi(x)
  const float cdf = fmaf(0.5f, erff(x * 0.70710678118654752f), 0.5f);
  return fmaf(x * 0.39894228040143268f, __expf(-0.5f * x2), cdf);
}

// Activation codes of the GEMM epilogue.  Odd codes act on the value itself (then an optional residual is added); even
// codes multiply the value by the derivative of the matching activation, evaluated at the epilogue operand:
//   1 GELU(x)               2 x * GELU'(aux)          aux = saved pre-activation
//   3 max(x, 0)             4 x * [aux > 0]           aux = saved OUTPUT of the ReLU
//   5 softshrink(x, param)  6 x * [aux != 0]          aux = saved OUTPUT of the soft shrinkage
__device__ __forceinline__ float act_fwd(float x, int act, float param, int tanh_form) {
  if (act == 1) return gelu_fwd(x, tanh_form);
  if (act == 3) return fmaxf(x, 0.f);
  if (act == 5) return x > param ? x - param : (x < -param ? x + param : 0.f);
  return x;
}
__device__ __forceinline__ float act_bwd(float aux, int act, int tanh_form) {
  if (act == 2) return gelu_bwd(aux, tanh_form);
  if (act == 4) return aux > 0.f ? 1.f : 0.f;
  if (act == 6) return aux != 0.f ? 1.f : 0.f;
  return 1.f;
}

}  // namespace mk
