// Memory-bound fused kernels for sm_100a: instance norm (+GELU), quadrature-weighted Lp norms, multi-tensor
// AdamW with bf16 shadow weights, spectral-weight re-layout.  Each kernel makes the minimum number of passes
// over HBM (vectorised 16-byte accesses) and keeps reductions in fp32.
#include "fused_ops.cuh"
#include "gelu.cuh"
#include <cstring>

#include <math.h>

namespace mk {

namespace {
int g_gelu_tanh = 0;
}
void set_gelu_tanh(int on) { g_gelu_tanh = on ? 1 : 0; }
int gelu_tanh() { return g_gelu_tanh; }

// number of SMs of the current device (cached per device index)
int sm_count() {
  static int cache[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cache[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev] = n;
  }
  return cache[dev];
}

namespace {

constexpr int NT = 512;

// act: 0 none, 1 GELU (exact erf form), 2 GELU (tanh form); the launchers map the caller's on/off flag to 1 or 2
// according to the process-wide setting
__device__ __forceinline__ GeluCoef coef_of(int act) {
  return act == 2 ? GeluCoef{0.7978845608f, 0.0356774081f, 0.f} : GeluCoef{0.797717881f, 0.0367982429f, -3.15818913e-4f};
}
__device__ __forceinline__ float gelu_f(float x, int act) { return gelu_fwd(x, coef_of(act)); }
__device__ __forceinline__ float dgelu_f(float x, int act) { return gelu_bwd(x, coef_of(act)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// block-wide sum of two values; result valid in all threads
__device__ __forceinline__ void block_sum2(float& a, float& b) {
  __shared__ float sh[2][32];
  __shared__ float res[2];
  a = warp_sum(a);
  b = warp_sum(b);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) {
    sh[0][w] = a;
    sh[1][w] = b;
  }
  __syncthreads();
  if (w == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    float x = l < nw ? sh[0][l] : 0.f;
    float y = l < nw ? sh[1][l] : 0.f;
    x = warp_sum(x);
    y = warp_sum(y);
    if (l == 0) {
      res[0] = x;
      res[1] = y;
    }
  }
  __syncthreads();
  a = res[0];
  b = res[1];
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 x = __bfloat1622float2(h[j]);
    f[2 * j] = x.x;
    f[2 * j + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  return v;
}

// ------------------------------------------------------------------------------------------ instance norm

// mode 0: full forward; mode 1: partial sums only (sums -> stats[plane] = (sum, sumsq)); mode 2: normalise with given stats
template <bool VEC>
__global__ void __launch_bounds__(NT) inorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                       const float* __restrict__ w, const float* __restrict__ b,
                                                       float* __restrict__ stats, int C, long long hw, float eps, int act,
                                                       int mode) {
  const int plane = blockIdx.x;
  const int c = plane % C;
  const __nv_bfloat16* xp = x + static_cast<long long>(plane) * hw;
  float mean, rstd;
  if (mode != 2) {
    float s = 0.f, ss = 0.f;
    if (VEC) {
      const uint4* xv = reinterpret_cast<const uint4*>(xp);
      const long long nv = hw >> 3;
      for (long long i = threadIdx.x; i < nv; i += NT) {
        float f[8];
        unpack8(xv[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s += f[j];
          ss += f[j] * f[j];
        }
      }
    } else {
      for (long long i = threadIdx.x; i < hw; i += NT) {
        const float f = __bfloat162float(xp[i]);
        s += f;
        ss += f * f;
      }
    }
    block_sum2(s, ss);
    if (mode == 1) {
      if (threadIdx.x == 0) {
        stats[2 * plane] = s;
        stats[2 * plane + 1] = ss;
      }
      return;
    }
    mean = s / static_cast<float>(hw);
    const float var = fmaxf(ss / static_cast<float>(hw) - mean * mean, 0.f);
    rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      stats[2 * plane] = mean;
      stats[2 * plane + 1] = rstd;
    }
  } else {
    mean = stats[2 * plane];
    rstd = stats[2 * plane + 1];
  }
  const float ga = (w ? w[c] : 1.f) * rstd;
  const float be = (b ? b[c] : 0.f) - mean * ga;
  __nv_bfloat16* yp = y + static_cast<long long>(plane) * hw;
  if (VEC) {
    const uint4* xv = reinterpret_cast<const uint4*>(xp);
    uint4* yv = reinterpret_cast<uint4*>(yp);
    const long long nv = hw >> 3;
    for (long long i = threadIdx.x; i < nv; i += NT) {
      float f[8];
      unpack8(xv[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v = f[j] * ga + be;
        f[j] = act ? gelu_f(v, act) : v;
      }
      yv[i] = pack8(f);
    }
  } else {
    for (long long i = threadIdx.x; i < hw; i += NT) {
      float v = __bfloat162float(xp[i]) * ga + be;
      yp[i] = __float2bfloat16(act ? gelu_f(v, act) : v);
    }
  }
}

// phase control: ext 0: both phases; 1: phase 1 only (write sums); 2: phase 2 only (read merged sums)
template <bool VEC>
__global__ void __launch_bounds__(NT) inorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                                       __nv_bfloat16* __restrict__ dx, const float* __restrict__ w,
                                                       const float* __restrict__ b, const float* __restrict__ stats,
                                                       float* __restrict__ dw, float* __restrict__ db, float* __restrict__ sums_io,
                                                       int C, long long hw, float inv_count, int act, int ext) {
  const int plane = blockIdx.x;
  const int c = plane % C;
  const float mean = stats[2 * plane], rstd = stats[2 * plane + 1];
  const float wc = w ? w[c] : 1.f, bc = b ? b[c] : 0.f;
  const __nv_bfloat16* xp = x + static_cast<long long>(plane) * hw;
  const __nv_bfloat16* gp = dy + static_cast<long long>(plane) * hw;
  float s1 = 0.f, s2 = 0.f;
  if (ext != 2) {
    if (VEC) {
      const uint4* xv = reinterpret_cast<const uint4*>(xp);
      const uint4* gv = reinterpret_cast<const uint4*>(gp);
      const long long nv = hw >> 3;
      for (long long i = threadIdx.x; i < nv; i += NT) {
        float f[8], g[8];
        unpack8(xv[i], f);
        unpack8(gv[i], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (f[j] - mean) * rstd;
          float gg = g[j];
          if (act) gg *= dgelu_f(xh * wc + bc, act);
          s1 += gg;
          s2 += gg * xh;
        }
      }
    } else {
      for (long long i = threadIdx.x; i < hw; i += NT) {
        const float xh = (__bfloat162float(xp[i]) - mean) * rstd;
        float gg = __bfloat162float(gp[i]);
        if (act) gg *= dgelu_f(xh * wc + bc, act);
        s1 += gg;
        s2 += gg * xh;
      }
    }
    block_sum2(s1, s2);
    if (threadIdx.x == 0) {
      if (dw) atomicAdd(dw + c, s2);
      if (db) atomicAdd(db + c, s1);
      if (sums_io) {
        sums_io[2 * plane] = s1;
        sums_io[2 * plane + 1] = s2;
      }
    }
    if (ext == 1) return;
  } else {
    s1 = sums_io[2 * plane];
    s2 = sums_io[2 * plane + 1];
  }
  const float m1 = s1 * inv_count, m2 = s2 * inv_count;
  const float sc = rstd * wc;
  __nv_bfloat16* op = dx + static_cast<long long>(plane) * hw;
  if (VEC) {
    const uint4* xv = reinterpret_cast<const uint4*>(xp);
    const uint4* gv = reinterpret_cast<const uint4*>(gp);
    uint4* ov = reinterpret_cast<uint4*>(op);
    const long long nv = hw >> 3;
    for (long long i = threadIdx.x; i < nv; i += NT) {
      float f[8], g[8];
      unpack8(xv[i], f);
      unpack8(gv[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (f[j] - mean) * rstd;
        float gg = g[j];
        if (act) gg *= dgelu_f(xh * wc + bc, act);
        f[j] = sc * (gg - m1 - xh * m2);
      }
      ov[i] = pack8(f);
    }
  } else {
    for (long long i = threadIdx.x; i < hw; i += NT) {
      const float xh = (__bfloat162float(xp[i]) - mean) * rstd;
      float gg = __bfloat162float(gp[i]);
      if (act) gg *= dgelu_f(xh * wc + bc, act);
      op[i] = __float2bfloat16(sc * (gg - m1 - xh * m2));
    }
  }
}

// ------------------------------------------------------------------------------------------ instance norm, channels-last
// x: [B, T, C] with C contiguous (C % 8 == 0, C <= 1024).  Thread (v, r) = (tid % V, tid / V), V = C / 8, owns 8
// channels and walks the tokens r, r + R, ... of its slab, so per-channel constants stay in registers.

constexpr int CL_THREADS = 512;

// mode 0: sums of (x, x^2).  mode 1: sums of (g, g * xhat) with g = dy * act'(xhat * w + b) for the backward pass.
__device__ __forceinline__ unsigned int xch_ld_acquire(const unsigned int* ptr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long xch_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// bounded wait (2 s) of one thread on the peers' flags; false + error word on expiry
__device__ bool xch_wait(const StatExchange& xc, int code) {
  const unsigned int need = *xc.wait_exp + static_cast<unsigned int>(xc.wait_off);
  for (int peer = 0; peer < xc.npeers; ++peer) {
    unsigned long long t0 = 0;
    for (unsigned int it = 0;; ++it) {
      if (static_cast<int>(xch_ld_acquire(xc.wait + peer) - need) >= 0) break;
      if ((it & 255u) == 255u) {
        const unsigned long long now = xch_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > 2000000000ull) {
          atomicExch(xc.err, code);
          return false;
        }
      }
    }
  }
  return true;
}
__device__ void xch_signal(const StatExchange& xc) {
  *xc.done_ctr = 0;
  if (*reinterpret_cast<volatile int*>(xc.err) != 0) return;   // nothing is published after an expired wait
  atomicAdd(xc.bump, 1u);
  __threadfence_system();
  for (int peer = 0; peer < xc.npeers; ++peer)
    if (xc.sig[peer]) atomicAdd_system(xc.sig[peer], 1u);
}

template <int MODE>
__global__ void __launch_bounds__(CL_THREADS) inorm_cl_sums_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                                                   const float* __restrict__ w, const float* __restrict__ b,
                                                                   const float* __restrict__ stats, float* __restrict__ sums,
                                                                   float* __restrict__ dw, float* __restrict__ db, int C, long long T,
                                                                   int act, int slab, int shifted, const StatExchange xc) {
  extern __shared__ float sh_acc[];   // [C][2]
  const int V = C >> 3;
  const int R = CL_THREADS / V;
  const int v = threadIdx.x % V, r = threadIdx.x / V;
  const int bidx = blockIdx.y;
  for (int i = threadIdx.x; i < 2 * C; i += CL_THREADS) sh_acc[i] = 0.f;
  __syncthreads();
  if (r < R) {
    float a0[8], a1[8], mean[8], rstd[8], wc[8], bc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      a0[j] = 0.f;
      a1[j] = 0.f;
      if (MODE == 1) {
        const int c = v * 8 + j;
        mean[j] = stats[(static_cast<long long>(bidx) * C + c) * 2];
        rstd[j] = stats[(static_cast<long long>(bidx) * C + c) * 2 + 1];
        wc[j] = w ? w[c] : 1.f;
        bc[j] = b ? b[c] : 0.f;
      }
    }
    const long long t0 = static_cast<long long>(blockIdx.x) * slab;
    long long t1 = t0 + slab;
    if (t1 > T) t1 = T;
    const uint4* xv = reinterpret_cast<const uint4*>(x + static_cast<long long>(bidx) * T * C) + v;
    const uint4* gv = MODE == 1 ? reinterpret_cast<const uint4*>(dy + static_cast<long long>(bidx) * T * C) + v : nullptr;
    // Shifted sums: sum (x - s) and sum (x - s)^2 with s = the sample's first token, so that the one-pass variance
    // E[(x-s)^2] - E[x-s]^2 does not cancel when |mean| >> std.  (Only when the statistics are local to this device:
    // sums that are merged across ranks need one common shift and stay unshifted.)
    float sft[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) sft[j] = 0.f;
    if (MODE == 0 && shifted) unpack8(xv[0], sft);
    // four rows in flight per thread: independent 16-byte loads cover the HBM latency
    auto accum = [&](const uint4& xr, const uint4& gr) {
      float f[8];
      unpack8(xr, f);
      if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = f[j] - sft[j];
          a0[j] += d;
          a1[j] += d * d;
        }
      } else {
        float g[8];
        unpack8(gr, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (f[j] - mean[j]) * rstd[j];
          float gg = g[j];
          if (act) gg *= dgelu_f(xh * wc[j] + bc[j], act);
          a0[j] += gg;
          a1[j] += gg * xh;
        }
      }
    };
    long long t = t0 + r;
    for (; t + 3LL * R < t1; t += 4LL * R) {
      uint4 xr[4], gr[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        xr[u] = xv[(t + u * R) * V];
        if (MODE == 1) gr[u] = gv[(t + u * R) * V];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) accum(xr[u], gr[u]);
    }
    for (; t < t1; t += R) {
      const uint4 xr = xv[t * V];
      uint4 gr = xr;
      if (MODE == 1) gr = gv[t * V];
      accum(xr, gr);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      atomicAdd(&sh_acc[(v * 8 + j) * 2], a0[j]);
      atomicAdd(&sh_acc[(v * 8 + j) * 2 + 1], a1[j]);
    }
  }
  __syncthreads();
  // one 16-byte vector atomic per two channels (C is a multiple of 8, the buffer is 16-byte aligned)
  for (int i = threadIdx.x * 4; i < 2 * C; i += CL_THREADS * 4) {
    const float4 val = *reinterpret_cast<const float4*>(sh_acc + i);
    atomicAdd(reinterpret_cast<float4*>(sums + static_cast<long long>(bidx) * 2 * C + i), val);
    if (MODE == 1) {
      const int c = i >> 1;
      if (db) {
        atomicAdd(db + c, val.x);
        atomicAdd(db + c + 1, val.z);
      }
      if (dw) {
        atomicAdd(dw + c, val.y);
        atomicAdd(dw + c + 1, val.w);
      }
    }
  }
  if (xc.npeers > 0) {
    // the last CTA of the grid hands this rank's sums to every peer
    __shared__ int last_s;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int prev = atomicAdd(xc.done_ctr, 1u);
      int last = (prev == gridDim.x * gridDim.y - 1) ? 1 : 0;
      if (last && !xch_wait(xc, 56)) last = 2;     // peers still read the previous statistics: give up (error word set)
      last_s = last;
    }
    __syncthreads();
    if (last_s == 1) {
      __threadfence();
      const int n = static_cast<int>(gridDim.y) * 2 * C;
      for (int i = threadIdx.x; i < n; i += CL_THREADS) {
        const float val = __ldcg(sums + i);
        for (int q = 0; q < xc.ndst; ++q) xc.dst[q][i] = val;
      }
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) xch_signal(xc);
    } else if (last_s == 2 && threadIdx.x == 0) {
      *xc.done_ctr = 0;
    }
  }
}

// mode 0: y = act(xhat * w + b), statistics derived from `sums` (and stored to `stats`).
// mode 1: dx = rstd * w * (g - s1/T - xhat * s2/T) with (s1, s2) in `sums`, (mean, rstd) in `stats`.
template <int MODE>
__global__ void __launch_bounds__(CL_THREADS) inorm_cl_apply_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                                                    __nv_bfloat16* __restrict__ out, const float* __restrict__ w,
                                                                    const float* __restrict__ b, const float* __restrict__ sums,
                                                                    float* __restrict__ stats, int C, long long T, float inv_count,
                                                                    float eps, int act, int slab, int shifted, const StatExchange xc) {
  const int V = C >> 3;
  const int R = CL_THREADS / V;
  const int v = threadIdx.x % V, r = threadIdx.x / V;
  const int bidx = blockIdx.y;
  extern __shared__ float sh_sum[];   // [C][2] merged sums of this sample (exchange mode only)
  if (xc.npeers > 0) {
    // every peer's sums must have arrived in the local buffer
    __shared__ int ok_s;
    if (threadIdx.x == 0) ok_s = xch_wait(xc, 57) ? 1 : 0;
    __syncthreads();
    if (!ok_s) return;
    // merge the segments once per CTA (coalesced, L1 bypassed: the buffer is rewritten by peers between launches);
    // fixed order, so every rank computes bit-identical statistics
    for (int i = threadIdx.x; i < 2 * C; i += CL_THREADS) {
      float acc = 0.f;
      for (int q = 0; q < xc.nsrc; ++q) acc += __ldcg(xc.src + q * xc.src_stride + static_cast<long long>(bidx) * 2 * C + i);
      sh_sum[i] = acc;
    }
    __syncthreads();
  }
  if (r >= R) {
    if (xc.npeers > 0) __syncthreads();   // matches the barrier before the completion count below
    return;
  }
  float k0[8], k1[8], k2[8], k3[8], kw[8], kb[8];   // per-channel constants
  float sft[8];                                      // shift of the statistics pass (the sample's first token) or 0
#pragma unroll
  for (int j = 0; j < 8; ++j) sft[j] = 0.f;
  if (MODE == 0 && shifted) unpack8((reinterpret_cast<const uint4*>(x + static_cast<long long>(bidx) * T * C) + v)[0], sft);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int c = v * 8 + j;
    const long long sc = (static_cast<long long>(bidx) * C + c) * 2;
    const float wc = w ? w[c] : 1.f, bc = b ? b[c] : 0.f;
    kw[j] = wc;
    kb[j] = bc;
    float s0, s1;
    if (xc.npeers > 0) {
      s0 = sh_sum[2 * c];
      s1 = sh_sum[2 * c + 1];
    } else {
      s0 = sums[sc];
      s1 = sums[sc + 1];
    }
    if (MODE == 0) {
      const float dm = s0 * inv_count;                 // mean of (x - shift)
      const float mean = sft[j] + dm;
      const float var = fmaxf(s1 * inv_count - dm * dm, 0.f);
      const float rstd = rsqrtf(var + eps);
      k0[j] = wc * rstd;
      k1[j] = bc - mean * k0[j];
      if (stats && blockIdx.x == 0 && r == 0) {
        stats[sc] = mean;
        stats[sc + 1] = rstd;
      }
    } else {
      k0[j] = stats[sc];          // mean
      k1[j] = stats[sc + 1];      // rstd
      k2[j] = s0 * inv_count;
      k3[j] = s1 * inv_count;
    }
  }
  const long long t0 = static_cast<long long>(blockIdx.x) * slab;
  long long t1 = t0 + slab;
  if (t1 > T) t1 = T;
  const long long base = static_cast<long long>(bidx) * T * C;
  const uint4* xv = reinterpret_cast<const uint4*>(x + base) + v;
  const uint4* gv = MODE == 1 ? reinterpret_cast<const uint4*>(dy + base) + v : nullptr;
  uint4* ov = reinterpret_cast<uint4*>(out + base) + v;
  auto transform = [&](const uint4& xr, const uint4& gr) -> uint4 {
    float f[8];
    unpack8(xr, f);
    if (MODE == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float val = fmaf(f[j], k0[j], k1[j]);
        f[j] = act ? gelu_f(val, act) : val;
      }
    } else {
      float g[8];
      unpack8(gr, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (f[j] - k0[j]) * k1[j];
        float gg = g[j];
        if (act) gg *= dgelu_f(fmaf(xh, kw[j], kb[j]), act);
        f[j] = k1[j] * kw[j] * (gg - k2[j] - xh * k3[j]);
      }
    }
    return pack8(f);
  };
  // four rows in flight per thread: independent 16-byte loads cover the HBM latency
  long long t = t0 + r;
  for (; t + 3LL * R < t1; t += 4LL * R) {
    uint4 xr[4], gr[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      xr[u] = xv[(t + u * R) * V];
      if (MODE == 1) gr[u] = gv[(t + u * R) * V];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) ov[(t + u * R) * V] = transform(xr[u], gr[u]);
  }
  for (; t < t1; t += R) {
    const uint4 xr = xv[t * V];
    uint4 gr = xr;
    if (MODE == 1) gr = gv[t * V];
    ov[t * V] = transform(xr, gr);
  }
  if (xc.npeers > 0) {
    // the last CTA tells the peers that this rank is done with their sums
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int prev = atomicAdd(xc.done_ctr, 1u);
      if (prev == gridDim.x * gridDim.y - 1) xch_signal(xc);
    }
  }
}

// ------------------------------------------------------------------------------------------ Lp norms

constexpr int LP_CHUNK = 1 << 16;   // elements of one plane handled by one CTA

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }


// 16-byte vector access for the loss kernels: VW elements of one latitude row per load (W is a multiple of VW there)
template <typename T>
struct LpVec;
template <>
struct LpVec<float> {
  static constexpr int VW = 4;
  static __device__ __forceinline__ void load(const float* p, long long i, float (&v)[4]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p + i));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  }
  static __device__ __forceinline__ void store(float* p, long long i, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p + i) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct LpVec<__nv_bfloat16> {
  static constexpr int VW = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, long long i, float (&v)[8]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p + i));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, long long i, const float (&v)[8]) {
    uint4 a;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    *reinterpret_cast<uint4*>(p + i) = a;
  }
};

template <typename T, int P, bool VEC>
__global__ void __launch_bounds__(NT) lp_norms_kernel(const T* __restrict__ pred, const T* __restrict__ tgt,
                                                      const float* __restrict__ qlat, float* __restrict__ out,
                                                      float* __restrict__ partial, int* __restrict__ counters, int W,
                                                      long long hw, int chunks) {
  const int plane = blockIdx.y, chunk = blockIdx.x;
  const T* pp = pred + static_cast<long long>(plane) * hw;
  const T* tp = tgt + static_cast<long long>(plane) * hw;
  const long long beg = static_cast<long long>(chunk) * LP_CHUNK;
  long long end = beg + LP_CHUNK;
  if (end > hw) end = hw;
  float sd = 0.f, st = 0.f;
  if (VEC) {
    constexpr int VW = LpVec<T>::VW;
#pragma unroll 4
    for (long long i = beg + static_cast<long long>(threadIdx.x) * VW; i < end; i += static_cast<long long>(NT) * VW) {
      const float q = qlat[static_cast<unsigned>(i) / static_cast<unsigned>(W)];
      float p[VW], t[VW];
      LpVec<T>::load(pp, i, p);
      LpVec<T>::load(tp, i, t);
      float ad = 0.f, at = 0.f;
#pragma unroll
      for (int j = 0; j < VW; ++j) {
        const float d = p[j] - t[j];
        if (P == 2) {
          ad = fmaf(d, d, ad);
          at = fmaf(t[j], t[j], at);
        } else {
          ad += fabsf(d);
          at += fabsf(t[j]);
        }
      }
      sd = fmaf(q, ad, sd);
      st = fmaf(q, at, st);
    }
  } else {
    for (long long i = beg + threadIdx.x; i < end; i += NT) {
      const float q = qlat[i / W];
      const float p = ldf<T>(pp, i), t = ldf<T>(tp, i);
      const float d = p - t;
      if (P == 2) {
        sd += q * d * d;
        st += q * t * t;
      } else {
        sd += q * fabsf(d);
        st += q * fabsf(t);
      }
    }
  }
  block_sum2(sd, st);
  __shared__ int last;
  if (threadIdx.x == 0) {
    float* pr = partial + (static_cast<long long>(plane) * chunks + chunk) * 2;
    pr[0] = sd;
    pr[1] = st;
    __threadfence();
    const int done = atomicAdd(counters + plane, 1);
    last = (done == chunks - 1);
  }
  __syncthreads();
  if (last) {
    // fixed-order final sum -> deterministic result
    __threadfence();
    float a = 0.f, b = 0.f;
    const volatile float* pr = partial + static_cast<long long>(plane) * chunks * 2;
    for (int i = threadIdx.x; i < chunks; i += NT) {
      a += pr[2 * i];
      b += pr[2 * i + 1];
    }
    block_sum2(a, b);
    if (threadIdx.x == 0) {
      out[2 * plane] = a;
      out[2 * plane + 1] = b;
      counters[plane] = 0;
    }
  }
}

template <typename T>
__device__ __forceinline__ void stf(T* p, long long i, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

template <typename T, int P, bool VEC>
__global__ void __launch_bounds__(NT) lp_bwd_kernel(const T* __restrict__ pred, const T* __restrict__ tgt,
                                                    const float* __restrict__ qlat, const float* __restrict__ coef,
                                                    T* __restrict__ grad, int W, long long hw) {
  const int plane = blockIdx.y;
  const float cf = coef[plane];
  const long long base = static_cast<long long>(plane) * hw;
  const long long beg = static_cast<long long>(blockIdx.x) * LP_CHUNK;
  long long end = beg + LP_CHUNK;
  if (end > hw) end = hw;
  if (VEC) {
    constexpr int VW = LpVec<T>::VW;
#pragma unroll 4
    for (long long i = beg + static_cast<long long>(threadIdx.x) * VW; i < end; i += static_cast<long long>(NT) * VW) {
      const float cq = cf * qlat[static_cast<unsigned>(i) / static_cast<unsigned>(W)];
      float p[VW], t[VW];
      LpVec<T>::load(pred, base + i, p);
      LpVec<T>::load(tgt, base + i, t);
#pragma unroll
      for (int j = 0; j < VW; ++j) {
        const float d = p[j] - t[j];
        const float g = (P == 2) ? 2.f * d : ((d > 0.f) ? 1.f : ((d < 0.f) ? -1.f : 0.f));
        p[j] = cq * g;
      }
      LpVec<T>::store(grad, base + i, p);
    }
  } else {
    for (long long i = beg + threadIdx.x; i < end; i += NT) {
      const float q = qlat[i / W];
      const float d = ldf<T>(pred, base + i) - ldf<T>(tgt, base + i);
      float g;
      if (P == 2) g = 2.f * d;
      else g = (d > 0.f) ? 1.f : ((d < 0.f) ? -1.f : 0.f);
      stf<T>(grad, base + i, cf * q * g);
    }
  }
}

// ------------------------------------------------------------------------------------------ AdamW

__global__ void __launch_bounds__(256) adamw_kernel(const AdamEntry* __restrict__ table, const int* __restrict__ chunk_tensor,
                                                    const long long* __restrict__ chunk_off, long long chunk,
                                                    const float* __restrict__ hyper, const int* __restrict__ err) {
  // A bounded wait that ran out earlier in this step (a lost peer in the gradient all-reduce, a handshake that timed
  // out) leaves gradients that are incomplete: the update is skipped, so that the replicas stay identical until the
  // host reads the error word and raises.
  if (err != nullptr && *reinterpret_cast<const volatile int*>(err) != 0) return;
  const AdamEntry e = table[chunk_tensor[blockIdx.x]];
  const long long off = chunk_off[blockIdx.x];
  long long n = e.n - off;
  if (n > chunk) n = chunk;
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4] * e.wd_scale, step = hyper[5],
              gs = hyper[6];
  const bool decoupled = hyper[7] != 0.f;
  const float bc1 = 1.f - powf(b1, step), bc2 = 1.f - powf(b2, step);
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  float* p = e.p + off;
  const float* g = e.g + off;
  float* m = e.m + off;
  float* v = e.v + off;
  __nv_bfloat16* sh = e.shadow ? e.shadow + off : nullptr;
  // chunk and off are multiples of 4, so float4 access is aligned whenever the tensor base is
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v)) & 15) == 0;
  const long long n4 = vec ? (n >> 2) : 0;
  for (long long i = threadIdx.x; i < n4; i += blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    const float4 gg4 = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float P[4] = {pp.x, pp.y, pp.z, pp.w}, G[4] = {gg4.x * gs, gg4.y * gs, gg4.z * gs, gg4.w * gs};
    float M[4] = {mm.x, mm.y, mm.z, mm.w}, V[4] = {vv.x, vv.y, vv.z, vv.w};
    float G2[4];
    if (e.pair_mode) {
      G2[0] = G2[1] = G[0] * G[0] + G[1] * G[1];
      G2[2] = G2[3] = G[2] * G[2] + G[3] * G[3];
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) G2[j] = G[j] * G[j];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gj = G[j];
      if (decoupled) P[j] *= (1.f - lr * wd);
      else gj += wd * P[j];
      M[j] = b1 * M[j] + (1.f - b1) * gj;
      V[j] = b2 * V[j] + (1.f - b2) * (decoupled ? G2[j] : (e.pair_mode ? G2[j] : gj * gj));
      const float denom = sqrtf(V[j]) * inv_sqrt_bc2 + eps;
      P[j] -= step_size * M[j] / denom;
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(P[0], P[1], P[2], P[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(M[0], M[1], M[2], M[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(V[0], V[1], V[2], V[3]);
    if (sh) {
      sh[4 * i] = __float2bfloat16(P[0]);
      sh[4 * i + 1] = __float2bfloat16(P[1]);
      sh[4 * i + 2] = __float2bfloat16(P[2]);
      sh[4 * i + 3] = __float2bfloat16(P[3]);
    }
  }
  for (long long i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) {
    float gj = g[i] * gs;
    float g2 = gj * gj;
    if (e.pair_mode) {
      const float go = g[i ^ 1] * gs;   // partner of the (re, im) pair; off is even
      g2 += go * go;
    }
    float pj = p[i];
    if (decoupled) pj *= (1.f - lr * wd);
    else gj += wd * pj;
    const float mj = b1 * m[i] + (1.f - b1) * gj;
    const float vj = b2 * v[i] + (1.f - b2) * ((decoupled || e.pair_mode) ? g2 : gj * gj);
    pj -= step_size * mj / (sqrtf(vj) * inv_sqrt_bc2 + eps);
    p[i] = pj;
    m[i] = mj;
    v[i] = vj;
    if (sh) sh[i] = __float2bfloat16(pj);
  }
}

// ------------------------------------------------------------------------------------------ spectral weights

// grid: (Cin/32, Cout, ceil(L/32)); block 32x8
__global__ void spectral_expand_kernel(const float2* __restrict__ w, __nv_bfloat16* __restrict__ wx, int Cin, int Cout, int L) {
  __shared__ float2 tile[32][33];
  const int c0 = blockIdx.x * 32, o = blockIdx.y, l0 = blockIdx.z * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int c = c0 + j, l = l0 + threadIdx.x;
    float2 v = make_float2(0.f, 0.f);
    if (c < Cin && l < L) v = w[(static_cast<long long>(c) * Cout + o) * L + l];
    tile[j][threadIdx.x] = v;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int l = l0 + j, c = c0 + threadIdx.x;
    if (l < L && c < Cin) {
      const float2 v = tile[threadIdx.x][j];
      // planar 2x2-block form: rows (ri', o), columns (ri, c):  [[Wr, -Wi], [Wi, Wr]]
      __nv_bfloat16* base = wx + static_cast<long long>(l) * 4 * Cout * Cin;
      const long long r0 = static_cast<long long>(o) * 2 * Cin, r1 = static_cast<long long>(Cout + o) * 2 * Cin;
      base[r0 + c] = __float2bfloat16(v.x);
      base[r0 + Cin + c] = __float2bfloat16(-v.y);
      base[r1 + c] = __float2bfloat16(v.y);
      base[r1 + Cin + c] = __float2bfloat16(v.x);
    }
  }
}

// two_block == 0: dwx is the full real 2x2-block gradient [L, 2Cout, 2Cin];  two_block == 1: dwx is [2][L][Cout][Cin]
// holding (dWr, dWi) already.  assign != 0 overwrites dw instead of accumulating into it.
__global__ void spectral_fold_kernel(const float* __restrict__ dwx, float2* __restrict__ dw, int Cin, int Cout, int L,
                                     int two_block, int assign) {
  __shared__ float2 tile[32][33];
  const int c0 = blockIdx.x * 32, o = blockIdx.y, l0 = blockIdx.z * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int l = l0 + j, c = c0 + threadIdx.x;
    float2 v = make_float2(0.f, 0.f);
    if (l < L && c < Cin) {
      if (two_block) {
        const long long e = (static_cast<long long>(l) * Cout + o) * Cin + c;
        v.x = dwx[e];
        v.y = dwx[e + static_cast<long long>(L) * Cout * Cin];
      } else {
        const float* base = dwx + static_cast<long long>(l) * 4 * Cout * Cin;
        const long long r0 = static_cast<long long>(o) * 2 * Cin, r1 = static_cast<long long>(Cout + o) * 2 * Cin;
        v.x = base[r0 + c] + base[r1 + Cin + c];   // dWr
        v.y = base[r1 + c] - base[r0 + Cin + c];   // dWi
      }
    }
    tile[j][threadIdx.x] = v;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int c = c0 + j, l = l0 + threadIdx.x;
    if (c < Cin && l < L) {
      float2* d = dw + (static_cast<long long>(c) * Cout + o) * L + l;
      const float2 v = tile[threadIdx.x][j];
      if (assign) {
        *d = v;
      } else {
        float2 cur = *d;
        cur.x += v.x;
        cur.y += v.y;
        *d = cur;
      }
    }
  }
}

// rows of (re[C], im[C]) bf16 -> (im[C], -re[C]); C a multiple of 8 (16-byte vectors, sign flip on the bit pattern)
__global__ void swap_ri_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, long long rows, int cv) {
  const long long total = rows * 2 * cv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / (2 * cv);
    const int j = static_cast<int>(i - row * 2 * cv);
    if (j < cv) {
      out[i] = in[row * 2 * cv + cv + j];
    } else {
      uint4 v = in[row * 2 * cv + (j - cv)];
      v.x ^= 0x80008000u;
      v.y ^= 0x80008000u;
      v.z ^= 0x80008000u;
      v.w ^= 0x80008000u;
      out[i] = v;
    }
  }
}

__global__ void cast_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = __float2bfloat16(x[i]);
}

__device__ __forceinline__ uint64_t splitmix(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// counter-based N(0,1): two 64-bit hashes -> Box-Muller; deterministic in (seed, index)
__global__ void fill_normal_kernel(__nv_bfloat16* __restrict__ y, long long n, uint64_t seed) {
  const long long pairs = (n + 1) >> 1;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < pairs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint64_t h = splitmix(seed ^ splitmix(static_cast<uint64_t>(i)));
    const float u1 = (static_cast<float>(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = (static_cast<float>((h >> 16) & 0xFFFFFF) + 0.5f) * (1.0f / 16777216.0f);
    const float r = sqrtf(-2.f * __logf(u1));
    float sn, cs;
    __sincosf(6.283185307179586f * u2, &sn, &cs);
    y[2 * i] = __float2bfloat16(r * cs);
    if (2 * i + 1 < n) y[2 * i + 1] = __float2bfloat16(r * sn);
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

cudaError_t inorm_fwd(const __nv_bfloat16* x, __nv_bfloat16* y, const float* w, const float* b, float* stats, int planes,
                      int C, long long hw, float eps, int act, int ext_stats, cudaStream_t s) {
  if (act) act = gelu_tanh() ? 2 : 1;
  if (planes <= 0) return cudaSuccess;
  const bool vec = (hw % 8 == 0) && aligned16(x) && aligned16(y);
  const int mode = ext_stats ? 2 : 0;
  if (vec) inorm_fwd_kernel<true><<<planes, NT, 0, s>>>(x, y, w, b, stats, C, hw, eps, act, mode);
  else inorm_fwd_kernel<false><<<planes, NT, 0, s>>>(x, y, w, b, stats, C, hw, eps, act, mode);
  return cudaGetLastError();
}

cudaError_t inorm_partial_stats(const __nv_bfloat16* x, float* sums, int planes, long long hw, cudaStream_t s) {
  if (planes <= 0) return cudaSuccess;
  const bool vec = (hw % 8 == 0) && aligned16(x);
  if (vec) inorm_fwd_kernel<true><<<planes, NT, 0, s>>>(x, nullptr, nullptr, nullptr, sums, 1, hw, 0.f, 0, 1);
  else inorm_fwd_kernel<false><<<planes, NT, 0, s>>>(x, nullptr, nullptr, nullptr, sums, 1, hw, 0.f, 0, 1);
  return cudaGetLastError();
}

cudaError_t inorm_bwd(const __nv_bfloat16* x, const __nv_bfloat16* dy, __nv_bfloat16* dx, const float* w, const float* b,
                      const float* stats, float* dw, float* db, float* sums_io, int planes, int C, long long hw,
                      double count, int act, int ext_sums, cudaStream_t s) {
  if (act) act = gelu_tanh() ? 2 : 1;
  if (planes <= 0) return cudaSuccess;
  const bool vec = (hw % 8 == 0) && aligned16(x) && aligned16(dy) && (dx == nullptr || aligned16(dx));
  const float inv = static_cast<float>(1.0 / count);
  if (vec) inorm_bwd_kernel<true><<<planes, NT, 0, s>>>(x, dy, dx, w, b, stats, dw, db, sums_io, C, hw, inv, act, ext_sums);
  else inorm_bwd_kernel<false><<<planes, NT, 0, s>>>(x, dy, dx, w, b, stats, dw, db, sums_io, C, hw, inv, act, ext_sums);
  return cudaGetLastError();
}

static inline bool cl_ok(int C) { return C % 8 == 0 && C >= 8 && C <= 1024 && (CL_THREADS / (C / 8)) >= 1; }
// tokens per CTA: enough CTAs to fill the machine a few times over, but at least a few passes of the row loop each
static inline int cl_slab(int C, long long T, int B, int ctas_per_sm = 4) {
  const int R = CL_THREADS / (C / 8);
  long long target = (static_cast<long long>(ctas_per_sm) * sm_count() + B - 1) / B;
  long long slab = (T + target - 1) / target;
  if (slab < 4LL * R) slab = 4LL * R;
  return static_cast<int>(slab);
}

cudaError_t inorm_cl_sums(const __nv_bfloat16* x, const __nv_bfloat16* dy, const float* w, const float* b, const float* stats,
                          float* sums, float* dw, float* db, int B, int C, long long T, int act, int mode, cudaStream_t s,
                          const StatExchange* xch) {
  if (act) act = gelu_tanh() ? 2 : 1;
  // mode: bit 0 = backward pass, bit 1 = forward statistics shifted by the first token (local statistics only)
  const int shifted = ((mode >> 1) & 1) && (!xch || xch->npeers == 0);
  mode &= 1;
  if (!cl_ok(C)) return cudaErrorInvalidValue;
  StatExchange xc;
  memset(&xc, 0, sizeof(xc));
  if (xch) xc = *xch;
  // every CTA ends with 2C atomics on the same [B, C, 2] words: fewer, longer CTAs than the streaming pass
  const int slab = cl_slab(C, T, B, 2);
  dim3 grid(static_cast<unsigned>((T + slab - 1) / slab), B);
  const size_t sh = 2 * C * sizeof(float);
  if (mode == 0) inorm_cl_sums_kernel<0><<<grid, CL_THREADS, sh, s>>>(x, dy, w, b, stats, sums, dw, db, C, T, act, slab, shifted, xc);
  else inorm_cl_sums_kernel<1><<<grid, CL_THREADS, sh, s>>>(x, dy, w, b, stats, sums, dw, db, C, T, act, slab, 0, xc);
  return cudaGetLastError();
}

cudaError_t inorm_cl_apply(const __nv_bfloat16* x, const __nv_bfloat16* dy, __nv_bfloat16* out, const float* w, const float* b,
                           const float* sums, float* stats, int B, int C, long long T, double count, float eps, int act, int mode,
                           cudaStream_t s, const StatExchange* xch) {
  if (act) act = gelu_tanh() ? 2 : 1;
  // mode: bit 0 = backward pass, bit 1 = forward statistics shifted by the first token (local statistics only)
  const int shifted = ((mode >> 1) & 1) && (!xch || xch->npeers == 0);
  mode &= 1;
  if (!cl_ok(C)) return cudaErrorInvalidValue;
  StatExchange xc;
  memset(&xc, 0, sizeof(xc));
  if (xch) xc = *xch;
  const int slab = cl_slab(C, T, B);
  dim3 grid(static_cast<unsigned>((T + slab - 1) / slab), B);
  const float inv = static_cast<float>(1.0 / count);
  const size_t shx = xc.npeers > 0 ? 2 * C * sizeof(float) : 0;
  if (mode == 0) inorm_cl_apply_kernel<0><<<grid, CL_THREADS, shx, s>>>(x, dy, out, w, b, sums, stats, C, T, inv, eps, act, slab, shifted, xc);
  else inorm_cl_apply_kernel<1><<<grid, CL_THREADS, shx, s>>>(x, dy, out, w, b, sums, stats, C, T, inv, eps, act, slab, 0, xc);
  return cudaGetLastError();
}

// The 16-byte path of the loss kernels needs every row to hold a whole number of vectors, 16-byte aligned planes and
// element indices that fit 32 bits (the row index is a 32-bit division there).
static bool lp_vec_ok(const void* a, const void* b, const void* c, int is_f32, int W, long long hw) {
  const int vw = is_f32 ? 4 : 8;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c);
  return (W % vw) == 0 && (bits & 15) == 0 && hw < (1ll << 31);
}

int lp_norms_chunks(long long hw) { return static_cast<int>((hw + LP_CHUNK - 1) / LP_CHUNK); }

cudaError_t lp_norms(const void* pred, const void* tgt, int is_f32, const float* qlat, float* out, float* scratch,
                     int planes, int H, int W, int P, cudaStream_t s) {
  if (planes <= 0) return cudaSuccess;
  const long long hw = static_cast<long long>(H) * W;
  const int chunks = lp_norms_chunks(hw);
  float* partial = scratch;
  int* counters = reinterpret_cast<int*>(scratch + static_cast<long long>(planes) * chunks * 2);
  // The counters' position depends on (planes, chunks): a scratch buffer that served another shape holds partial sums
  // there.  They are cleared on the stream before every launch (a memset node under graph capture).
  cudaError_t me = cudaMemsetAsync(counters, 0, sizeof(int) * static_cast<size_t>(planes), s);
  if (me != cudaSuccess) return me;
  dim3 grid(chunks, planes);
  const bool vec = lp_vec_ok(pred, tgt, nullptr, is_f32, W, hw);
#define MK_LP_NORMS(T, PP, V) \
  lp_norms_kernel<T, PP, V><<<grid, NT, 0, s>>>((const T*)pred, (const T*)tgt, qlat, out, partial, counters, W, hw, chunks)
#define MK_LP_NORMS_T(T)                        \
  do {                                          \
    if (P == 2) {                               \
      if (vec) MK_LP_NORMS(T, 2, true);         \
      else MK_LP_NORMS(T, 2, false);            \
    } else {                                    \
      if (vec) MK_LP_NORMS(T, 1, true);         \
      else MK_LP_NORMS(T, 1, false);            \
    }                                           \
  } while (0)
  if (is_f32) MK_LP_NORMS_T(float);
  else MK_LP_NORMS_T(__nv_bfloat16);
#undef MK_LP_NORMS_T
#undef MK_LP_NORMS
  return cudaGetLastError();
}

cudaError_t lp_norms_bwd(const void* pred, const void* tgt, int is_f32, const float* qlat, const float* coef, void* grad,
                         int planes, int H, int W, int P, cudaStream_t s) {
  if (planes <= 0) return cudaSuccess;
  const long long hw = static_cast<long long>(H) * W;
  dim3 grid(lp_norms_chunks(hw), planes);
  const bool vec = lp_vec_ok(pred, tgt, grad, is_f32, W, hw);
#define MK_LP_BWD(T, PP, V) \
  lp_bwd_kernel<T, PP, V><<<grid, NT, 0, s>>>((const T*)pred, (const T*)tgt, qlat, coef, (T*)grad, W, hw)
#define MK_LP_BWD_T(T)                        \
  do {                                        \
    if (P == 2) {                             \
      if (vec) MK_LP_BWD(T, 2, true);         \
      else MK_LP_BWD(T, 2, false);            \
    } else {                                  \
      if (vec) MK_LP_BWD(T, 1, true);         \
      else MK_LP_BWD(T, 1, false);            \
    }                                         \
  } while (0)
  if (is_f32) MK_LP_BWD_T(float);
  else MK_LP_BWD_T(__nv_bfloat16);
#undef MK_LP_BWD_T
#undef MK_LP_BWD
  return cudaGetLastError();
}

cudaError_t adamw_step(const AdamEntry* table, const int* chunk_tensor, const long long* chunk_off, int nchunks,
                       long long chunk, const float* hyper, const int* err, cudaStream_t s) {
  if (nchunks <= 0) return cudaSuccess;
  adamw_kernel<<<nchunks, 256, 0, s>>>(table, chunk_tensor, chunk_off, chunk, hyper, err);
  return cudaGetLastError();
}

cudaError_t spectral_expand(const float* w, __nv_bfloat16* wx, int Cin, int Cout, int L, cudaStream_t s) {
  dim3 grid((Cin + 31) / 32, Cout, (L + 31) / 32), block(32, 8);
  spectral_expand_kernel<<<grid, block, 0, s>>>(reinterpret_cast<const float2*>(w), wx, Cin, Cout, L);
  return cudaGetLastError();
}

cudaError_t spectral_fold(const float* dwx, float* dw, int Cin, int Cout, int L, cudaStream_t s, int two_block, int assign) {
  dim3 grid((Cin + 31) / 32, Cout, (L + 31) / 32), block(32, 8);
  spectral_fold_kernel<<<grid, block, 0, s>>>(dwx, reinterpret_cast<float2*>(dw), Cin, Cout, L, two_block, assign);
  return cudaGetLastError();
}

cudaError_t swap_ri_bf16(const __nv_bfloat16* in, __nv_bfloat16* out, long long rows, int C, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  if (C <= 0 || (C & 7) || (reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return cudaErrorInvalidValue;
  const long long total = rows * 2 * (C / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  swap_ri_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(reinterpret_cast<const uint4*>(in), reinterpret_cast<uint4*>(out),
                                                               rows, C / 8);
  return cudaGetLastError();
}

cudaError_t cast_f32_bf16(const float* x, __nv_bfloat16* y, long long n, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  long long blocks = (n + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  cast_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(x, y, n);
  return cudaGetLastError();
}

cudaError_t fill_normal_bf16(__nv_bfloat16* y, long long n, uint64_t seed, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  long long blocks = ((n + 1) / 2 + 255) / 256;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  fill_normal_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(y, n, seed);
  return cudaGetLastError();
}

}  // namespace mk
