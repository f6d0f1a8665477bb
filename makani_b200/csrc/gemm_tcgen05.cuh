// Declarations for the sm_100a tensor-core GEMM engine (tcgen05 + TMEM + TMA).
//
// One persistent, warp-specialised kernel computes, for every batch index z = z_hi * zlo_n + z_lo,
//
//     D_z[r, n] = epilogue( alpha * sum_k A_z[r, k] * B_z[n, k] )
//
// A is (M x K), B is (N x K); either operand may be K-major (k contiguous) or MN-major (row index
// contiguous).  Operands are bf16 (kind::f16) or fp32 read as tf32 (kind::tf32); accumulation is fp32
// in tensor memory.  The destination is addressed with split strides so that a tile can be scattered
// straight into the layout the next transform stage wants:
//
//     addr(z, r, n) = D + z_hi*d_zhi + z_lo*d_zlo + (r / rdiv)*rs_hi + (r % rdiv)*rs_lo
//                       + (n / ndiv)*ns_hi + (n % ndiv)            (n is contiguous)
//
// "Triangular" structure (associated Legendre functions vanish for l < m) is expressed as affine
// functions of z_hi: rows outside [rmin, rmax) are known to be zero (tiles entirely outside are
// written as zeros without touching the tensor cores) and the k-loop is restricted to [kmin, kmax).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mk {

struct GemmOperand {
  const void* ptr;      // 16-byte aligned base
  int rows;             // M (for A) or N (for B)
  int mn_major;         // 0: k contiguous, 1: row index contiguous
  long long ld;         // stride in elements of the non-contiguous dimension (multiple of 16 bytes)
  long long zs_lo;      // batch strides in elements (0 = operand shared across that batch index)
  long long zs_hi;
};

struct GemmEpilogue {
  void* D;
  int out_f32;          // 0: bf16 output, 1: fp32 output
  int accumulate;       // 1: atomically add into fp32 D (used by split-k / batch-reduced weight gradients)
  long long d_zlo, d_zhi;
  int rdiv; long long rs_hi, rs_lo;
  int ndiv; long long ns_hi;
  float alpha;
  const float* bias;    // fp32, may be null
  int bias_mode;        // 1: per row r, 2: per column n
  long long bias_zs;    // elements between the bias vectors of consecutive z_lo batches (0: one vector for all)
  int act;              // 0 none; 1 GELU, 3 ReLU, 5 soft shrinkage (threshold act_param); 2 / 4 / 6: multiply by the
                        // derivative of GELU / ReLU / soft shrinkage evaluated at `resid`; 8: multiply by `resid`
                        // itself (see gelu.cuh)
  int save_deriv;       // act == 1 with a second output: that output receives GELU'(pre-activation) instead of the
                        // pre-activation, so that the backward pass multiplies by it (act 8) without evaluating anything
  float act_param;
  const void* resid;    // optional tensor added after the activation (odd act or 0), or the operand of the derivative
                        // (even act: saved pre-activation for GELU, saved output for ReLU / shrinkage); same
                        // addressing and dtype as D
  // optional second output: the pre-activation value (alpha*acc + bias) in the same layout / dtype
  void* preact;
};

struct GemmProblem {
  int M, N, K;
  int zlo_n, zhi_n;
  int elem_bytes;       // 2: bf16, 4: tf32
  int splits;           // split-k factor (requires accumulate)
  int rmin_a, rmin_b, rmax_a, rmax_b;   // valid rows [rmin_a*z_hi+rmin_b, rmax_a*z_hi+rmax_b)
  int kmin_a, kmin_b, kmax_a, kmax_b;   // contributing k range
  int bn;               // tile width: 128 or 256 (0 = choose)
};

// Optional: B operand gathered from several devices and cross-device handshakes (see gemm_tcgen05.cu).
struct GemmPeer {
  int nseg;                        // 0/1: B is the ordinary single operand
  const void* seg_ptr[8];          // base pointer of segment s (peer memory mapped into this process)
  int seg_len[8], seg_apos[8], seg_gstart[8];
  int np_wait[2], np_sig[2], nwait, nsig;   // peers per wait list / signal list; number of lists in use
  const unsigned int* wait[2];
  const unsigned int* wait_exp[2];
  int wait_off[2];
  unsigned int* bump[2];
  unsigned int* sig[2][8];
  unsigned int* done_ctr;
  int ndx;                         // additional destinations of the output (peers' copies of the same buffer)
  void* Dx[7];                     // base pointers matching GemmEpilogue::D (offset already applied)
};

// Copy of a strided 2-D block into the same place of `ndst` destination buffers (this device's and its peers'),
// with the producer side of the handshake in `g` (wait list 0, signal list 0) executed by the same kernel.
cudaError_t peer_publish_launch(const void* src, long long rows, long long row_bytes, long long src_stride_bytes,
                                long long dst_stride_bytes, void* const* dsts, int ndst, const GemmPeer& g, int* err_flag,
                                cudaStream_t stream);

// out[i] = sum_q srcs[q][i] (+ bias[i % C]) over `n_elems` bf16 values (multiple of 8), reading `nsrc` local segments that
// peers have filled; consumer side of the handshake in `g` (wait list 0, signal list 0) executed by the same kernel.
cudaError_t peer_sum_launch(void* out, long long n_elems, const void* const* srcs, int nsrc, const float* bias, int C,
                            const GemmPeer& g, int* err_flag, cudaStream_t stream);

// Returns cudaSuccess or an error; never throws.  `err_flag` is a device int that the kernel sets to a
// non-zero code when a bounded barrier wait runs out (the launch still terminates).
cudaError_t gemm_launch(const GemmProblem& p, const GemmOperand& A, const GemmOperand& B,
                        const GemmEpilogue& e, int* err_flag, cudaStream_t stream, const GemmPeer* peer = nullptr);

const char* gemm_last_error();

}  // namespace mk
