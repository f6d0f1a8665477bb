// Python bindings (pybind11 / torch tensors) for the sm_100a kernels. Every entry validates device, dtype
// and contiguity, launches on the current CUDA stream and raises on a launch error.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <vector>

#include "fused_ops.cuh"
#include "gelu.cuh"
#include "gemm_tcgen05.cuh"
#include "peer.cuh"
#include "spectral_modes.cuh"

namespace {

using torch::Tensor;

#define MK_CHECK(cond, ...) TORCH_CHECK(cond, "makani_b200: ", __VA_ARGS__)

inline void check_cuda(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "makani_b200: ", what, " failed: ", cudaGetErrorString(e), " ", mk::gemm_last_error());
}

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// one error word per device, set by kernels whose bounded waits expire
std::map<int, Tensor>& err_flags() {
  static std::map<int, Tensor> m;
  return m;
}

Tensor err_flag_for(const Tensor& t) {
  const int dev = t.get_device();
  auto& m = err_flags();
  auto it = m.find(dev);
  if (it == m.end()) {
    Tensor f = torch::zeros({4}, torch::dtype(torch::kInt32).device(t.device()));
    it = m.emplace(dev, f).first;
  }
  return it->second;
}

int64_t read_error_flag(int64_t device) {
  auto& m = err_flags();
  auto it = m.find(static_cast<int>(device));
  if (it == m.end()) return 0;
  return it->second.cpu().data_ptr<int>()[0];
}

void clear_error_flag(int64_t device) {
  auto& m = err_flags();
  auto it = m.find(static_cast<int>(device));
  if (it != m.end()) it->second.zero_();
}

inline const char* base_ptr(const Tensor& t) { return static_cast<const char*>(t.data_ptr()); }

// iparams layout: see makani_b200/ops/gemm.py (GemmSpec.pack)
static bool parse_peer(mk::GemmPeer& g, const std::vector<int64_t>& seg, const std::vector<int64_t>& sync) {
  memset(&g, 0, sizeof(g));
  if (!seg.empty()) {
    g.nseg = static_cast<int>(seg[0]);
    MK_CHECK(g.nseg >= 1 && g.nseg <= 8 && seg.size() == static_cast<size_t>(1 + 4 * g.nseg), "gemm_peer: bad segment list");
    for (int q = 0; q < g.nseg; ++q) {
      g.seg_ptr[q] = reinterpret_cast<const void*>(seg[1 + 4 * q]);
      g.seg_len[q] = static_cast<int>(seg[2 + 4 * q]);
      g.seg_apos[q] = static_cast<int>(seg[3 + 4 * q]);
      g.seg_gstart[q] = static_cast<int>(seg[4 + 4 * q]);
    }
  }
  if (!sync.empty()) {
    // [nwait, nsig, done_ctr, {wait, wait_exp, wait_off, bump, np_wait} x2, {np_sig, sig[8]} x2]
    MK_CHECK(sync.size() == 31, "gemm_peer: sync descriptor must have 31 entries");
    g.nwait = static_cast<int>(sync[0]);
    g.nsig = static_cast<int>(sync[1]);
    g.done_ctr = reinterpret_cast<unsigned int*>(sync[2]);
    for (int i = 0; i < 2; ++i) {
      const size_t o = 3 + 5 * i;
      g.wait[i] = reinterpret_cast<const unsigned int*>(sync[o]);
      g.wait_exp[i] = reinterpret_cast<const unsigned int*>(sync[o + 1]);
      g.wait_off[i] = static_cast<int>(sync[o + 2]);
      g.bump[i] = reinterpret_cast<unsigned int*>(sync[o + 3]);
      g.np_wait[i] = static_cast<int>(sync[o + 4]);
      MK_CHECK(g.np_wait[i] >= 0 && g.np_wait[i] <= 8, "gemm_peer: at most 8 peers");
      const size_t q0 = 13 + 9 * i;
      g.np_sig[i] = static_cast<int>(sync[q0]);
      MK_CHECK(g.np_sig[i] >= 0 && g.np_sig[i] <= 8, "gemm_peer: at most 8 peers");
      for (int q = 0; q < 8; ++q) g.sig[i][q] = reinterpret_cast<unsigned int*>(sync[q0 + 1 + q]);
    }
    MK_CHECK(g.nwait >= 0 && g.nwait <= 2 && g.nsig >= 0 && g.nsig <= 2, "gemm_peer: at most two wait and two signal lists");
  }
  return !seg.empty() || !sync.empty();
}

// Host-side guard for the strided addressing of the GEMM engine: the lowest and highest element a launch can touch
// must lie inside the tensor's storage.  `terms` are (count, stride) pairs; every index runs 0..count-1.
static void check_extent(const Tensor& t, int64_t off, std::initializer_list<std::pair<int64_t, int64_t>> terms, const char* what) {
  int64_t lo = off, hi = off;
  for (const auto& ts : terms) {
    if (ts.first <= 1) continue;
    const int64_t span = (ts.first - 1) * ts.second;
    if (span >= 0) hi += span; else lo += span;
  }
  const int64_t esz = static_cast<int64_t>(t.element_size());
  const int64_t before = t.storage_offset();
  const int64_t total = static_cast<int64_t>(t.storage().nbytes()) / esz;
  MK_CHECK(lo + before >= 0 && hi + before < total, "gemm: ", what, " addressing leaves the tensor's storage (elements ", lo + before,
           "..", hi + before, " of ", total, ")");
}

void gemm_impl(const Tensor& a, const Tensor& b, Tensor& d, const c10::optional<Tensor>& bias,
               const c10::optional<Tensor>& resid, const c10::optional<Tensor>& preact, const std::vector<int64_t>& ip,
               double alpha, const mk::GemmPeer* peer);

void gemm(const Tensor& a, const Tensor& b, Tensor& d, const c10::optional<Tensor>& bias,
          const c10::optional<Tensor>& resid, const c10::optional<Tensor>& preact, const std::vector<int64_t>& ip,
          double alpha) {
  gemm_impl(a, b, d, bias, resid, preact, ip, alpha, nullptr);
}

// GEMM whose B operand is gathered from peer devices along k and/or that takes part in cross-device handshakes
void gemm_peer(const Tensor& a, const Tensor& b, Tensor& d, const c10::optional<Tensor>& bias,
               const c10::optional<Tensor>& resid, const c10::optional<Tensor>& preact, const std::vector<int64_t>& ip,
               double alpha, const std::vector<int64_t>& seg, const std::vector<int64_t>& sync,
               const std::vector<int64_t>& dests) {
  mk::GemmPeer g;
  parse_peer(g, seg, sync);
  MK_CHECK(dests.size() <= 7, "gemm_peer: at most 7 additional destinations");
  g.ndx = static_cast<int>(dests.size());
  const int64_t d_off = ip[25];
  const int64_t osz = d.element_size();
  for (size_t q = 0; q < dests.size(); ++q) g.Dx[q] = reinterpret_cast<char*>(dests[q]) + d_off * osz;
  gemm_impl(a, b, d, bias, resid, preact, ip, alpha, &g);
}

// out (bf16, contiguous in memory) = sum of the segments at `srcs` (+ bias over the innermost `C` channels)
void peer_sum(Tensor& out, const std::vector<int64_t>& srcs, const c10::optional<Tensor>& bias, int64_t C,
              const std::vector<int64_t>& sync) {
  MK_CHECK(out.is_cuda() && out.scalar_type() == torch::kBFloat16, "peer_sum: bf16 CUDA output expected");
  MK_CHECK(!srcs.empty() && srcs.size() <= 8, "peer_sum: 1..8 segments");
  mk::GemmPeer g;
  parse_peer(g, {}, sync);
  c10::cuda::CUDAGuard guard(out.device());
  Tensor ef = err_flag_for(out);
  const void* sp[8];
  for (size_t q = 0; q < srcs.size(); ++q) sp[q] = reinterpret_cast<const void*>(srcs[q]);
  const float* bp = (bias.has_value() && bias->defined()) ? bias->data_ptr<float>() : nullptr;
  check_cuda(mk::peer_sum_launch(out.data_ptr(), out.numel(), sp, static_cast<int>(srcs.size()), bp, static_cast<int>(C), g,
                                 ef.data_ptr<int>(), cur_stream()),
             "peer_sum");
}

// src: local tensor whose data pointer is the first row; dsts: device addresses (this rank's copy and its peers')
void peer_publish(const Tensor& src, int64_t rows, int64_t row_bytes, int64_t src_stride_bytes, int64_t dst_stride_bytes,
                  const std::vector<int64_t>& dsts, const std::vector<int64_t>& sync) {
  MK_CHECK(src.is_cuda(), "peer_publish: CUDA tensor expected");
  MK_CHECK(!dsts.empty() && dsts.size() <= 8, "peer_publish: 1..8 destinations");
  mk::GemmPeer g;
  parse_peer(g, {}, sync);
  c10::cuda::CUDAGuard guard(src.device());
  Tensor ef = err_flag_for(src);
  void* dp[8];
  for (size_t q = 0; q < dsts.size(); ++q) dp[q] = reinterpret_cast<void*>(dsts[q]);
  check_cuda(mk::peer_publish_launch(src.data_ptr(), rows, row_bytes, src_stride_bytes, dst_stride_bytes, dp,
                                     static_cast<int>(dsts.size()), g, ef.data_ptr<int>(), cur_stream()),
             "peer_publish");
}

void gemm_impl(const Tensor& a, const Tensor& b, Tensor& d, const c10::optional<Tensor>& bias,
               const c10::optional<Tensor>& resid, const c10::optional<Tensor>& preact, const std::vector<int64_t>& ip,
               double alpha, const mk::GemmPeer* peer) {
  MK_CHECK(ip.size() == 40, "gemm: expected 40 integer parameters, got ", ip.size());
  MK_CHECK(a.is_cuda() && b.is_cuda() && d.is_cuda(), "gemm: tensors must be CUDA");
  MK_CHECK(a.scalar_type() == b.scalar_type(), "gemm: A and B dtypes differ");
  const int eb = static_cast<int>(a.element_size());
  MK_CHECK((a.scalar_type() == torch::kBFloat16) || (a.scalar_type() == torch::kFloat32), "gemm: operands must be bf16 or fp32");
  MK_CHECK((d.scalar_type() == torch::kBFloat16) || (d.scalar_type() == torch::kFloat32), "gemm: output must be bf16 or fp32");
  c10::cuda::CUDAGuard guard(a.device());
  int k = 0;
  mk::GemmProblem p;
  p.M = ip[k++]; p.N = ip[k++]; p.K = ip[k++];
  p.zlo_n = ip[k++]; p.zhi_n = ip[k++];
  p.elem_bytes = eb;
  p.splits = ip[k++]; p.bn = ip[k++];
  p.rmin_a = ip[k++]; p.rmin_b = ip[k++]; p.rmax_a = ip[k++]; p.rmax_b = ip[k++];
  p.kmin_a = ip[k++]; p.kmin_b = ip[k++]; p.kmax_a = ip[k++]; p.kmax_b = ip[k++];
  mk::GemmOperand A, B;
  const int64_t a_off = ip[k++];
  A.rows = p.M; A.mn_major = ip[k++]; A.ld = ip[k++]; A.zs_lo = ip[k++]; A.zs_hi = ip[k++];
  const int64_t b_off = ip[k++];
  B.rows = p.N; B.mn_major = ip[k++]; B.ld = ip[k++]; B.zs_lo = ip[k++]; B.zs_hi = ip[k++];
  A.ptr = base_ptr(a) + a_off * eb;
  B.ptr = base_ptr(b) + b_off * eb;
  // operand extents: the TMA descriptors clip rows and K to the problem, so the corner elements bound every load
  check_extent(a, a_off, {{A.mn_major ? p.K : p.M, A.ld}, {A.mn_major ? p.M : p.K, 1}, {p.zlo_n, A.zs_lo}, {p.zhi_n, A.zs_hi}}, "A");
  if (peer == nullptr || peer->nseg == 0)   // with segments B is gathered from the segment pointers instead
    check_extent(b, b_off, {{B.mn_major ? p.K : p.N, B.ld}, {B.mn_major ? p.N : p.K, 1}, {p.zlo_n, B.zs_lo}, {p.zhi_n, B.zs_hi}}, "B");
  mk::GemmEpilogue e;
  const int64_t d_off = ip[k++];
  const int osz = static_cast<int>(d.element_size());
  e.D = const_cast<char*>(base_ptr(d)) + d_off * osz;
  e.out_f32 = d.scalar_type() == torch::kFloat32;
  e.accumulate = ip[k++];
  e.d_zlo = ip[k++]; e.d_zhi = ip[k++];
  e.rdiv = ip[k++]; e.rs_hi = ip[k++]; e.rs_lo = ip[k++];
  e.ndiv = ip[k++]; e.ns_hi = ip[k++];
  {
    const int64_t rdiv = e.rdiv > 0 ? e.rdiv : (1 << 30), ndiv = e.ndiv > 0 ? e.ndiv : (1 << 30);   // <= 0: no split
    check_extent(d, d_off, {{p.zhi_n, e.d_zhi}, {p.zlo_n, e.d_zlo}, {(p.M + rdiv - 1) / rdiv, e.rs_hi},
                            {std::min<int64_t>(p.M, rdiv), e.rs_lo}, {(p.N + ndiv - 1) / ndiv, e.ns_hi},
                            {std::min<int64_t>(p.N, ndiv), 1}}, "output");
  }
  e.alpha = static_cast<float>(alpha);
  e.bias_mode = ip[k++];
  {
    const int64_t actw = ip[k++];     // low byte: activation code; bit 8: the second output holds the derivative
    e.act = static_cast<int>(actw & 0xff);
    e.save_deriv = static_cast<int>((actw >> 8) & 1);
  }
  const int64_t resid_off = ip[k++];
  const int64_t preact_off = ip[k++];
  {
    // bit pattern of the activation parameter (fp32), then one reserved slot
    const uint32_t bits = static_cast<uint32_t>(ip[k++]);
    float f;
    memcpy(&f, &bits, sizeof(f));
    e.act_param = f;
    e.bias_zs = ip[k++];
  }
  e.bias = nullptr;
  if (bias.has_value() && bias->defined()) {
    MK_CHECK(bias->is_cuda() && bias->scalar_type() == torch::kFloat32 && bias->is_contiguous(), "gemm: bias must be contiguous fp32 CUDA");
    e.bias = bias->data_ptr<float>();
  }
  e.resid = nullptr;
  if (resid.has_value() && resid->defined()) {
    MK_CHECK(resid->scalar_type() == d.scalar_type(), "gemm: residual dtype must match output");
    e.resid = base_ptr(*resid) + resid_off * osz;
  }
  e.preact = nullptr;
  if (preact.has_value() && preact->defined()) {
    MK_CHECK(preact->scalar_type() == d.scalar_type(), "gemm: preact dtype must match output");
    e.preact = const_cast<char*>(base_ptr(*preact)) + preact_off * osz;
  }
  Tensor ef = err_flag_for(a);
  check_cuda(mk::gemm_launch(p, A, B, e, ef.data_ptr<int>(), cur_stream(), peer), "gemm launch");
}

void inorm_fwd(const Tensor& x, Tensor& y, const c10::optional<Tensor>& w, const c10::optional<Tensor>& b, Tensor& stats,
               int64_t C, double eps, int64_t act, int64_t ext_stats) {
  MK_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == torch::kBFloat16, "inorm_fwd: x must be contiguous bf16 CUDA");
  MK_CHECK(y.is_contiguous() && y.scalar_type() == torch::kBFloat16 && y.numel() == x.numel(), "inorm_fwd: bad y");
  MK_CHECK(stats.scalar_type() == torch::kFloat32 && stats.is_contiguous(), "inorm_fwd: bad stats");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t planes = stats.numel() / 2;
  const int64_t hw = x.numel() / planes;
  const float* wp = (w.has_value() && w->defined()) ? w->data_ptr<float>() : nullptr;
  const float* bp = (b.has_value() && b->defined()) ? b->data_ptr<float>() : nullptr;
  check_cuda(mk::inorm_fwd(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), wp, bp,
                           stats.data_ptr<float>(), static_cast<int>(planes), static_cast<int>(C), hw, static_cast<float>(eps),
                           static_cast<int>(act), static_cast<int>(ext_stats), cur_stream()),
             "inorm_fwd");
}

void inorm_partial_stats(const Tensor& x, Tensor& sums) {
  MK_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == torch::kBFloat16, "inorm_partial_stats: bad x");
  MK_CHECK(sums.scalar_type() == torch::kFloat32 && sums.is_contiguous(), "inorm_partial_stats: bad sums");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t planes = sums.numel() / 2;
  check_cuda(mk::inorm_partial_stats(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), sums.data_ptr<float>(),
                                     static_cast<int>(planes), x.numel() / planes, cur_stream()),
             "inorm_partial_stats");
}

void inorm_bwd(const Tensor& x, const Tensor& dy, c10::optional<Tensor> dx, const c10::optional<Tensor>& w,
               const c10::optional<Tensor>& b, const Tensor& stats, c10::optional<Tensor> dw, c10::optional<Tensor> db,
               c10::optional<Tensor> sums_io, int64_t C, double count, int64_t act, int64_t ext_sums) {
  MK_CHECK(x.is_cuda() && x.is_contiguous() && dy.is_contiguous(), "inorm_bwd: tensors must be contiguous CUDA");
  MK_CHECK(x.scalar_type() == torch::kBFloat16 && dy.scalar_type() == torch::kBFloat16, "inorm_bwd: bf16 expected");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t planes = stats.numel() / 2;
  const int64_t hw = x.numel() / planes;
  auto fp = [](const c10::optional<Tensor>& t) -> float* {
    return (t.has_value() && t->defined()) ? t->data_ptr<float>() : nullptr;
  };
  __nv_bfloat16* dxp = (dx.has_value() && dx->defined()) ? reinterpret_cast<__nv_bfloat16*>(dx->data_ptr()) : nullptr;
  check_cuda(mk::inorm_bwd(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr()),
                           dxp, fp(w), fp(b), stats.data_ptr<float>(), fp(dw), fp(db), fp(sums_io), static_cast<int>(planes),
                           static_cast<int>(C), hw, count, static_cast<int>(act), static_cast<int>(ext_sums), cur_stream()),
             "inorm_bwd");
}

// channels-last instance norm: x is [B, T, C] contiguous (a channels_last NCHW tensor viewed as tokens x channels)
// Builds the statistic-exchange descriptor from the first wait / signal list of a 31-entry handshake descriptor.
static bool make_exchange(mk::StatExchange& xc, const std::vector<int64_t>& sync, const std::vector<int64_t>& addrs, bool producer,
                          const Tensor& like) {
  memset(&xc, 0, sizeof(xc));
  if (sync.empty()) return false;
  mk::GemmPeer g;
  parse_peer(g, {}, sync);
  MK_CHECK(g.nwait == 1 && g.nsig == 1, "instance norm exchange: one wait list and one signal list expected");
  xc.npeers = g.np_wait[0];
  xc.wait = g.wait[0];
  xc.wait_exp = g.wait_exp[0];
  xc.wait_off = g.wait_off[0];
  xc.bump = g.bump[0];
  for (int q = 0; q < 8; ++q) xc.sig[q] = g.sig[0][q];
  xc.done_ctr = g.done_ctr;
  xc.err = err_flag_for(like).data_ptr<int>();
  MK_CHECK(!addrs.empty() && addrs.size() <= 8, "instance norm exchange: 1..8 segment addresses");
  if (producer) {
    xc.ndst = static_cast<int>(addrs.size());
    for (size_t q = 0; q < addrs.size(); ++q) xc.dst[q] = reinterpret_cast<float*>(addrs[q]);
  } else {
    xc.nsrc = static_cast<int>(addrs.size());
    xc.src = reinterpret_cast<const float*>(addrs[0]);
    xc.src_stride = addrs.size() > 1 ? (addrs[1] - addrs[0]) / 4 : 0;
    for (size_t q = 1; q < addrs.size(); ++q)
      MK_CHECK(addrs[q] - addrs[q - 1] == addrs[1] - addrs[0], "instance norm exchange: segments must be equally spaced");
  }
  return true;
}

void inorm_cl_sums(const Tensor& x, const c10::optional<Tensor>& dy, const c10::optional<Tensor>& w, const c10::optional<Tensor>& b,
                   const c10::optional<Tensor>& stats, Tensor& sums, c10::optional<Tensor> dw, c10::optional<Tensor> db, int64_t B,
                   int64_t C, int64_t act, int64_t mode, const std::vector<int64_t>& sync, const std::vector<int64_t>& dsts) {
  MK_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16, "inorm_cl_sums: bf16 CUDA expected");
  MK_CHECK(sums.scalar_type() == torch::kFloat32 && sums.is_contiguous() && sums.numel() == B * C * 2, "inorm_cl_sums: bad sums");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t T = x.numel() / (B * C);
  auto fp = [](const c10::optional<Tensor>& t) -> float* { return (t.has_value() && t->defined()) ? t->data_ptr<float>() : nullptr; };
  const __nv_bfloat16* dyp = (dy.has_value() && dy->defined()) ? reinterpret_cast<const __nv_bfloat16*>(dy->data_ptr()) : nullptr;
  mk::StatExchange xc;
  const bool ex = make_exchange(xc, sync, dsts, true, x);
  check_cuda(mk::inorm_cl_sums(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), dyp, fp(w), fp(b), fp(stats), sums.data_ptr<float>(),
                               fp(dw), fp(db), static_cast<int>(B), static_cast<int>(C), T, static_cast<int>(act), static_cast<int>(mode),
                               cur_stream(), ex ? &xc : nullptr),
             "inorm_cl_sums");
}

void inorm_cl_apply(const Tensor& x, const c10::optional<Tensor>& dy, Tensor& out, const c10::optional<Tensor>& w,
                    const c10::optional<Tensor>& b, const Tensor& sums, c10::optional<Tensor> stats, int64_t B, int64_t C, double count,
                    double eps, int64_t act, int64_t mode, const std::vector<int64_t>& sync, const std::vector<int64_t>& srcs) {
  MK_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16, "inorm_cl_apply: bf16 CUDA expected");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t T = x.numel() / (B * C);
  auto fp = [](const c10::optional<Tensor>& t) -> float* { return (t.has_value() && t->defined()) ? t->data_ptr<float>() : nullptr; };
  const __nv_bfloat16* dyp = (dy.has_value() && dy->defined()) ? reinterpret_cast<const __nv_bfloat16*>(dy->data_ptr()) : nullptr;
  mk::StatExchange xc;
  const bool ex = make_exchange(xc, sync, srcs, false, x);
  check_cuda(mk::inorm_cl_apply(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), dyp, reinterpret_cast<__nv_bfloat16*>(out.data_ptr()),
                                fp(w), fp(b), sums.data_ptr<float>(), fp(stats), static_cast<int>(B), static_cast<int>(C), T, count,
                                static_cast<float>(eps), static_cast<int>(act), static_cast<int>(mode), cur_stream(), ex ? &xc : nullptr),
             "inorm_cl_apply");
}

int64_t lp_scratch_floats(int64_t planes, int64_t hw) { return planes * mk::lp_norms_chunks(hw) * 2 + planes; }

void lp_norms(const Tensor& pred, const Tensor& tgt, const Tensor& qlat, Tensor& out, Tensor& scratch, int64_t P) {
  MK_CHECK(pred.is_cuda() && pred.is_contiguous() && tgt.is_contiguous() && pred.dim() == 4, "lp_norms: [B,C,H,W] contiguous CUDA expected");
  MK_CHECK(pred.scalar_type() == tgt.scalar_type(), "lp_norms: dtype mismatch");
  MK_CHECK(P == 1 || P == 2, "lp_norms: P must be 1 or 2");
  c10::cuda::CUDAGuard guard(pred.device());
  const int64_t planes = pred.size(0) * pred.size(1), H = pred.size(2), W = pred.size(3);
  MK_CHECK(qlat.numel() == H && qlat.scalar_type() == torch::kFloat32, "lp_norms: qlat must be fp32 [H]");
  MK_CHECK(out.numel() == planes * 2 && out.scalar_type() == torch::kFloat32, "lp_norms: out must be fp32 [B*C,2]");
  MK_CHECK(scratch.numel() >= lp_scratch_floats(planes, H * W) && scratch.scalar_type() == torch::kFloat32, "lp_norms: scratch too small");
  const int is_f32 = pred.scalar_type() == torch::kFloat32;
  MK_CHECK(is_f32 || pred.scalar_type() == torch::kBFloat16, "lp_norms: fp32 or bf16");
  check_cuda(mk::lp_norms(pred.data_ptr(), tgt.data_ptr(), is_f32, qlat.data_ptr<float>(), out.data_ptr<float>(), scratch.data_ptr<float>(),
                          static_cast<int>(planes), static_cast<int>(H), static_cast<int>(W), static_cast<int>(P), cur_stream()),
             "lp_norms");
}

void lp_norms_bwd(const Tensor& pred, const Tensor& tgt, const Tensor& qlat, const Tensor& coef, Tensor& grad, int64_t P) {
  MK_CHECK(pred.is_cuda() && pred.is_contiguous() && tgt.is_contiguous() && grad.is_contiguous(), "lp_norms_bwd: contiguous CUDA expected");
  c10::cuda::CUDAGuard guard(pred.device());
  const int64_t planes = pred.size(0) * pred.size(1), H = pred.size(2), W = pred.size(3);
  MK_CHECK(coef.numel() == planes && coef.scalar_type() == torch::kFloat32 && coef.is_contiguous(), "lp_norms_bwd: coef fp32 [B*C]");
  const int is_f32 = pred.scalar_type() == torch::kFloat32;
  check_cuda(mk::lp_norms_bwd(pred.data_ptr(), tgt.data_ptr(), is_f32, qlat.data_ptr<float>(), coef.data_ptr<float>(), grad.data_ptr(),
                              static_cast<int>(planes), static_cast<int>(H), static_cast<int>(W), static_cast<int>(P), cur_stream()),
             "lp_norms_bwd");
}

// table: int64 tensor [ntensors, 8] on the device holding (p, g, m, v, shadow, n, wd_scale bits, pair_mode)
void adamw_step(const Tensor& table, const Tensor& chunk_tensor, const Tensor& chunk_off, int64_t chunk, const Tensor& hyper) {
  MK_CHECK(table.is_cuda() && table.scalar_type() == torch::kInt64 && table.is_contiguous(), "adamw: bad table");
  static_assert(sizeof(mk::AdamEntry) == 56 || sizeof(mk::AdamEntry) == 64, "AdamEntry layout");
  MK_CHECK(table.size(1) * 8 == (int64_t)sizeof(mk::AdamEntry), "adamw: table row must be ", sizeof(mk::AdamEntry), " bytes");
  c10::cuda::CUDAGuard guard(table.device());
  Tensor ef = err_flag_for(table);
  check_cuda(mk::adamw_step(reinterpret_cast<const mk::AdamEntry*>(table.data_ptr()), chunk_tensor.data_ptr<int>(),
                            reinterpret_cast<const long long*>(chunk_off.data_ptr<int64_t>()), static_cast<int>(chunk_tensor.numel()),
                            chunk, hyper.data_ptr<float>(), ef.data_ptr<int>(), cur_stream()),
             "adamw_step");
}

int64_t adam_entry_bytes() { return sizeof(mk::AdamEntry); }

// ---- mode-wise complex contractions (complex64 tensors, contiguous, mode index last)
static const float* cfp(const Tensor& t) { return reinterpret_cast<const float*>(t.data_ptr()); }
static float* cfpm(Tensor& t) { return reinterpret_cast<float*>(t.data_ptr()); }
static void check_c64(const Tensor& t, const char* what) {
  MK_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == torch::kComplexFloat, what, ": contiguous complex64 CUDA tensor expected");
}

// mode: 0 out = a . w (a [B,I,S], w [I,O,S], out [B,O,S]); 1 da = dy . conj(w) (first arg dy, out da [B,I,S]);
//       2 dw = conj(a) . dy (args a, dy; out [I,O,S])
void modes_diag(const Tensor& x, const Tensor& y, Tensor& out, int64_t B, int64_t I, int64_t O, int64_t S, int64_t mode) {
  check_c64(x, "modes_diag"); check_c64(y, "modes_diag"); check_c64(out, "modes_diag");
  c10::cuda::CUDAGuard guard(x.device());
  cudaError_t e;
  if (mode == 0) {
    MK_CHECK(x.numel() == B * I * S && y.numel() == I * O * S && out.numel() == B * O * S, "modes_diag fwd: shape mismatch");
    e = mk::modes_diag_fwd(cfp(x), cfp(y), cfpm(out), (int)B, (int)I, (int)O, S, cur_stream());
  } else if (mode == 1) {
    MK_CHECK(x.numel() == B * O * S && y.numel() == I * O * S && out.numel() == B * I * S, "modes_diag dgrad: shape mismatch");
    e = mk::modes_diag_dgrad(cfp(x), cfp(y), cfpm(out), (int)B, (int)I, (int)O, S, cur_stream());
  } else {
    MK_CHECK(x.numel() == B * I * S && y.numel() == B * O * S && out.numel() == I * O * S, "modes_diag wgrad: shape mismatch");
    e = mk::modes_diag_wgrad(cfp(x), cfp(y), cfpm(out), (int)B, (int)I, (int)O, S, cur_stream());
  }
  check_cuda(e, "modes_diag");
}

// mode: 0 out = a * w; 1 out = a * conj(w) (a, out [B,I,S]; w [I,S/wdiv]); 2 dw = sum conj(a) dy (args a, dy; out [I,S/wdiv])
void modes_sep(const Tensor& x, const Tensor& y, Tensor& out, int64_t B, int64_t I, int64_t S, int64_t wdiv, int64_t mode) {
  check_c64(x, "modes_sep"); check_c64(y, "modes_sep"); check_c64(out, "modes_sep");
  MK_CHECK(wdiv >= 1 && S % wdiv == 0, "modes_sep: the mode count must be a multiple of wdiv");
  c10::cuda::CUDAGuard guard(x.device());
  cudaError_t e;
  if (mode == 2) {
    MK_CHECK(x.numel() == B * I * S && y.numel() == B * I * S && out.numel() == I * (S / wdiv), "modes_sep wgrad: shape mismatch");
    e = mk::modes_sep_wgrad(cfp(x), cfp(y), cfpm(out), (int)B, (int)I, S, (int)wdiv, cur_stream());
  } else {
    MK_CHECK(x.numel() == B * I * S && y.numel() == I * (S / wdiv) && out.numel() == B * I * S, "modes_sep: shape mismatch");
    e = mk::modes_sep_mul(cfp(x), cfp(y), cfpm(out), (int)B, (int)I, S, (int)wdiv, (int)mode, cur_stream());
  }
  check_cuda(e, "modes_sep");
}

void spectral_expand(const Tensor& w, Tensor& wx) {
  MK_CHECK(w.is_cuda() && w.is_contiguous() && w.scalar_type() == torch::kComplexFloat && w.dim() == 3, "spectral_expand: complex64 [Cin,Cout,L]");
  const int64_t Cin = w.size(0), Cout = w.size(1), L = w.size(2);
  MK_CHECK(wx.is_contiguous() && wx.scalar_type() == torch::kBFloat16 && wx.numel() == 4 * Cin * Cout * L, "spectral_expand: bad wx");
  c10::cuda::CUDAGuard guard(w.device());
  check_cuda(mk::spectral_expand(reinterpret_cast<const float*>(w.data_ptr()), reinterpret_cast<__nv_bfloat16*>(wx.data_ptr()),
                                 static_cast<int>(Cin), static_cast<int>(Cout), static_cast<int>(L), cur_stream()),
             "spectral_expand");
}

void spectral_fold(const Tensor& dwx, Tensor& dw, bool two_block, bool assign) {
  MK_CHECK(dw.is_cuda() && dw.is_contiguous() && dw.scalar_type() == torch::kComplexFloat && dw.dim() == 3, "spectral_fold: complex64 [Cin,Cout,L]");
  const int64_t Cin = dw.size(0), Cout = dw.size(1), L = dw.size(2);
  MK_CHECK(dwx.is_contiguous() && dwx.scalar_type() == torch::kFloat32 && dwx.numel() == (two_block ? 2 : 4) * Cin * Cout * L,
           "spectral_fold: bad dwx");
  c10::cuda::CUDAGuard guard(dw.device());
  check_cuda(mk::spectral_fold(dwx.data_ptr<float>(), reinterpret_cast<float*>(dw.data_ptr()), static_cast<int>(Cin),
                               static_cast<int>(Cout), static_cast<int>(L), cur_stream(), two_block ? 1 : 0, assign ? 1 : 0),
             "spectral_fold");
}

void swap_ri(const Tensor& x, Tensor& y, int64_t C) {
  MK_CHECK(x.is_cuda() && x.is_contiguous() && y.is_contiguous() && x.numel() == y.numel(), "swap_ri: bad tensors");
  MK_CHECK(x.scalar_type() == torch::kBFloat16 && y.scalar_type() == torch::kBFloat16, "swap_ri: bf16 expected");
  MK_CHECK(C > 0 && x.numel() % (2 * C) == 0, "swap_ri: the innermost extent must be (2, C)");
  c10::cuda::CUDAGuard guard(x.device());
  check_cuda(mk::swap_ri_bf16(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), reinterpret_cast<__nv_bfloat16*>(y.data_ptr()),
                              x.numel() / (2 * C), static_cast<int>(C), cur_stream()),
             "swap_ri");
}

void cast_bf16(const Tensor& x, Tensor& y) {
  MK_CHECK(x.is_cuda() && x.is_contiguous() && y.is_contiguous() && x.numel() == y.numel(), "cast_bf16: bad tensors");
  MK_CHECK(x.scalar_type() == torch::kFloat32 && y.scalar_type() == torch::kBFloat16, "cast_bf16: fp32 -> bf16");
  c10::cuda::CUDAGuard guard(x.device());
  check_cuda(mk::cast_f32_bf16(x.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), x.numel(), cur_stream()), "cast_bf16");
}

void fill_normal(Tensor& y, int64_t seed) {
  MK_CHECK(y.is_cuda() && y.is_contiguous() && y.scalar_type() == torch::kBFloat16, "fill_normal: contiguous bf16 CUDA");
  c10::cuda::CUDAGuard guard(y.device());
  check_cuda(mk::fill_normal_bf16(reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), y.numel(), static_cast<uint64_t>(seed), cur_stream()),
             "fill_normal");
}

// ------------------------------------------------------------------------------------------ peer memory

py::bytes peer_alloc(int64_t bytes, py::list out_ptr) {
  void* p = nullptr;
  char handle[64];
  check_cuda(mk::peer_alloc(static_cast<size_t>(bytes), &p, handle), "peer_alloc");
  out_ptr.append(reinterpret_cast<int64_t>(p));
  return py::bytes(handle, 64);
}

int64_t peer_open(py::bytes handle) {
  std::string h = handle;
  MK_CHECK(h.size() == 64, "peer_open: handle must be 64 bytes");
  void* p = nullptr;
  check_cuda(mk::peer_open(h.data(), &p), "peer_open");
  return reinterpret_cast<int64_t>(p);
}

void peer_close(int64_t ptr) { check_cuda(mk::peer_close(reinterpret_cast<void*>(ptr)), "peer_close"); }
void peer_free(int64_t ptr) { check_cuda(mk::peer_free(reinterpret_cast<void*>(ptr)), "peer_free"); }

Tensor tensor_from_ptr(int64_t ptr, int64_t bytes, int64_t device) {
  auto opts = torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, static_cast<int>(device));
  return torch::from_blob(reinterpret_cast<void*>(ptr), {bytes}, opts);
}

// in-place sum over ranks of `data` (fp32 or bf16) living in symmetric memory: ptrs[r] = rank r's copy.
void peer_allreduce(const std::vector<int64_t>& data_ptrs, const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t n,
                    int64_t is_bf16, double scale, double wait_seconds, int64_t device) {
  const int world = static_cast<int>(data_ptrs.size());
  MK_CHECK(world >= 1 && world <= mk::PEER_MAX, "peer_allreduce: world size out of range");
  c10::cuda::CUDAGuard guard(c10::Device(c10::kCUDA, static_cast<int>(device)));
  mk::PeerPtrs pp;
  for (int i = 0; i < world; ++i) {
    pp.data[i] = reinterpret_cast<void*>(data_ptrs[i]);
    pp.flags[i] = reinterpret_cast<unsigned int*>(flag_ptrs[i]);
  }
  Tensor dummy = torch::empty({1}, torch::dtype(torch::kUInt8).device(torch::kCUDA, static_cast<int>(device)));
  Tensor ef = err_flag_for(dummy);
  check_cuda(mk::peer_allreduce(pp, world, static_cast<int>(rank), n, static_cast<int>(is_bf16), static_cast<float>(scale),
                                wait_seconds, ef.data_ptr<int>(), cur_stream()),
             "peer_allreduce");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "tcgen05 GEMM with fused epilogue");
  m.def("gemm_peer", &gemm_peer, "tcgen05 GEMM reading its B operand from peer devices");
  m.def("peer_sum", &peer_sum, "sum of the local segments of a peer buffer with the consumer handshake");
  m.def("peer_publish", &peer_publish, "strided copy into this rank's and its peers' buffers with the producer handshake");
  m.def("set_gelu_tanh", [](int64_t on) { mk::set_gelu_tanh(static_cast<int>(on)); });
  m.def("read_error_flag", &read_error_flag);
  m.def("clear_error_flag", &clear_error_flag);
  m.def("inorm_fwd", &inorm_fwd);
  m.def("inorm_partial_stats", &inorm_partial_stats);
  m.def("inorm_bwd", &inorm_bwd);
  m.def("inorm_cl_sums", &inorm_cl_sums, py::arg("x"), py::arg("dy"), py::arg("w"), py::arg("b"), py::arg("stats"), py::arg("sums"),
        py::arg("dw"), py::arg("db"), py::arg("B"), py::arg("C"), py::arg("act"), py::arg("mode"),
        py::arg("sync") = std::vector<int64_t>(), py::arg("dsts") = std::vector<int64_t>());
  m.def("inorm_cl_apply", &inorm_cl_apply, py::arg("x"), py::arg("dy"), py::arg("out"), py::arg("w"), py::arg("b"), py::arg("sums"),
        py::arg("stats"), py::arg("B"), py::arg("C"), py::arg("count"), py::arg("eps"), py::arg("act"), py::arg("mode"),
        py::arg("sync") = std::vector<int64_t>(), py::arg("srcs") = std::vector<int64_t>());
  m.def("lp_scratch_floats", &lp_scratch_floats);
  m.def("lp_norms", &lp_norms);
  m.def("lp_norms_bwd", &lp_norms_bwd);
  m.def("adamw_step", &adamw_step);
  m.def("modes_diag", &modes_diag);
  m.def("modes_sep", &modes_sep);
  m.def("adam_entry_bytes", &adam_entry_bytes);
  m.def("spectral_expand", &spectral_expand);
  m.def("spectral_fold", &spectral_fold, py::arg("dwx"), py::arg("dw"), py::arg("two_block") = false, py::arg("assign") = false);
  m.def("cast_bf16", &cast_bf16);
  m.def("swap_ri", &swap_ri, "rows of (re, im) -> (im, -re)");
  m.def("fill_normal", &fill_normal);
  m.def("peer_alloc", &peer_alloc);
  m.def("peer_open", &peer_open);
  m.def("peer_close", &peer_close);
  m.def("peer_free", &peer_free);
  m.def("tensor_from_ptr", &tensor_from_ptr);
  m.def("peer_allreduce", &peer_allreduce);
}
