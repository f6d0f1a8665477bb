// Persistent warp-specialised GEMM for sm_100a: TMA -> shared memory (128B swizzle) -> tcgen05.mma with
// accumulators in tensor memory -> tcgen05.ld epilogue with fused bias / GELU / residual / scatter.
//
// Roles per CTA (320 threads, one CTA per SM):
//   warp 0      : TMA producer (one elected lane)
//   warp 1      : TMEM allocator + MMA issuer (one elected lane)
//   warps 2..9  : epilogue; warp w reads TMEM lanes [32*(w%4), 32*(w%4)+32), the two warps that share a lane
//                 quarter take alternating column chunks
//   warp 10     : only in launches whose epilogue operand (residual, saved pre-activation) is prefetched by TMA
//                 (352 threads): its producer, so that waiting for a free operand buffer never delays A and B
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
// Every mbarrier wait is bounded; on expiry the kernel records a code in *err and drains.
//
// CTA pairs (template parameter CG = 2, single-GPU launches only): two CTAs of a thread-block cluster share one
// 256-row tile.  Each CTA loads its own 128 rows of A and HALF of the B tile (plain TMA loads, no multicast, whose
// completion is counted on the leader CTA's barrier); the leader issues tcgen05.mma.cta_group::2, which reads both
// CTAs' shared memory and writes 128 accumulator rows into each CTA's TMEM; tcgen05.commit multicasts the
// "stage free" and "accumulator full" signals to both CTAs.  Per tensor-core cycle every SM then takes a third less
// data from L2 (two thirds with 128-wide tiles), which is what bounds these GEMMs.
//
// Multi-GPU use (one process per GPU, buffers mapped through CUDA IPC):
//   * the k axis of the B operand may be cut into up to 8 segments with their own base pointers and tensor maps
//     (the per-rank segments of a gathered buffer in this device's own memory);
//   * the bf16 output may be replicated into up to 7 more buffers with the layout of D (the same segment of every
//     peer's copy), by plain 16-byte stores or TMA stores over NVLink: no load ever targets peer memory;
//   * producer / consumer ordering across devices uses monotonic counters (PeerSync) checked by the first thread of
//     every CTA before any work and advanced by the last CTA of the grid.
#include "gemm_tcgen05.cuh"
#include "gelu.cuh"
#include "fused_ops.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace mk {

namespace {

constexpr int BM = 128;
constexpr int A_STAGE_BYTES = BM * 128;
constexpr int NUM_THREADS = 320;   // TMA warp + MMA warp + 8 epilogue warps
constexpr int E_WARP = 10;         // launches with a TMA-fed epilogue operand run an eleventh warp: its producer
constexpr int MAX_STAGES = 6;
constexpr int MAX_SEG = 8;

// Handshake of a kernel that consumes buffers its peers have filled and/or fills a buffer that its peers consume.
//   wait[i]   : local flag array (one slot per peer) that must reach *wait_exp[i] + wait_off[i] before the first load
//   bump[i]   : local counter incremented by one when the whole grid has finished
//   sig[i][p] : flag slot in peer p's memory incremented by one when the whole grid has finished
struct PeerSync {
  int np_wait[2], np_sig[2];      // number of peers of the group each wait / signal list refers to
  int nwait, nsig;
  const unsigned int* wait[2];
  const unsigned int* wait_exp[2];
  int wait_off[2];
  unsigned int* bump[2];
  unsigned int* sig[2][MAX_SEG];
  unsigned int* done_ctr;
};

struct BMaps {
  CUtensorMap m[MAX_SEG];
};
// tensor maps of the additional destinations (the same output written into peers' memory)
struct DMaps {
  CUtensorMap m[MAX_SEG - 1];
};
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;   // 2 s per barrier wait

struct KParams {
  int M, N, K;
  int zlo_n, zhi_n;
  int splits, k_per_split;
  int a_mn, b_mn;
  int a_zlo, a_zhi, b_zlo, b_zhi;
  int rmin_a, rmin_b, rmax_a, rmax_b, kmin_a, kmin_b, kmax_a, kmax_b;
  long long d_zlo, d_zhi;
  int rdiv; long long rs_hi, rs_lo;
  int ndiv; long long ns_hi;
  float alpha;
  const float* bias;
  long long bias_zs;              // elements between the bias vectors of consecutive z_lo batches (0: one shared vector)
  int bias_mode, act, save_deriv;
  GeluCoef gelu;
  float act_param;
  const void* resid;
  void* preact;
  void* D;
  int out_f32, accumulate, vec_ok;
  int m_tiles, n_tiles;
  long long total_tiles;
  int stages, e_tma, plain_cols;
  int n_fast;                     // tile order: 1 = n-tile index fastest, 0 = m-tile index fastest
  int* err;
  // ---- B operand gathered from several devices: segment s of the k axis was written by rank s into the local buffer
  int nseg;                       // 1: ordinary single-map operand
  int seg_len[MAX_SEG];           // local k extent of each segment
  int seg_apos[MAX_SEG];          // k coordinate of the segment start in the A operand (padded layout)
  int seg_gstart[MAX_SEG];        // global k index of the segment start (for the kmin/kmax structure)
  // ---- output replicated into peers' memory: ndx additional destinations with the layout of D
  int ndx;
  void* Dx[MAX_SEG - 1];
  // ---- cross-device handshakes (all counters are monotonic and live in device memory)
  PeerSync sync;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Bounded wait: polls the barrier and gives up after WAIT_LIMIT_NS of wall time. Returns false on expiry.
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// The suspend-time hint lets the hardware park a waiting thread until the phase completes (it wakes at once when it
// does) instead of returning to the polling loop every few dozen cycles: the three single-thread roles of a CTA spend
// most of their time waiting, and their polling instructions competed with the epilogue warps for issue slots.
constexpr uint32_t MBAR_SUSPEND_HINT_NS = 4000;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P1;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, P1;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(MBAR_SUSPEND_HINT_NS)
        : "memory");
    if (ok) return true;
    if ((it & 63u) == 63u) {
      const uint64_t now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) return false;
    }
  }
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// CTA-pair form: the destination is this CTA's shared memory, the barrier that counts the bytes lives in the leader CTA
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int c0, int c1,
                                                 int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map), "r"(src),
               "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// pair form: arrives on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const unsigned short mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}

template <int EB, int CG>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accum) {
  if constexpr (EB == 2 && CG == 2) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accum)
        : "memory");
  } else if constexpr (EB == 2) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accum)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accum)
        : "memory");
  }
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 version field = 1.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;   // descriptor version
  d |= static_cast<uint64_t>(2) << 61;   // SWIZZLE_128B
  return d;
}

struct TileCoord {
  int zhi, zlo, split, mt, nt;
  int k_begin, k_end;   // element range, k_begin multiple of BK
  bool skip;
};

// CG = 2: `t` counts 256-row pair tiles (p.m_tiles is then the number of pair tiles) and `half` (0 / 1) selects this
// CTA's 128 rows; skip decisions are taken for the pair as a whole because the MMA is issued once for both CTAs.
template <int BK, int CG = 1>
__device__ __forceinline__ TileCoord decode_tile(const KParams& p, long long t, int half = 0) {
  TileCoord c;
  // The index that varies fastest walks over the tiles that share the larger operand, so that the CTAs of one wave
  // fetch that operand's tile from DRAM once and hit L2 for the rest (token-major convolutions: many m-tiles of
  // activations against two to six n-tiles of weights -> n fastest).
  if (p.n_fast) {
    c.nt = static_cast<int>(t % p.n_tiles);
    t /= p.n_tiles;
    c.mt = static_cast<int>(t % p.m_tiles);
    t /= p.m_tiles;
  } else {
    c.mt = static_cast<int>(t % p.m_tiles);
    t /= p.m_tiles;
    c.nt = static_cast<int>(t % p.n_tiles);
    t /= p.n_tiles;
  }
  c.split = static_cast<int>(t % p.splits);
  t /= p.splits;
  c.zlo = static_cast<int>(t % p.zlo_n);
  c.zhi = static_cast<int>(t / p.zlo_n);
  const int rmin = p.rmin_a * c.zhi + p.rmin_b;
  const int rmax = p.rmax_a * c.zhi + p.rmax_b;
  int kmin = p.kmin_a * c.zhi + p.kmin_b;
  int kmax = p.kmax_a * c.zhi + p.kmax_b;
  if (kmin < 0) kmin = 0;
  if (kmax > p.K) kmax = p.K;
  int kb = c.split * p.k_per_split;
  int ke = kb + p.k_per_split;
  if (ke > p.K) ke = p.K;
  const int kmin_al = (kmin / BK) * BK;
  if (kb < kmin_al) kb = kmin_al;
  if (ke > kmax) ke = kmax;
  c.k_begin = kb;
  c.k_end = ke;
  const int r0 = c.mt * (BM * CG);
  c.skip = (r0 + BM * CG <= rmin) || (r0 >= rmax) || (p.nseg == 1 && kb >= ke);
  if constexpr (CG == 2) c.mt = c.mt * 2 + half;   // from here on: this CTA's own 128-row block
  return c;
}

// Specialised epilogues stage their output for TMA stores in 32-row x 128-byte boxes, two per epilogue warp.  The
// epilogues with a TMA-fed operand (3, 4) run 128-column tiles, where a warp writes one box per tile: its previous
// store left the box a whole tile ago, so one box is enough and the other 32 KB go to a further operand stage.
__host__ __device__ constexpr int stg_warp_bytes(int epi) { return (epi == 3 || epi == 4) ? 32 * 128 : 2 * 32 * 128; }
__host__ __device__ constexpr int stg_bytes(int epi) { return epi == 0 ? 0 : 8 * stg_warp_bytes(epi); }

// EPI selects a compile-time specialised epilogue (bf16 output, 16-byte vector stores, row bias only):
//   0 generic (all options decided at run time)      1 plain store
//   2 GELU + saved pre-activation                     3 + residual (TMA-prefetched)      4 * GELU'(aux) (TMA-prefetched)
// local k range [lb, le) of segment `sg` for tile `c` (multi-device B operand)
template <int BK>
__device__ __forceinline__ void seg_range(const KParams& p, const TileCoord& c, int sg, int& lb, int& le) {
  int kmin = p.kmin_a * c.zhi + p.kmin_b - p.seg_gstart[sg];
  int kmax = p.kmax_a * c.zhi + p.kmax_b - p.seg_gstart[sg];
  lb = kmin > 0 ? (kmin / BK) * BK : 0;
  le = kmax < p.seg_len[sg] ? kmax : p.seg_len[sg];
}

__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* ptr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}

template <int BN, int EB, int EPI, int CG>
__global__ void __launch_bounds__(NUM_THREADS + 32, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ BMaps maps_b,
            const __grid_constant__ CUtensorMap map_e, const __grid_constant__ CUtensorMap map_d,
            const __grid_constant__ CUtensorMap map_p, const __grid_constant__ DMaps maps_dx, const KParams p) {
  const CUtensorMap& map_b = maps_b.m[0];
  constexpr int BK = 128 / EB;            // elements per 128-byte k-slab
  constexpr int UMMA_K = 32 / EB;         // elements per tcgen05.mma
  constexpr int BNL = BN / CG;            // rows of the B tile this CTA loads (a pair splits the tile)
  constexpr int B_STAGE_BYTES = BNL * 128;
  constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  constexpr int MN_BOX = 128 / EB;        // extent of an MN-major box along the contiguous dimension
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr int E_BYTES = BM * BN * 2;    // bf16 epilogue-operand tile
  const int STAGES = p.stages;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;

  // layout: [stages][E tile x2 (optional)][staging][barriers]
  const uint32_t e_off = STAGES * STAGE_BYTES;
  const uint32_t stg_off = e_off + (p.e_tma ? 2 * E_BYTES : 0);
  const uint32_t bar_off = stg_off + stg_bytes(EPI);
  uint8_t* bar_ptr = smem + bar_off;
  const uint32_t bar_base = smem_base + bar_off;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + 2 + b); };
  auto efull_bar = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + 4 + b); };
  auto eempty_bar = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + 6 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 8 * (2 * MAX_STAGES + 8));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // pair geometry: `crank` = rank inside the cluster (the leader is rank 0), tiles are dealt out per cluster
  const int crank = (CG == 2) ? static_cast<int>(cluster_ctarank()) : 0;
  const long long tile0 = (CG == 2) ? (blockIdx.x >> 1) : blockIdx.x;
  const long long tile_step = (CG == 2) ? (gridDim.x >> 1) : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8 * CG);
      mbar_init(efull_bar(b), 1);
      mbar_init(eempty_bar(b), 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // segments written by the peers (and the peers' copies this kernel overwrites) must be ready: bounded wait on local flags.
    // The whole CTA waits (not only the producer) so that no epilogue store of an all-zero tile can run early.
    bool ok = true;
    for (int w = 0; w < p.sync.nwait && ok; ++w) {
      const unsigned int need = *p.sync.wait_exp[w] + static_cast<unsigned int>(p.sync.wait_off[w]);
      for (int peer = 0; peer < p.sync.np_wait[w] && ok; ++peer) {
        uint64_t t0 = 0;
        for (uint32_t it = 0;; ++it) {
          if (static_cast<int>(ld_acquire_sys_u32(p.sync.wait[w] + peer) - need) >= 0) break;
          if ((it & 255u) == 255u) {
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS) {
              atomicExch(p.err, 32 + w);
              ok = false;
              break;
            }
          }
        }
      }
    }
    tmem_slot[1] = ok ? 1u : 0u;
  }
  if (warp == 1) {
    if constexpr (CG == 2) {
      // the same warp of both CTAs allocates, with the same destination offset
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(const_cast<uint32_t*>(tmem_slot))),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(const_cast<uint32_t*>(tmem_slot))),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();   // the partner's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool peers_ready = tmem_slot[1] != 0u;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = peers_ready;
      if (p.sync.nwait > 0) asm volatile("fence.proxy.async;" ::: "memory");   // flags acquired in the prologue order the TMA loads below
      // pair: every load of both CTAs is counted on the leader's "full" barrier
      const uint32_t leader_full0 = (CG == 2) ? mapa_u32(full_bar(0), 0) : 0u;
      for (long long t = tile0; t < p.total_tiles && ok; t += tile_step) {
        const TileCoord c = decode_tile<BK, CG>(p, t, crank);
        const int m0 = c.mt * BM, n0 = c.nt * BN;
        if (c.skip) continue;
        const int azl = p.a_zlo ? c.zlo : 0, azh = p.a_zhi ? c.zhi : 0;
        const int bzl = p.b_zlo ? c.zlo : 0, bzh = p.b_zhi ? c.zhi : 0;
        for (int sg = 0; sg < p.nseg && ok; ++sg) {
          int lb = c.k_begin, le = c.k_end, apos = 0;
          const CUtensorMap* mb = &map_b;
          if (p.nseg > 1) {
            seg_range<BK>(p, c, sg, lb, le);
            apos = p.seg_apos[sg];
            mb = &maps_b.m[sg];
          }
          for (int k = lb; k < le; k += BK) {
            if (!mbar_wait(empty_bar(s), ph ^ 1u)) {
              atomicExch(p.err, 1);
              ok = false;
              break;
            }
            const uint32_t sa = smem_base + s * STAGE_BYTES;
            const uint32_t sb = sa + A_STAGE_BYTES;
            const int ka = apos + k;
            if constexpr (CG == 2) {
              // the leader announces the bytes of both CTAs; the partner's loads may land first (the barrier's byte
              // count goes negative for a moment, its phase cannot complete before the leader's arrival)
              if (crank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
              const uint32_t lbar = leader_full0 + 8u * s;
              const int nb0 = n0 + crank * BNL;
              if (!p.a_mn) {
                tma_load_4d_pair(sa, &map_a, lbar, ka, m0, azl, azh);
              } else {
#pragma unroll
                for (int j = 0; j < BM / MN_BOX; ++j)
                  tma_load_4d_pair(sa + j * (BK * 128), &map_a, lbar, m0 + j * MN_BOX, ka, azl, azh);
              }
              if (!p.b_mn) {
                tma_load_4d_pair(sb, mb, lbar, k, nb0, bzl, bzh);
              } else {
#pragma unroll
                for (int j = 0; j < BNL / MN_BOX; ++j)
                  tma_load_4d_pair(sb + j * (BK * 128), mb, lbar, nb0 + j * MN_BOX, k, bzl, bzh);
              }
            } else {
              mbar_expect_tx(full_bar(s), STAGE_BYTES);
              if (!p.a_mn) {
                tma_load_4d(sa, &map_a, full_bar(s), ka, m0, azl, azh);
              } else {
#pragma unroll
                for (int j = 0; j < BM / MN_BOX; ++j)
                  tma_load_4d(sa + j * (BK * 128), &map_a, full_bar(s), m0 + j * MN_BOX, ka, azl, azh);
              }
              if (!p.b_mn) {
                tma_load_4d(sb, mb, full_bar(s), k, n0, bzl, bzh);
              } else {
#pragma unroll
                for (int j = 0; j < BN / MN_BOX; ++j)
                  tma_load_4d(sb + j * (BK * 128), mb, full_bar(s), n0 + j * MN_BOX, k, bzl, bzh);
              }
            }
            if (++s == STAGES) {
              s = 0;
              ph ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == E_WARP) {
    // ------------------------------------------------------------------ producer of the epilogue operand
    // A warp of its own: the tile of the residual / saved pre-activation for tile t+2 can only be requested when the
    // epilogue of tile t has released its buffer.  Issued from the operand producer's loop, that wait held back the
    // A and B loads of the tiles in between; issued from another lane of the producer warp, its polling held up that
    // warp's TMA issue.
    if (lane == 0 && p.e_tma && peers_ready) {
      if (p.sync.nwait > 0) asm volatile("fence.proxy.async;" ::: "memory");
      uint32_t epi_it = 0;
      for (long long t = tile0; t < p.total_tiles; t += tile_step) {
        const TileCoord c = decode_tile<BK, CG>(p, t, crank);
        if (c.skip && p.accumulate) continue;
        const int eb = epi_it & 1;
        if (!mbar_wait(eempty_bar(eb), ((epi_it >> 1) & 1u) ^ 1u)) {
          atomicExch(p.err, 5);
          break;
        }
        mbar_expect_tx(efull_bar(eb), E_BYTES);
#pragma unroll
        for (int j = 0; j < BN / 64; ++j)
          tma_load_4d(smem_base + e_off + eb * E_BYTES + j * (BM * 128), &map_e, efull_bar(eb), c.nt * BN + j * 64, c.mt * BM,
                      c.zlo, c.zhi);
        ++epi_it;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && crank == 0) {
      // instruction descriptor: fp32 accumulate, operand format, majors, N, M (256 rows for a CTA pair)
      const uint32_t fmt = (EB == 2) ? 1u : 2u;   // BF16 : TF32
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(p.a_mn) << 15) |
                             (static_cast<uint32_t>(p.b_mn) << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
                             (static_cast<uint32_t>((BM * CG) >> 4) << 24);
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, a_sbo = 1024;
      const uint32_t b_lbo = p.b_mn ? BK * 128 : 16, b_sbo = 1024;
      const uint32_t a_kstep = p.a_mn ? UMMA_K * 128 : 32;
      const uint32_t b_kstep = p.b_mn ? UMMA_K * 128 : 32;
      int s = 0;
      uint32_t ph = 0, acc_it = 0;
      bool ok = peers_ready;
      for (long long t = tile0; t < p.total_tiles && ok; t += tile_step) {
        const TileCoord c = decode_tile<BK, CG>(p, t, crank);
        if (c.skip) continue;
        const int buf = acc_it & 1;
        if (!mbar_wait(tempty_bar(buf), ((acc_it >> 1) & 1u) ^ 1u)) {
          atomicExch(p.err, 2);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        uint32_t accum = 0;
        int nblocks = 0;
        if (p.nseg > 1) {
          for (int sg = 0; sg < p.nseg; ++sg) {
            int lb, le;
            seg_range<BK>(p, c, sg, lb, le);
            if (le > lb) nblocks += (le - lb + BK - 1) / BK;
          }
        } else {
          nblocks = (c.k_end - c.k_begin + BK - 1) / BK;
        }
        for (int kb = 0; kb < nblocks; ++kb) {
          if (!mbar_wait(full_bar(s), ph)) {
            atomicExch(p.err, 3);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = make_desc(sa + kk * a_kstep, a_lbo, a_sbo);
            const uint64_t db = make_desc(sb + kk * b_kstep, b_lbo, b_sbo);
            tc_mma<EB, CG>(tmem_d, da, db, idesc, accum);
            accum = 1;
          }
          // frees the smem stage (in both CTAs of a pair) once these MMAs have read it
          if constexpr (CG == 2) tc_commit_pair(empty_bar(s));
          else tc_commit(empty_bar(s));
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        if constexpr (CG == 2) tc_commit_pair(tfull_bar(buf));   // accumulator complete (both halves)
        else tc_commit(tfull_bar(buf));
        ++acc_it;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    // Eight warps: warp w serves TMEM lanes [32*(w%4), +32) (one accumulator row per thread) and the 32-column
    // chunks with (chunk % 2) == (w-2)/4, so two warps per scheduler hide each other's latency.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t acc_it = 0, epi_it = 0;
    bool ok = peers_ready;
    // the "accumulator drained" barrier of a pair lives in the leader and counts the warps of both CTAs
    const uint32_t leader_tempty0 = (CG == 2) ? mapa_u32(tempty_bar(0), 0) : 0u;
    for (long long t = tile0; t < p.total_tiles; t += tile_step) {
      const TileCoord c = decode_tile<BK, CG>(p, t, crank);
      if (c.skip && p.accumulate) continue;
      const int rt = q * 32 + lane;                 // row inside the tile
      const int r = c.mt * BM + rt;
      const int n0 = c.nt * BN;
      const bool row_ok = r < p.M;
      const long long row_off = static_cast<long long>(c.zhi) * p.d_zhi + static_cast<long long>(c.zlo) * p.d_zlo +
                                static_cast<long long>(r / p.rdiv) * p.rs_hi + static_cast<long long>(r % p.rdiv) * p.rs_lo;
      const float* const bias_z = p.bias + static_cast<long long>(c.zlo) * p.bias_zs;
      float rbias = 0.f;
      if (p.bias_mode == 1 && row_ok) rbias = __ldg(bias_z + r);
      int buf = 0, ebuf = 0;
      if (!c.skip) {
        buf = acc_it & 1;
        if (ok && !mbar_wait(tfull_bar(buf), (acc_it >> 1) & 1u)) {
          atomicExch(p.err, 4);
          ok = false;
        }
        tc_fence_after();
      }
      const uint8_t* esm = nullptr;
      if (p.e_tma) {
        ebuf = epi_it & 1;
        if (ok && !mbar_wait(efull_bar(ebuf), (epi_it >> 1) & 1u)) {
          atomicExch(p.err, 6);
          ok = false;
        }
        esm = smem + e_off + ebuf * E_BYTES;
      }
      if constexpr (EPI != 0) {
        // ---------------- specialised bf16 epilogues: registers -> swizzled smem box -> TMA store (full lines, clipped
        // at the matrix edge by the tensor map)
        constexpr bool ONE_BOX = (EPI == 3 || EPI == 4);
        const uint32_t stg_base = smem_base + stg_off + (warp - 2) * stg_warp_bytes(EPI);
        uint8_t* const stg_ptr = smem + stg_off + (warp - 2) * stg_warp_bytes(EPI);
        int sb = 0;
#pragma unroll 1
        for (int bx = half; bx < BN / 64; bx += 2) {
          const int nb = n0 + bx * 64;
          if (nb >= p.N) break;
          const uint32_t taddr = tmem_base + buf * BN + bx * 64 + (static_cast<uint32_t>(q * 32) << 16);
          // the staging box written two stores ago (one for the two-output epilogue) must have been read out
          if constexpr (EPI == 2 || ONE_BOX) tma_store_wait_read<0>();
          else tma_store_wait_read<1>();
          __syncwarp();
          uint8_t* const box_d = stg_ptr + (EPI == 2 ? 32 * 128 : (ONE_BOX ? 0 : sb * 32 * 128));
          uint8_t* const box_p = stg_ptr;
          // The 64 columns of a box go through a ROLLED loop of four 16-column steps.  Unrolled, the body of one box ran
          // to tens of KB of straight-line code per epilogue flavour, the eight epilogue warps (each at another place
          // in it) missed the instruction caches on most fetches, and "no instruction" was their top stall reason.
#pragma unroll 1
          for (int it = 0; it < 4; ++it) {
          uint32_t v[16];
          if (!c.skip) {
            tmem_ld16(taddr + it * 16, v);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0u;
          }
#pragma unroll
          for (int gg = 0; gg < 2; ++gg) {
            const int g = it * 2 + gg;
            const int n = nb + g * 8;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = rbias;
            if (p.bias_mode == 2) {      // the column bias rides on the scaling fma below
              if (n + 8 <= p.N) {
                const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias_z + n));
                const float4 b1 = __ldg(reinterpret_cast<const float4*>(bias_z + n) + 1);
                f[0] = b0.x; f[1] = b0.y; f[2] = b0.z; f[3] = b0.w;
                f[4] = b1.x; f[5] = b1.y; f[6] = b1.z; f[7] = b1.w;
              } else {
                for (int j = 0; j < 8 && n + j < p.N; ++j) f[j] = __ldg(bias_z + n + j);
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = fmaf(__uint_as_float(v[gg * 8 + j]), p.alpha, f[j]);
            const uint32_t sw = static_cast<uint32_t>((g ^ (lane & 7)) << 4) + lane * 128;
            if constexpr (EPI == 1) {
              if (p.act != 0) {      // ReLU / soft shrinkage (uniform over the launch)
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = act_fwd(f[j], p.act, p.act_param, p.gelu);
              }
            }
            if constexpr (EPI == 2) {
              __nv_bfloat162 h[4];
              if (p.save_deriv) {      // uniform over the launch: second output = GELU'(pre-activation)
                float d[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) gelu_fwd_bwd(f[j], p.gelu, f[j], d[j]);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(d[2 * j], d[2 * j + 1]);
                *reinterpret_cast<uint4*>(box_p + sw) = *reinterpret_cast<uint4*>(h);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
                *reinterpret_cast<uint4*>(box_p + sw) = *reinterpret_cast<uint4*>(h);
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = gelu_fwd(f[j], p.gelu);
              }
            }
            if constexpr (EPI == 3 || EPI == 4) {
              const uint4 ev = *reinterpret_cast<const uint4*>(esm + bx * (BM * 128) + rt * 128 + ((g ^ (rt & 7)) << 4));
              const __nv_bfloat162* eh = reinterpret_cast<const __nv_bfloat162*>(&ev);
              if constexpr (EPI == 3) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 x = __bfloat1622float2(eh[j]);
                  f[2 * j] += x.x;
                  f[2 * j + 1] += x.y;
                }
              } else if (p.act == 8) {      // uniform over the launch: the operand is the saved derivative
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 x = __bfloat1622float2(eh[j]);
                  f[2 * j] *= x.x;
                  f[2 * j + 1] *= x.y;
                }
              } else if (p.act == 2) {      // uniform over the launch: the GELU case carries no per-element selects
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 x = __bfloat1622float2(eh[j]);
                  f[2 * j] *= gelu_bwd(x.x, p.gelu);
                  f[2 * j + 1] *= gelu_bwd(x.y, p.gelu);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 x = __bfloat1622float2(eh[j]);
                  f[2 * j] *= act_bwd(x.x, p.act, p.gelu);
                  f[2 * j + 1] *= act_bwd(x.y, p.act, p.gelu);
                }
              }
            }
            __nv_bfloat162 h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
            *reinterpret_cast<uint4*>(box_d + sw) = *reinterpret_cast<uint4*>(h);
          }
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int r0 = c.mt * BM + q * 32;
            if (r0 < p.M) {
              if constexpr (EPI == 2) tma_store_4d(&map_p, stg_base, nb, r0, c.zlo, c.zhi);
              tma_store_4d(&map_d, stg_base + (EPI == 2 ? 32 * 128 : (ONE_BOX ? 0 : sb * 32 * 128)), nb, r0, c.zlo, c.zhi);
              if constexpr (EPI == 1) {
                for (int dq = 0; dq < p.ndx; ++dq)   // the same box goes to every peer's copy (plain stores over NVLink)
                  tma_store_4d(&maps_dx.m[dq], stg_base + sb * 32 * 128, nb, r0, c.zlo, c.zhi);
              }
            }
            tma_store_commit();
          }
          sb ^= 1;
        }
      } else
#pragma unroll 1
      for (int cc = half; cc < BN / 32; cc += 2) {
        const int nc = n0 + cc * 32;
        if (nc >= p.N) break;       // uniform across the warp
        const uint32_t taddr = tmem_base + buf * BN + cc * 32 + (static_cast<uint32_t>(q * 32) << 16);
        // rolled: one copy of the (large, many-layout) body serves the four 8-column groups, which keeps the
        // epilogue within the instruction cache
#pragma unroll 1
        for (int g = 0; g < 4; ++g) {
          const int n = nc + g * 8;
          if (n >= p.N) break;      // uniform across the warp
          uint32_t v[8];
          if (!c.skip) {
            tmem_ld8(taddr + g * 8, v);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0u;
          }
          if (!row_ok) continue;
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[j]) * p.alpha;
          if (p.bias_mode == 1) {
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] += rbias;
          } else if (p.bias_mode == 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (n + j < p.N) f[j] += __ldg(bias_z + n + j);
          }
          const bool full = (n + 8 <= p.N);
          const long long off = row_off + static_cast<long long>(n / p.ndiv) * p.ns_hi + (n % p.ndiv);
          // epilogue operand for these 8 columns (bf16 tile prefetched by TMA, 128-byte swizzle: the 16-byte chunk
          // index inside each 128-byte row segment is XORed with (row % 8))
          float e8[8];
          if (p.e_tma) {
            const int col = cc * 32 + g * 8;                     // column inside the tile
            const int box = col >> 6, chunk = (col & 63) >> 3;
            const uint4 ev = *reinterpret_cast<const uint4*>(esm + box * (BM * 128) + rt * 128 + ((chunk ^ (rt & 7)) << 4));
            const __nv_bfloat162* eh = reinterpret_cast<const __nv_bfloat162*>(&ev);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 x = __bfloat1622float2(eh[j]);
              e8[2 * j] = x.x;
              e8[2 * j + 1] = x.y;
            }
          }
          if (full && p.vec_ok && !p.accumulate) {
            // ---- vector path: 8 consecutive columns
            if (p.preact) {
              float s8[8];     // second output: the pre-activation, or GELU' of it
#pragma unroll
              for (int j = 0; j < 8; ++j) s8[j] = p.save_deriv ? gelu_bwd(f[j], p.gelu) : f[j];
              if (p.out_f32) {
                float4* o = reinterpret_cast<float4*>(static_cast<float*>(p.preact) + off);
                o[0] = make_float4(s8[0], s8[1], s8[2], s8[3]);
                o[1] = make_float4(s8[4], s8[5], s8[6], s8[7]);
              } else {
                __nv_bfloat162 h[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(s8[2 * j], s8[2 * j + 1]);
                *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.preact) + off) = *reinterpret_cast<uint4*>(h);
              }
            }
            if (p.act & 1) {
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = act_fwd(f[j], p.act, p.act_param, p.gelu);
            }
            if (p.resid) {
              if (!p.e_tma) {
                if (p.out_f32) {
                  const float4* ri = reinterpret_cast<const float4*>(static_cast<const float*>(p.resid) + off);
                  const float4 a = ri[0], b = ri[1];
                  e8[0] = a.x; e8[1] = a.y; e8[2] = a.z; e8[3] = a.w;
                  e8[4] = b.x; e8[5] = b.y; e8[6] = b.z; e8[7] = b.w;
                } else {
                  const uint4 rv = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.resid) + off);
                  const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 x = __bfloat1622float2(rh[j]);
                    e8[2 * j] = x.x;
                    e8[2 * j + 1] = x.y;
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = (p.act != 0 && !(p.act & 1)) ? f[j] * act_bwd(e8[j], p.act, p.gelu) : f[j] + e8[j];
            }
            if (p.out_f32) {
              float4* o = reinterpret_cast<float4*>(static_cast<float*>(p.D) + off);
              o[0] = make_float4(f[0], f[1], f[2], f[3]);
              o[1] = make_float4(f[4], f[5], f[6], f[7]);
            } else {
              __nv_bfloat162 h[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.D) + off) = *reinterpret_cast<uint4*>(h);
              for (int dq = 0; dq < p.ndx; ++dq)
                *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.Dx[dq]) + off) = *reinterpret_cast<uint4*>(h);
            }
          } else if (full && p.vec_ok && p.accumulate && p.out_f32 && !p.preact && p.act == 0) {
            // ---- split-k / batch accumulation in fp32: two 16-byte vector atomics instead of eight scalar ones
            float4* o = reinterpret_cast<float4*>(static_cast<float*>(p.D) + off);
            atomicAdd(o, make_float4(f[0], f[1], f[2], f[3]));
            atomicAdd(o + 1, make_float4(f[4], f[5], f[6], f[7]));
          } else {
            // ---- scalar path (ragged edge, unaligned layouts, atomic accumulation)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int nj = n + j;
              if (nj >= p.N) break;
              const long long o = row_off + static_cast<long long>(nj / p.ndiv) * p.ns_hi + (nj % p.ndiv);
              float x = f[j];
              if (p.preact) {
                const float sx = p.save_deriv ? gelu_bwd(x, p.gelu) : x;
                if (p.out_f32) static_cast<float*>(p.preact)[o] = sx;
                else static_cast<__nv_bfloat16*>(p.preact)[o] = __float2bfloat16(sx);
              }
              if (p.act & 1) x = act_fwd(x, p.act, p.act_param, p.gelu);
              if (p.accumulate) {
                atomicAdd(static_cast<float*>(p.D) + o, x);
              } else {
                if (p.resid) {
                  float rr;
                  if (p.e_tma) rr = e8[j];
                  else rr = p.out_f32 ? static_cast<const float*>(p.resid)[o]
                                      : __bfloat162float(static_cast<const __nv_bfloat16*>(p.resid)[o]);
                  x = (p.act != 0 && !(p.act & 1)) ? x * act_bwd(rr, p.act, p.gelu) : x + rr;
                }
                if (p.out_f32) static_cast<float*>(p.D)[o] = x;
                else {
                  static_cast<__nv_bfloat16*>(p.D)[o] = __float2bfloat16(x);
                  for (int dq = 0; dq < p.ndx; ++dq) static_cast<__nv_bfloat16*>(p.Dx[dq])[o] = __float2bfloat16(x);
                }
              }
            }
          }
        }
      }
      if (!c.skip) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 2) mbar_arrive_cluster(leader_tempty0 + 8u * buf);
          else mbar_arrive(tempty_bar(buf));
        }
        ++acc_it;
      }
      if (p.e_tma) {
        __syncwarp();
        if (lane == 0) mbar_arrive(eempty_bar(ebuf));
        ++epi_it;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if constexpr (EPI != 0) {
    if (warp >= 2 && warp < E_WARP && lane == 0) {
      tma_store_wait_all();
      asm volatile("fence.proxy.async;" ::: "memory");   // order the bulk stores before the generic-proxy signalling below
    }
  }
  tc_fence_before();
  __syncthreads();
  if (p.sync.done_ctr != nullptr && threadIdx.x == 0) {
    // last CTA of the grid: everything this kernel wrote (here and into the peers' copies) is complete and everything it
    // consumed may be overwritten
    __threadfence_system();
    const unsigned int prev = atomicAdd(p.sync.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *p.sync.done_ctr = 0;
      // after an expired wait nothing is published: the counters keep describing the last complete generation
      if (*reinterpret_cast<volatile int*>(p.err) == 0) {
        for (int i = 0; i < p.sync.nwait; ++i)
          if (p.sync.bump[i]) atomicAdd(p.sync.bump[i], 1u);
        __threadfence_system();
        for (int i = 0; i < p.sync.nsig; ++i)
          for (int peer = 0; peer < p.sync.np_sig[i]; ++peer)
            if (p.sync.sig[i][peer]) atomicAdd_system(p.sync.sig[i][peer], 1u);
      }
    }
  }
  if constexpr (CG == 2) cluster_sync_all();   // neither CTA leaves (or frees TMEM) while its partner may still touch it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (CG == 2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

char g_err[512] = {0};

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || sym == nullptr) return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

bool make_map(CUtensorMap* map, const GemmOperand& op, int K, int eb, int zlo_n, int zhi_n, int box_rows_kmajor) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    snprintf(g_err, sizeof(g_err), "cuTensorMapEncodeTiled entry point not available");
    return false;
  }
  const int bk = 128 / eb;
  cuuint64_t dims[4];
  cuuint64_t strides[3];
  cuuint32_t box[4];
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const bool use_lo = (op.zs_lo != 0) && zlo_n > 1;
  const bool use_hi = (op.zs_hi != 0) && zhi_n > 1;
  if (!op.mn_major) {
    dims[0] = static_cast<cuuint64_t>(K);
    dims[1] = static_cast<cuuint64_t>(op.rows);
    box[0] = bk;
    box[1] = box_rows_kmajor;
  } else {
    dims[0] = static_cast<cuuint64_t>(op.rows);
    dims[1] = static_cast<cuuint64_t>(K);
    box[0] = 128 / eb;
    box[1] = bk;
  }
  dims[2] = use_lo ? zlo_n : 1;
  dims[3] = use_hi ? zhi_n : 1;
  box[2] = 1;
  box[3] = 1;
  strides[0] = static_cast<cuuint64_t>(op.ld) * eb;
  strides[1] = use_lo ? static_cast<cuuint64_t>(op.zs_lo) * eb : strides[0];
  strides[2] = use_hi ? static_cast<cuuint64_t>(op.zs_hi) * eb : strides[0];
  if ((reinterpret_cast<uintptr_t>(op.ptr) & 15) || (strides[0] & 15) || (strides[1] & 15) || (strides[2] & 15)) {
    snprintf(g_err, sizeof(g_err), "gemm operand not 16-byte aligned (ptr %p ld %lld zs %lld %lld)", op.ptr, op.ld,
             op.zs_lo, op.zs_hi);
    return false;
  }
  CUresult r = enc(map, eb == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
                   const_cast<void*>(op.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_err, sizeof(g_err),
             "cuTensorMapEncodeTiled failed (%d): dims %llu %llu %llu %llu strides %llu %llu %llu box %u %u", (int)r,
             (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
             (unsigned long long)dims[3], (unsigned long long)strides[0], (unsigned long long)strides[1],
             (unsigned long long)strides[2], box[0], box[1]);
    return false;
  }
  return true;
}

constexpr int SMEM_LIMIT = 232448;   // 227 KB per CTA on sm_100

template <int BN, int EB, int EPI, int CG>
cudaError_t launch_t(const CUtensorMap& ma, const BMaps& mb, const CUtensorMap& me, const CUtensorMap& md,
                     const CUtensorMap& mp, const DMaps& mdx, KParams& kp, cudaStream_t stream) {
  constexpr int STAGE = A_STAGE_BYTES + (BN / CG) * 128;
  constexpr int FIXED = stg_bytes(EPI) + 8 * (2 * MAX_STAGES + 8) + 16 + 1024;
  const int e_bytes = kp.e_tma ? 2 * BM * BN * 2 : 0;
  int stages = (SMEM_LIMIT - FIXED - e_bytes) / STAGE;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) {
    snprintf(g_err, sizeof(g_err), "not enough shared memory for the requested tile configuration");
    return cudaErrorInvalidValue;
  }
  kp.stages = stages;
  const int smem = stages * STAGE + e_bytes + FIXED;
  const int threads = kp.e_tma ? NUM_THREADS + 32 : NUM_THREADS;
  static bool configured = false;
  static int pair_clusters = 0;     // CTA pairs that can be resident at once (CG = 2)
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<BN, EB, EPI, CG>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    if (e != cudaSuccess) return e;
    if (CG == 2) {
      cudaLaunchConfig_t qc;
      memset(&qc, 0, sizeof(qc));
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = 1;
      qc.gridDim = dim3(2 * (sm_count() / 2), 1, 1);
      qc.blockDim = dim3(NUM_THREADS + 32, 1, 1);
      qc.dynamicSmemBytes = SMEM_LIMIT;
      qc.attrs = qa;
      qc.numAttrs = 1;
      int n = 0;
      e = cudaOccupancyMaxActiveClusters(&n, gemm_kernel<BN, EB, EPI, CG>, &qc);
      if (e != cudaSuccess || n < 1) {
        (void)cudaGetLastError();
        n = sm_count() / 2;
      }
      pair_clusters = n;
    }
    configured = true;
  }
  const int num_sms = sm_count();
  // tile order (MAKANI_B200_TILE_ORDER=m|n forces one order for A/B timing)
  static const int forced_order = [] {
    const char* e = getenv("MAKANI_B200_TILE_ORDER");
    return (e && e[0] == 'm') ? 0 : ((e && e[0] == 'n') ? 1 : -1);
  }();
  kp.n_fast = forced_order >= 0 ? forced_order : (kp.m_tiles > kp.n_tiles ? 1 : 0);
  if (CG == 2) {
    long long clusters = kp.total_tiles < pair_clusters ? kp.total_tiles : pair_clusters;
    if (clusters < 1) clusters = 1;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters), 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_kernel<BN, EB, EPI, CG>, ma, mb, me, md, mp, mdx, kp);
  }
  long long grid = kp.total_tiles < num_sms ? kp.total_tiles : num_sms;
  if (grid < 1) grid = 1;
  gemm_kernel<BN, EB, EPI, CG><<<static_cast<unsigned>(grid), threads, smem, stream>>>(ma, mb, me, md, mp, mdx, kp);
  return cudaGetLastError();
}

// tensor map for the epilogue operand: plain [M rows][N contiguous] bf16 with two batch dimensions, no swizzle
bool make_map_e(CUtensorMap* map, const void* ptr, int M, int N, long long row_stride, long long zs_lo, long long zs_hi,
                int zlo_n, int zhi_n, int bn, int box_rows = BM) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(zlo_n),
                        static_cast<cuuint64_t>(zhi_n)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(row_stride) * 2,
                           static_cast<cuuint64_t>(zlo_n > 1 ? zs_lo : row_stride) * 2,
                           static_cast<cuuint64_t>(zhi_n > 1 ? zs_hi : row_stride) * 2};
  (void)bn;
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};   // 64 bf16 = one 128-byte swizzle row
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (strides[0] & 15) || (strides[1] & 15) || (strides[2] & 15)) return false;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

const char* gemm_last_error() { return g_err; }

namespace {
// Copies `rows` rows of `row_bytes` (multiple of 16) from local memory into the same place of up to 8 destination
// buffers (this device's and its peers'), with the producer handshake folded in: every block waits until all
// peers have consumed the previous contents, the last block to finish publishes the new generation.
__global__ void __launch_bounds__(256) peer_publish_kernel(const uint4* __restrict__ src, long long rows, int row_vec,
                                                           long long src_stride_vec, long long dst_stride_vec, int ndst,
                                                           const PeerSync sy, int* err) {
  struct Dst {
    uint4* p[MAX_SEG];
  };
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int w = 0; w < sy.nwait && ok; ++w) {
      const unsigned int need = *sy.wait_exp[w] + static_cast<unsigned int>(sy.wait_off[w]);
      for (int peer = 0; peer < sy.np_wait[w] && ok; ++peer) {
        uint64_t t0 = 0;
        for (uint32_t it = 0;; ++it) {
          if (static_cast<int>(ld_acquire_sys_u32(sy.wait[w] + peer) - need) >= 0) break;
          if ((it & 255u) == 255u) {
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS) {
              atomicExch(err, 40 + w);
              ok = false;
              break;
            }
          }
        }
      }
    }
    ok_s = ok ? 1 : 0;
  }
  __syncthreads();
  if (ok_s) {
    const long long total = rows * row_vec;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long r = i / row_vec;
      const int c = static_cast<int>(i - r * row_vec);
      const uint4 v = src[r * src_stride_vec + c];
      for (int q = 0; q < ndst; ++q) reinterpret_cast<uint4*>(sy.sig[1][q])[r * dst_stride_vec + c] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && sy.done_ctr != nullptr) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(sy.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *sy.done_ctr = 0;
      if (*reinterpret_cast<volatile int*>(err) == 0) {   // nothing is published after an expired wait
        for (int i = 0; i < sy.nwait; ++i)
          if (sy.bump[i]) atomicAdd(sy.bump[i], 1u);
        __threadfence_system();
        for (int peer = 0; peer < sy.np_sig[0]; ++peer)
          if (sy.sig[0][peer]) atomicAdd_system(sy.sig[0][peer], 1u);
      }
    }
  }
}

// out = sum over `nsrc` local segments (+ per-channel bias), 8 bf16 per thread step, with the consumer side of the
// handshake folded in: every block waits until all peers have delivered their segment, the last block to finish tells
// the peers that the buffer may be overwritten.  The second signal list carries the segment base pointers.
__global__ void __launch_bounds__(256) peer_sum_kernel(uint4* __restrict__ out, long long nvec, int nsrc,
                                                       const float* __restrict__ bias, int C, const PeerSync sy, int* err) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int w = 0; w < sy.nwait && ok; ++w) {
      const unsigned int need = *sy.wait_exp[w] + static_cast<unsigned int>(sy.wait_off[w]);
      for (int peer = 0; peer < sy.np_wait[w] && ok; ++peer) {
        uint64_t t0 = 0;
        for (uint32_t it = 0;; ++it) {
          if (static_cast<int>(ld_acquire_sys_u32(sy.wait[w] + peer) - need) >= 0) break;
          if ((it & 255u) == 255u) {
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS) {
              atomicExch(err, 44 + w);
              ok = false;
              break;
            }
          }
        }
      }
    }
    ok_s = ok ? 1 : 0;
  }
  __syncthreads();
  if (ok_s) {
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      if (bias) {
        const int c0 = static_cast<int>((i * 8) % C);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __ldg(bias + c0 + j);
      }
      for (int q = 0; q < nsrc; ++q) {
        // L1 is bypassed: peers rewrite these buffers between launches
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(sy.sig[1][q]) + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      __nv_bfloat162 o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      out[i] = *reinterpret_cast<uint4*>(o);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && sy.done_ctr != nullptr) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(sy.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *sy.done_ctr = 0;
      if (*reinterpret_cast<volatile int*>(err) == 0) {   // nothing is published after an expired wait
        for (int i = 0; i < sy.nwait; ++i)
          if (sy.bump[i]) atomicAdd(sy.bump[i], 1u);
        __threadfence_system();
        for (int peer = 0; peer < sy.np_sig[0]; ++peer)
          if (sy.sig[0][peer]) atomicAdd_system(sy.sig[0][peer], 1u);
      }
    }
  }
}

void fill_sync(PeerSync& sy, const GemmPeer* g) {
  memset(&sy, 0, sizeof(sy));
  if (!g) return;
  for (int i = 0; i < 2; ++i) {
    sy.np_wait[i] = g->np_wait[i];
    sy.np_sig[i] = g->np_sig[i];
  }
  sy.nwait = g->nwait;
  sy.nsig = g->nsig;
  for (int i = 0; i < 2; ++i) {
    sy.wait[i] = g->wait[i];
    sy.wait_exp[i] = g->wait_exp[i];
    sy.wait_off[i] = g->wait_off[i];
    sy.bump[i] = g->bump[i];
    for (int q = 0; q < MAX_SEG; ++q) sy.sig[i][q] = g->sig[i][q];
  }
  sy.done_ctr = g->done_ctr;
}
}  // namespace

cudaError_t peer_publish_launch(const void* src, long long rows, long long row_bytes, long long src_stride_bytes,
                                long long dst_stride_bytes, void* const* dsts, int ndst, const GemmPeer& g, int* err_flag,
                                cudaStream_t stream) {
  if (rows <= 0 || row_bytes <= 0) return cudaSuccess;
  if ((row_bytes & 15) || (src_stride_bytes & 15) || (dst_stride_bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) ||
      ndst < 1 || ndst > MAX_SEG || g.nsig > 1)
    return cudaErrorInvalidValue;
  PeerSync sy;
  fill_sync(sy, &g);
  // the second signal list carries the destination base pointers (the protocol itself needs one list only)
  for (int q = 0; q < MAX_SEG; ++q) sy.sig[1][q] = q < ndst ? static_cast<unsigned int*>(dsts[q]) : nullptr;
  for (int q = 0; q < ndst; ++q)
    if (reinterpret_cast<uintptr_t>(dsts[q]) & 15) return cudaErrorInvalidValue;
  const long long total = rows * (row_bytes / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > sm_count() * 4LL) blocks = sm_count() * 4LL;
  peer_publish_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const uint4*>(src), rows, static_cast<int>(row_bytes / 16), src_stride_bytes / 16, dst_stride_bytes / 16,
      ndst, sy, err_flag);
  return cudaGetLastError();
}

cudaError_t peer_sum_launch(void* out, long long n_elems, const void* const* srcs, int nsrc, const float* bias, int C,
                            const GemmPeer& g, int* err_flag, cudaStream_t stream) {
  if (n_elems <= 0) return cudaSuccess;
  if ((n_elems & 7) || nsrc < 1 || nsrc > MAX_SEG || g.nsig > 1 || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (bias && (C <= 0 || (C & 7))))
    return cudaErrorInvalidValue;
  PeerSync sy;
  fill_sync(sy, &g);
  for (int q = 0; q < MAX_SEG; ++q) {
    if (q < nsrc && (reinterpret_cast<uintptr_t>(srcs[q]) & 15)) return cudaErrorInvalidValue;
    sy.sig[1][q] = q < nsrc ? static_cast<unsigned int*>(const_cast<void*>(srcs[q])) : nullptr;
  }
  const long long nvec = n_elems / 8;
  long long blocks = (nvec + 255) / 256;
  if (blocks > sm_count() * 4LL) blocks = sm_count() * 4LL;
  peer_sum_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<uint4*>(out), nvec, nsrc, bias, C, sy, err_flag);
  return cudaGetLastError();
}

cudaError_t gemm_launch(const GemmProblem& p, const GemmOperand& A, const GemmOperand& B, const GemmEpilogue& e,
                        int* err_flag, cudaStream_t stream, const GemmPeer* peer) {
  g_err[0] = 0;
  if (p.M <= 0 || p.N <= 0 || p.zlo_n <= 0 || p.zhi_n <= 0) return cudaSuccess;
  // cuTensorMapEncodeTiled is a driver call: make sure this host thread has the primary context bound (threads
  // that only inherited the device index, e.g. autograd workers, do not until their first runtime call)
  // (once per host thread: the call is not allowed while a stream is capturing, and threads are reused)
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cs) == cudaSuccess && cs == cudaStreamCaptureStatusNone) {
      cudaFree(nullptr);
      ctx_bound = true;
    }
  }
  const int eb = p.elem_bytes;
  if (eb != 2 && eb != 4) {
    snprintf(g_err, sizeof(g_err), "elem_bytes must be 2 or 4");
    return cudaErrorInvalidValue;
  }
  int bn = p.bn;
  if (bn == 0) bn = (p.N > 128) ? 256 : 128;
  if (bn != 128 && bn != 256) {
    snprintf(g_err, sizeof(g_err), "bn must be 128 or 256");
    return cudaErrorInvalidValue;
  }
  if (eb == 4 && (A.mn_major || B.mn_major)) {
    snprintf(g_err, sizeof(g_err), "tf32 operands must be k-major (row-contiguous tf32 operands are not supported)");
    return cudaErrorInvalidValue;
  }
  if (p.splits > 1 && !e.accumulate) {
    snprintf(g_err, sizeof(g_err), "split-k needs accumulate");
    return cudaErrorInvalidValue;
  }
  if (e.accumulate && (!e.out_f32 || e.resid || e.preact)) {
    snprintf(g_err, sizeof(g_err), "accumulate needs fp32 output without residual/preact");
    return cudaErrorInvalidValue;
  }
  const int bk = 128 / eb;
  KParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.M = p.M; kp.N = p.N; kp.K = p.K;
  kp.zlo_n = p.zlo_n; kp.zhi_n = p.zhi_n;
  kp.splits = p.splits < 1 ? 1 : p.splits;
  const int kblocks = (p.K + bk - 1) / bk;
  kp.k_per_split = ((kblocks + kp.splits - 1) / kp.splits) * bk;
  if (kp.k_per_split < bk) kp.k_per_split = bk;
  kp.a_mn = A.mn_major; kp.b_mn = B.mn_major;
  kp.a_zlo = (A.zs_lo != 0 && p.zlo_n > 1); kp.a_zhi = (A.zs_hi != 0 && p.zhi_n > 1);
  kp.b_zlo = (B.zs_lo != 0 && p.zlo_n > 1); kp.b_zhi = (B.zs_hi != 0 && p.zhi_n > 1);
  kp.rmin_a = p.rmin_a; kp.rmin_b = p.rmin_b; kp.rmax_a = p.rmax_a; kp.rmax_b = p.rmax_b;
  kp.kmin_a = p.kmin_a; kp.kmin_b = p.kmin_b; kp.kmax_a = p.kmax_a; kp.kmax_b = p.kmax_b;
  kp.d_zlo = e.d_zlo; kp.d_zhi = e.d_zhi;
  kp.rdiv = e.rdiv > 0 ? e.rdiv : 1 << 30; kp.rs_hi = e.rs_hi; kp.rs_lo = e.rs_lo;
  kp.ndiv = e.ndiv > 0 ? e.ndiv : 1 << 30; kp.ns_hi = e.ns_hi;
  kp.alpha = e.alpha; kp.bias = e.bias; kp.bias_zs = e.bias ? e.bias_zs : 0; kp.bias_mode = e.bias ? e.bias_mode : 0; kp.act = e.act; kp.save_deriv = (e.save_deriv && e.act == 1 && e.preact) ? 1 : 0; kp.gelu = gelu_coef(gelu_tanh()); kp.act_param = e.act_param;
  kp.resid = e.resid; kp.preact = e.preact; kp.D = e.D;
  kp.out_f32 = e.out_f32; kp.accumulate = e.accumulate;
  // 16-byte vector accesses need every stride (and the bases) aligned
  const int va = e.out_f32 ? 4 : 8;
  auto al = [&](long long s) { return (s % va) == 0; };
  const uintptr_t amask = 15;
  bool vec = al(e.d_zlo) && al(e.d_zhi) && al(e.rs_hi) && al(e.rs_lo) && al(e.ns_hi) && (kp.ndiv % 8 == 0) &&
             ((reinterpret_cast<uintptr_t>(e.D) & amask) == 0);
  if (e.resid) vec = vec && ((reinterpret_cast<uintptr_t>(e.resid) & amask) == 0);
  if (e.preact) vec = vec && ((reinterpret_cast<uintptr_t>(e.preact) & amask) == 0);
  kp.vec_ok = vec ? 1 : 0;
  kp.m_tiles = (p.M + BM - 1) / BM;
  kp.n_tiles = (p.N + bn - 1) / bn;
  kp.total_tiles = static_cast<long long>(kp.m_tiles) * kp.n_tiles * kp.splits * p.zlo_n * p.zhi_n;
  kp.err = err_flag;
  kp.nseg = 1;
  kp.ndx = 0;
  fill_sync(kp.sync, peer);
  if (peer && peer->ndx > 0) {
    if (peer->ndx > MAX_SEG - 1 || e.out_f32 || e.accumulate || kp.splits != 1 || e.preact) {
      snprintf(g_err, sizeof(g_err), "replicated output: bf16 plain stores only, at most %d extra destinations", MAX_SEG - 1);
      return cudaErrorInvalidValue;
    }
    kp.ndx = peer->ndx;
    for (int q = 0; q < peer->ndx; ++q) kp.Dx[q] = peer->Dx[q];
  }
  if (peer && peer->nseg > 1) {
    if (kp.splits != 1 || peer->nseg > MAX_SEG) {
      snprintf(g_err, sizeof(g_err), "multi-device operand: split-k not supported, at most %d segments", MAX_SEG);
      return cudaErrorInvalidValue;
    }
    kp.nseg = peer->nseg;
    for (int q = 0; q < peer->nseg; ++q) {
      kp.seg_len[q] = peer->seg_len[q];
      kp.seg_apos[q] = peer->seg_apos[q];
      kp.seg_gstart[q] = peer->seg_gstart[q];
    }
  }

  CUtensorMap ma, mb, me;
  memset(&me, 0, sizeof(me));
  // Epilogue operand through TMA when it is bf16 and the destination layout is a plain row-major matrix batch.
  kp.e_tma = 0;
  const bool plain = (e.rdiv <= 0 || e.rdiv >= (1 << 30)) && (e.ndiv <= 0 || e.ndiv >= (1 << 30));
  if (e.resid && !e.out_f32 && plain && kp.vec_ok && e.d_zlo >= 0 && e.d_zhi >= 0) {
    if (make_map_e(&me, e.resid, p.M, p.N, e.rs_lo, e.d_zlo, e.d_zhi, p.zlo_n, p.zhi_n, 128)) {
      kp.e_tma = 1;
      bn = 128;
    }
  }
  // CTA pairs (256-row tiles, each CTA loads half of the B tile): single-device bf16 launches without row-triangular
  // structure and with at least two row blocks.  MAKANI_B200_CTA_PAIRS=0 keeps every launch on single CTAs.
  // Measured at 721x1440 (1 GPU, CUDA events): pairs win where the k loop is long (K = 768 convolutions, weight
  // gradients, the longitude DFT: 3-11 %) and lose where it is short (K = 384: the epilogue, not the operand fill, is
  // the bound there, and a pair has half as many independent tiles in flight), so the default is K >= 512.
  // MAKANI_B200_CTA_PAIRS=0 / 1 forces none / all eligible launches.
  static const int pairs_mode = [] {
    const char* e = getenv("MAKANI_B200_CTA_PAIRS");
    return (e && e[0] == '0') ? 0 : ((e && e[0] == '1') ? 1 : 2);
  }();
  const bool no_peer = (peer == nullptr) || (peer->nseg <= 1 && peer->ndx == 0 && peer->nwait == 0 && peer->nsig == 0 &&
                                              peer->done_ctr == nullptr);
  const bool eligible = eb == 2 && no_peer && p.M > BM && p.rmin_a == 0 && p.rmax_a == 0;
  const int cg = (eligible && (pairs_mode == 1 || (pairs_mode == 2 && p.K >= 512))) ? 2 : 1;
  kp.m_tiles = (p.M + BM * cg - 1) / (BM * cg);
  kp.n_tiles = (p.N + bn - 1) / bn;
  kp.total_tiles = static_cast<long long>(kp.m_tiles) * kp.n_tiles * kp.splits * p.zlo_n * p.zhi_n;
  if (!make_map(&ma, A, p.K, eb, p.zlo_n, p.zhi_n, BM)) return cudaErrorInvalidValue;
  const int bn_box = bn / cg;     // rows of B one CTA loads per stage
  BMaps mbs;
  if (kp.nseg > 1) {
    for (int q = 0; q < kp.nseg; ++q) {
      GemmOperand Bq = B;
      Bq.ptr = peer->seg_ptr[q];
      if (!make_map(&mbs.m[q], Bq, peer->seg_len[q], eb, p.zlo_n, p.zhi_n, bn_box)) return cudaErrorInvalidValue;
    }
    for (int q = kp.nseg; q < MAX_SEG; ++q) mbs.m[q] = mbs.m[0];
  } else {
    if (!make_map(&mb, B, p.K, eb, p.zlo_n, p.zhi_n, bn_box)) return cudaErrorInvalidValue;
    for (int q = 0; q < MAX_SEG; ++q) mbs.m[q] = mb;
  }
  if (!kp.e_tma) me = ma;   // unused, but must be a valid descriptor

  kp.plain_cols = (e.ndiv <= 0 || e.ndiv >= (1 << 30)) ? 1 : 0;
  // pick a specialised epilogue (TMA stores of bf16 tiles) when the launch fits one
  int epi = 0;
  CUtensorMap md, mp;
  memset(&md, 0, sizeof(md));
  md = ma;
  mp = ma;
  DMaps mdx;
  for (int q = 0; q < MAX_SEG - 1; ++q) mdx.m[q] = ma;   // placeholders: always valid descriptors
  if (eb == 2 && !e.out_f32 && kp.vec_ok && !e.accumulate && plain && e.d_zlo >= 0 && e.d_zhi >= 0 &&
      (kp.bias_mode != 2 || ((reinterpret_cast<uintptr_t>(e.bias) & 15) == 0 && (kp.bias_zs % 4) == 0))) {
    if (!e.resid && !e.preact && (e.act == 0 || e.act == 3 || e.act == 5)) epi = 1;
    else if (!e.resid && e.preact && e.act == 1) epi = 2;
    else if (e.resid && kp.e_tma && !e.preact && e.act == 0) epi = 3;
    else if (e.resid && kp.e_tma && !e.preact && (e.act == 2 || e.act == 4 || e.act == 6 || e.act == 8)) epi = 4;
    if (epi != 0) {
      bool ok = make_map_e(&md, e.D, p.M, p.N, e.rs_lo, e.d_zlo, e.d_zhi, p.zlo_n, p.zhi_n, bn, 32);
      if (ok && epi == 2) ok = make_map_e(&mp, e.preact, p.M, p.N, e.rs_lo, e.d_zlo, e.d_zhi, p.zlo_n, p.zhi_n, bn, 32);
      if (ok && kp.ndx > 0) {
        if (epi != 1) ok = false;   // replicated output goes through the plain-store epilogue or the generic one
        for (int q = 0; ok && q < kp.ndx; ++q)
          ok = make_map_e(&mdx.m[q], kp.Dx[q], p.M, p.N, e.rs_lo, e.d_zlo, e.d_zhi, p.zlo_n, p.zhi_n, bn, 32);
      }
      if (!ok) epi = 0;
    }
  }
  if (eb == 4) {
    if (bn == 256) return launch_t<256, 4, 0, 1>(ma, mbs, me, md, mp, mdx, kp, stream);
    return launch_t<128, 4, 0, 1>(ma, mbs, me, md, mp, mdx, kp, stream);
  }
#define MK_DISPATCH(EPI_)                                                                              \
  if (cg == 2) {                                                                                       \
    if (bn == 256) return launch_t<256, 2, EPI_, 2>(ma, mbs, me, md, mp, mdx, kp, stream);             \
    return launch_t<128, 2, EPI_, 2>(ma, mbs, me, md, mp, mdx, kp, stream);                            \
  }                                                                                                    \
  if (bn == 256) return launch_t<256, 2, EPI_, 1>(ma, mbs, me, md, mp, mdx, kp, stream);               \
  return launch_t<128, 2, EPI_, 1>(ma, mbs, me, md, mp, mdx, kp, stream);
  switch (epi) {
    case 1: { MK_DISPATCH(1) }
    case 2: { MK_DISPATCH(2) }
    case 3: { MK_DISPATCH(3) }
    case 4: { MK_DISPATCH(4) }
    default: { MK_DISPATCH(0) }
  }
#undef MK_DISPATCH
}

}  // namespace mk
