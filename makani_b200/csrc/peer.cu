// Peer-memory allocation (CUDA IPC) and an NVLink all-reduce written as one kernel: barrier -> each rank
// pulls and reduces its slice from all peers -> pushes the reduced slice to all peers -> barrier.
#include "peer.cuh"

#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

namespace mk {

namespace {


__device__ __forceinline__ uint64_t gtime() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All `world` ranks' CTA `blockIdx.x` meet here. Slot layout per rank: [block][PEER_MAX + 1].
// Thread i < world signals peer i and waits for peer i's signal. Returns false if a wait ran out.
__device__ __forceinline__ bool cta_barrier(const PeerPtrs& p, int world, int rank, unsigned int value, uint64_t wait_ns) {
  bool ok = true;
  __syncthreads();
  if (threadIdx.x < world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    st_release_sys(p.flags[peer] + blockIdx.x * (PEER_MAX + 1) + rank, value);
    const unsigned int* mine = p.flags[rank] + blockIdx.x * (PEER_MAX + 1) + peer;
    uint64_t t0 = 0;
    for (unsigned int it = 0;; ++it) {
      // signed distance handles wrap-around of the epoch counter
      if (static_cast<int>(ld_acquire_sys(mine) - value) >= 0) break;
      if ((it & 255u) == 255u) {
        const uint64_t now = gtime();
        if (t0 == 0) t0 = now;
        else if (now - t0 > wait_ns) {
          ok = false;
          break;
        }
      }
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void add(const uint4& v, float (&a)[4]) {
    a[0] += __uint_as_float(v.x); a[1] += __uint_as_float(v.y); a[2] += __uint_as_float(v.z); a[3] += __uint_as_float(v.w);
  }
  static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
  static __device__ __forceinline__ void store_cs(float* p, const float (&f)[4]) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(f[0], f[1], f[2], f[3]));
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void add(const uint4& v, float (&a)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = __bfloat1622float2(h[j]);
      a[2 * j] += x.x;
      a[2 * j + 1] += x.y;
    }
  }
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = __bfloat1622float2(h[j]);
      f[2 * j] = x.x;
      f[2 * j + 1] = x.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    *reinterpret_cast<uint4*>(p) = v;
  }
  static __device__ __forceinline__ void store_cs(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    __stcs(reinterpret_cast<uint4*>(p), v);
  }
};

// 128 threads (one warp per SM sub-partition) x at most 64 registers: the register file is four banks of 16384
// registers, one per sub-partition, and a persistent GEMM CTA (10 warps x up to 144 registers) leaves only 2560 of them
// in the two sub-partitions that hold three of its warps.  A CTA of this kernel must fit into that remainder, or it
// cannot share an SM with a GEMM CTA: it then takes the SM from the next GEMM launch, whose displaced CTA runs as a
// straggler, and the reduction serialises with backward instead of overlapping it (measured: step time = compute +
// reduction time for every grid size, with 256- and 512-thread versions of this kernel).
constexpr int AR_THREADS = 128;

// WORLD is a template parameter so that the loops over the peers unroll completely: all WORLD loads of a vector (and U
// vectors per thread) are in flight together, which is what it takes to fill an NVLink round trip (about 2 us) with
// about a hundred CTAs; with a run-time peer loop each thread had a single 16-byte load outstanding and the pull ran at a third
// of the link rate.
template <typename T, int WORLD>
__global__ void __maxnreg__(64) allreduce_kernel(const PeerPtrs p, int rank, long long n, float scale,
                                                        uint64_t wait_ns, int* err) {
  constexpr int V = Vec16<T>::N;
  constexpr int U = (WORLD <= 2) ? 4 : ((WORLD <= 4) ? 2 : 1);   // vectors per thread and trip: U * WORLD (about 8) loads in flight
  unsigned int* my_epoch = p.flags[rank] + blockIdx.x * (PEER_MAX + 1) + PEER_MAX;
  const unsigned int epoch = *my_epoch;
  const unsigned int v0 = 2 * epoch + 1, v1 = 2 * epoch + 2;
  bool ok = cta_barrier(p, WORLD, rank, v0, wait_ns);
  if (ok) {
    // peers in staggered order (rank, rank + 1, ...), so that the ranks do not all hit the same peer at once
    T* peer[WORLD];
#pragma unroll
    for (int r = 0; r < WORLD; ++r) peer[r] = static_cast<T*>(p.data[(rank + r) % WORLD]);
    // slice of this rank, in 16-byte vectors
    const long long nvec = n / V;
    const long long per = (nvec + WORLD - 1) / WORLD;
    const long long beg = per * rank;
    long long end = beg + per;
    if (end > nvec) end = nvec;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = beg + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < end; i0 += stride * U) {
      uint4 raw[U][WORLD];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < end) {
#pragma unroll
          for (int r = 0; r < WORLD; ++r) raw[u][r] = __ldcs(reinterpret_cast<const uint4*>(peer[r] + i * V));   // streaming: keep L2 for the GEMMs
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < end) {
          float acc[V];
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] = 0.f;
#pragma unroll
          for (int r = 0; r < WORLD; ++r) Vec16<T>::add(raw[u][r], acc);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] *= scale;
#pragma unroll
          for (int r = 0; r < WORLD; ++r) Vec16<T>::store_cs(peer[r] + i * V, acc);
        }
      }
    }
    // ragged tail (n not a multiple of the vector width): the last rank handles it elementwise
    if (rank == WORLD - 1 && blockIdx.x == 0) {
      for (long long i = nvec * V + threadIdx.x; i < n; i += blockDim.x) {
        float a = 0.f;
        for (int r = 0; r < WORLD; ++r) a += static_cast<float>(static_cast<const T*>(p.data[r])[i]);
        a *= scale;
        for (int r = 0; r < WORLD; ++r) static_cast<T*>(p.data[r])[i] = static_cast<T>(a);
      }
    }
    ok = cta_barrier(p, WORLD, rank, v1, wait_ns);
  }
  if (!ok && threadIdx.x == 0) atomicExch(err, 16);
  if (threadIdx.x == 0) *my_epoch = epoch + 1;
}

template <typename T>
cudaError_t launch_allreduce(int world, unsigned blocks, cudaStream_t s, const PeerPtrs& p, int rank, long long n, float scale,
                             uint64_t wait_ns, int* err) {
  switch (world) {
  // The reduction has to run on SMs that a persistent GEMM CTA already occupies.  Kernels share an SM only under one
  // shared-memory / L1 split, and the GEMMs run with the largest shared-memory carve-out, so this kernel asks for the
  // same split although it uses no shared memory itself; otherwise it waits for SMs to drain and the GEMM CTA that
  // lost its SM to this kernel runs as a straggler after the others.
#define MK_AR(W)                                                                                                      \
  case W: {                                                                                                           \
    static bool carve = false;                                                                                        \
    if (!carve) {                                                                                                     \
      cudaFuncSetAttribute(allreduce_kernel<T, W>, cudaFuncAttributePreferredSharedMemoryCarveout,                    \
                           cudaSharedmemCarveoutMaxShared);                                                           \
      carve = true;                                                                                                   \
    }                                                                                                                 \
    allreduce_kernel<T, W><<<blocks, AR_THREADS, 0, s>>>(p, rank, n, scale, wait_ns, err);                            \
    break;                                                                                                            \
  }
    MK_AR(1) MK_AR(2) MK_AR(3) MK_AR(4) MK_AR(5) MK_AR(6) MK_AR(7) MK_AR(8)
#undef MK_AR
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t peer_alloc(size_t bytes, void** ptr, char* handle64) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return e;
  e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) return e;
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) return e;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  for (int i = 0; i < 64; ++i) handle64[i] = reinterpret_cast<const char*>(&h)[i];
  return cudaDeviceSynchronize();
}

cudaError_t peer_open(const char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  for (int i = 0; i < 64; ++i) reinterpret_cast<char*>(&h)[i] = handle64[i];
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

cudaError_t peer_close(void* ptr) { return cudaIpcCloseMemHandle(ptr); }
cudaError_t peer_free(void* ptr) { return cudaFree(ptr); }

cudaError_t peer_allreduce(const PeerPtrs& p, int world, int rank, long long n, int is_bf16, float scale, double wait_seconds,
                           int* err, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  if (!(wait_seconds > 0.0)) wait_seconds = 2.0;
  const uint64_t wait_ns = static_cast<uint64_t>(wait_seconds * 1e9);
  const int V = is_bf16 ? 8 : 4;
  long long per = (n / V + world - 1) / world;
  long long blocks = (per + AR_THREADS - 1) / AR_THREADS;
  if (blocks < 1) blocks = 1;
  // 128 CTAs x 128 threads x 8 vectors of 16 B in flight keep NVLink busy without starving compute (MAKANI_B200_AR_BLOCKS overrides,
  // read once; every rank of a group must use the same value because CTA i pairs with CTA i of its peers)
  static const int max_blocks = [] {
    const char* e = getenv("MAKANI_B200_AR_BLOCKS");
    int v = e ? atoi(e) : PEER_MAX_BLOCKS;
    return (v >= 1 && v <= PEER_MAX_BLOCKS) ? v : PEER_MAX_BLOCKS;
  }();
  if (blocks > max_blocks) blocks = max_blocks;
  if (is_bf16) return launch_allreduce<__nv_bfloat16>(world, static_cast<unsigned>(blocks), s, p, rank, n, scale, wait_ns, err);
  return launch_allreduce<float>(world, static_cast<unsigned>(blocks), s, p, rank, n, scale, wait_ns, err);
}

}  // namespace mk
