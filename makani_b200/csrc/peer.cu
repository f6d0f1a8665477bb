// Peer-memory allocation (CUDA IPC) and an NVLink all-reduce written as one kernel: barrier -> each rank
// pulls and reduces its slice from all peers -> pushes the reduced slice to all peers -> barrier.
#include "peer.cuh"

#include <cuda_bf16.h>
#include <stdint.h>

namespace mk {

namespace {

constexpr uint64_t PEER_WAIT_NS = 2000000000ull;

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
__device__ __forceinline__ bool cta_barrier(const PeerPtrs& p, int world, int rank, unsigned int value) {
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
        else if (now - t0 > PEER_WAIT_NS) {
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
  static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
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
};

template <typename T>
__global__ void __launch_bounds__(512) allreduce_kernel(const PeerPtrs p, int world, int rank, long long n, float scale,
                                                        int* err) {
  constexpr int V = Vec16<T>::N;
  unsigned int* my_epoch = p.flags[rank] + blockIdx.x * (PEER_MAX + 1) + PEER_MAX;
  const unsigned int epoch = *my_epoch;
  const unsigned int v0 = 2 * epoch + 1, v1 = 2 * epoch + 2;
  bool ok = cta_barrier(p, world, rank, v0);
  if (ok) {
    // slice of this rank, in 16-byte vectors
    const long long nvec = n / V;
    const long long per = (nvec + world - 1) / world;
    const long long beg = per * rank;
    long long end = beg + per;
    if (end > nvec) end = nvec;
    for (long long i = beg + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < end;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
      for (int r = 0; r < world; ++r) {
        const int src = (rank + r) % world;   // stagger the peers
        float f[V];
        Vec16<T>::load(static_cast<const T*>(p.data[src]) + i * V, f);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += f[j];
      }
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] *= scale;
      for (int r = 0; r < world; ++r) {
        const int dst = (rank + r) % world;
        Vec16<T>::store(static_cast<T*>(p.data[dst]) + i * V, acc);
      }
    }
    // ragged tail (n not a multiple of the vector width): the last rank handles it elementwise
    if (rank == world - 1 && blockIdx.x == 0) {
      for (long long i = nvec * V + threadIdx.x; i < n; i += blockDim.x) {
        float a = 0.f;
        for (int r = 0; r < world; ++r) a += static_cast<float>(static_cast<const T*>(p.data[r])[i]);
        a *= scale;
        for (int r = 0; r < world; ++r) static_cast<T*>(p.data[r])[i] = static_cast<T>(a);
      }
    }
    ok = cta_barrier(p, world, rank, v1);
  }
  if (!ok && threadIdx.x == 0) atomicExch(err, 16);
  if (threadIdx.x == 0) *my_epoch = epoch + 1;
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

cudaError_t peer_allreduce(const PeerPtrs& p, int world, int rank, long long n, int is_bf16, float scale, unsigned int,
                           int* err, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const int V = is_bf16 ? 8 : 4;
  long long per = (n / V + world - 1) / world;
  long long blocks = (per + 511) / 512;
  if (blocks < 1) blocks = 1;
  if (blocks > 64) blocks = 64;   // 64 CTAs x 512 threads x 16 B in flight saturate NVLink without starving compute
  if (is_bf16) allreduce_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 512, 0, s>>>(p, world, rank, n, scale, err);
  else allreduce_kernel<float><<<static_cast<unsigned>(blocks), 512, 0, s>>>(p, world, rank, n, scale, err);
  return cudaGetLastError();
}

}  // namespace mk
