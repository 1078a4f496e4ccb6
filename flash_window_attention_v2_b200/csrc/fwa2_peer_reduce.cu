// Cross-GPU sum of the window-summed dBias / dLogitScale, fused with the final cast: the exchange
// step of the window-sharded backward in ONE kernel per GPU, over peer memory (NVLink).
//
// Every rank has left its local fp32 sums [H*N*N dBias | H dLogitScale] in a buffer that all ranks
// have mapped (symmetric memory).  Each rank's kernel tells every peer "my sums of step `epoch`
// are complete" with one release store into the peer's flag array, waits (bounded) until every
// peer has said the same, then reads all ranks' buffers with plain loads, adds them in ascending
// rank order -- the same order on every GPU, so all ranks get bit-identical results and the sum is
// reproducible -- applies the clamp gate 1[g <= ln 100] to dLogitScale and casts
// (flash_win_attn_v2/kernels/attn_kernel_backward.py:703-711).  No collective library call, no
// multicast loads; replaces NCCL all-reduce + cast (two launches and a ring latency) by one launch.
//
// The caller alternates between two sets of buffers from step to step: a rank that has finished
// step e may already be writing step e + 1 while a slower peer still reads step e.  A peer cannot
// fall two steps behind, because nobody gets past step e + 1 without that peer's flag for e + 1.
#include "../../include/fwa2.h"
#include "fwa2_common.cuh"

#include <cuda_runtime.h>

namespace fwa2 {

constexpr int kMaxPeers = 8;

struct PeerReduceParams {
  const float* partial[kMaxPeers];   // rank r's sums, as mapped on this GPU
  uint32_t* flags[kMaxPeers];        // rank r's flag array (kMaxPeers words), as mapped on this GPU
  int rank, world;
  uint32_t epoch;
  long long total;                   // H * N * N
  int H;
  const void* logit_scale;
  void* dbias;
  void* dscale;
  DeviceStatus* status;
};

template <typename T>
__device__ __forceinline__ uint16_t peer_raw16(float x);
template <>
__device__ __forceinline__ uint16_t peer_raw16<__nv_bfloat16>(float x) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}
template <>
__device__ __forceinline__ uint16_t peer_raw16<__half>(float x) {
  return __half_as_ushort(__float2half_rn(x));
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// (plain, not read-only-path loads: the buffers are rewritten by their owners from step to step)
__device__ __forceinline__ float4 ld_peer_v4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ float ld_peer(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(256) peer_reduce_finalize_kernel(const PeerReduceParams p) {
  __shared__ uint32_t gave_up;
  const int tid = threadIdx.x;
  if (tid == 0) gave_up = 0u;
  // my sums were written by earlier kernels on this stream; announce them to every peer
  if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
    __threadfence_system();
    st_release_sys(p.flags[tid] + p.rank, p.epoch);
  }
  __syncthreads();
  // every block waits for every peer itself (bounded: about a second, then an error status)
  if (tid < p.world && tid != p.rank) {
    const uint32_t* f = p.flags[p.rank] + tid;
    const long long t0 = clock64();
    uint32_t spins = 0;
    // (flags only grow; the subtraction is the wrap-safe form of "flag >= epoch")
    while (static_cast<int32_t>(ld_acquire_sys(f) - p.epoch) < 0) {
      if ((++spins & 0x3FFu) == 0u && clock64() - t0 > kWaitLimitCycles) {
        gave_up = 1u;
        if (p.status != nullptr && atomicCAS(&p.status->code, 0u, (90u << 8) | kStatusTimeout) == 0u) {
          p.status->block = blockIdx.x;
          p.status->detail = static_cast<unsigned int>(tid);
        }
        break;
      }
    }
  }
  __syncthreads();
  if (gave_up) return;      // the outputs stay unwritten; the status word says why

  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + tid) * 4; i < p.total; i += stride) {
    if (i + 3 < p.total) {
      float4 s = ld_peer_v4(p.partial[0] + i);
      for (int r = 1; r < p.world; ++r) {
        const float4 v = ld_peer_v4(p.partial[r] + i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      if (p.dbias != nullptr) {
        uint2 o;
        o.x = static_cast<uint32_t>(peer_raw16<T>(s.x)) | (static_cast<uint32_t>(peer_raw16<T>(s.y)) << 16);
        o.y = static_cast<uint32_t>(peer_raw16<T>(s.z)) | (static_cast<uint32_t>(peer_raw16<T>(s.w)) << 16);
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.dbias) + i) = o;
      }
    } else {
      for (long long j = i; j < p.total; ++j) {
        float s = ld_peer(p.partial[0] + j);
        for (int r = 1; r < p.world; ++r) s += ld_peer(p.partial[r] + j);
        if (p.dbias != nullptr) static_cast<uint16_t*>(p.dbias)[j] = peer_raw16<T>(s);
      }
    }
  }
  if (blockIdx.x == 0 && tid < p.H && p.dscale != nullptr) {
    float s = ld_peer(p.partial[0] + p.total + tid);
    for (int r = 1; r < p.world; ++r) s += ld_peer(p.partial[r] + p.total + tid);
    const uint16_t raw = static_cast<const uint16_t*>(p.logit_scale)[tid];
    const float g = Elem<T>::from_raw(raw);
    const float lim = Elem<T>::from_raw(peer_raw16<T>(kLn100));
    static_cast<uint16_t*>(p.dscale)[tid] = peer_raw16<T>(g <= lim ? s : 0.f);
  }
}

}  // namespace fwa2

using namespace fwa2;

extern "C" int fwa2_peer_reduce_finalize(const float* const* partials, uint32_t* const* flags, int32_t rank,
                                         int32_t world, uint32_t epoch, int32_t dtype, int32_t heads, int32_t n,
                                         const void* logit_scale, void* dbias, void* dscale, void* status,
                                         void* stream) {
  if (partials == nullptr || flags == nullptr) return FWA2_ERR_NULL;
  if (dtype != FWA2_F16 && dtype != FWA2_BF16) return FWA2_ERR_DTYPE;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || heads <= 0 || heads > 256 || n <= 0)
    return FWA2_ERR_SHAPE;
  if (dscale != nullptr && logit_scale == nullptr) return FWA2_ERR_NULL;
  PeerReduceParams p{};
  for (int r = 0; r < world; ++r) {
    if (partials[r] == nullptr || flags[r] == nullptr) return FWA2_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(partials[r]) & 15u) != 0) return FWA2_ERR_ALIGN;
    p.partial[r] = partials[r];
    p.flags[r] = flags[r];
  }
  p.rank = rank;
  p.world = world;
  p.epoch = epoch;
  p.total = static_cast<long long>(heads) * n * n;
  p.H = heads;
  p.logit_scale = logit_scale;
  p.dbias = dbias;
  p.dscale = dscale;
  p.status = static_cast<DeviceStatus*>(status);
  long long blocks = (p.total / 4 + 255) / 256;
  if (blocks > 592) blocks = 592;
  if (blocks < 1) blocks = 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == FWA2_BF16) peer_reduce_finalize_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, s>>>(p);
  else peer_reduce_finalize_kernel<__half><<<static_cast<int>(blocks), 256, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? FWA2_OK : FWA2_ERR_LAUNCH;
}
