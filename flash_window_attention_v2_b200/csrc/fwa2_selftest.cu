// Single-CTA checks of the tcgen05 building blocks the attention kernels rely on: the shared
// memory descriptor conventions (K-major and MN-major operands, 64- and 128-byte swizzles), the
// packed 16-bit A operand in tensor memory, and the accumulator layout read back with
// tcgen05.ld.  Each mode multiplies two small matrices given in plain row-major global memory
// and writes the fp32 product; the host test compares with a matmul.
#include "fwa2_ptx.cuh"

namespace fwa2 {

// mode 0: D[128][64] = A[128][32] * B[64][32]^T      A,B K-major rows of 64 B (SW64)
// mode 1: D[128][32] = A[128][64] * B[64][32]        A K-major rows of 128 B (SW128), B MN-major SW64
// mode 2: same product as mode 1 with A taken from tensor memory (packed pairs)
// mode 3: D[128][32] = A^T * B, A given as [128 k][128 m] (MN-major SW128, two 64-column slabs),
//         B[128 k][32] MN-major SW64
template <typename T>
__global__ void __launch_bounds__(128, 1)
selftest_kernel(int mode, const uint16_t* __restrict__ a, const uint16_t* __restrict__ b,
                float* __restrict__ d, DeviceStatus* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t abort_flag;

  const uint32_t tid = threadIdx.x;
  const uint32_t warp = tid >> 5;
  uint32_t base = smem_u32(smem_raw);
  base = (base + 1023u) & ~1023u;
  const uint32_t a_smem = base;              // up to 32 KiB
  const uint32_t b_smem = base + 32768u;     // up to 8 KiB

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_slot), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;
  const uint32_t lane_base = (warp * 32u) << 16;
  const uint32_t d_cols = 0;     // accumulator columns [0, 64)
  const uint32_t a_cols = 64;    // packed A operand columns [64, 96)

  // ---- stage operands ----
  auto copy16 = [&](uint32_t dst, const uint16_t* src) {
    const uint4 v = *reinterpret_cast<const uint4*>(src);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    sts128(dst, w);
  };
  if (mode == 0) {
    for (uint32_t i = tid; i < 128 * 4; i += 128) {
      const uint32_t r = i >> 2, c = i & 3;
      copy16(a_smem + sw64_offset(r, c), a + r * 32 + c * 8);
    }
    for (uint32_t i = tid; i < 64 * 4; i += 128) {
      const uint32_t r = i >> 2, c = i & 3;
      copy16(b_smem + sw64_offset(r, c), b + r * 32 + c * 8);
    }
  } else if (mode == 1 || mode == 2) {
    if (mode == 1) {
      for (uint32_t i = tid; i < 128 * 8; i += 128) {
        const uint32_t r = i >> 3, c = i & 7;
        copy16(a_smem + sw128_offset(r, c), a + r * 64 + c * 8);
      }
    } else {
      // thread = row: 64 elements -> 32 packed columns of tensor memory
      uint32_t w[16];
      const uint32_t* src = reinterpret_cast<const uint32_t*>(a + tid * 64);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = src[half * 16 + i];
        tmem_st16(tmem + lane_base + a_cols + half * 16, w);
      }
      tmem_wait_st();
    }
    for (uint32_t i = tid; i < 64 * 4; i += 128) {
      const uint32_t r = i >> 2, c = i & 3;
      copy16(b_smem + sw64_offset(r, c), b + r * 32 + c * 8);
    }
  } else {
    // a is [k = 128][m = 128]; slab s holds columns m in [64 s, 64 s + 64)
    for (uint32_t i = tid; i < 128 * 16; i += 128) {
      const uint32_t k = i >> 4, c = i & 15;
      const uint32_t slab = c >> 3, cc = c & 7;
      copy16(a_smem + slab * 16384u + sw128_offset(k, cc), a + k * 128 + c * 8);
    }
    for (uint32_t i = tid; i < 128 * 4; i += 128) {
      const uint32_t r = i >> 2, c = i & 3;
      copy16(b_smem + sw64_offset(r, c), b + r * 32 + c * 8);
    }
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();

  // ---- one thread issues the MMAs ----
  if (tid == 0) {
    tc_fence_after();
    constexpr uint32_t fmt = Elem<T>::kFmt;
    if (mode == 0) {
      const uint32_t idesc = make_idesc(fmt, 128, 64, 0, 0);
      for (uint32_t k = 0; k < 2; ++k) {
        const uint64_t ad = make_smem_desc(a_smem + k * 32u, 16, 512, kSw64);
        const uint64_t bd = make_smem_desc(b_smem + k * 32u, 16, 512, kSw64);
        mma_ss(tmem + d_cols, ad, bd, idesc, k > 0);
      }
    } else if (mode == 1) {
      const uint32_t idesc = make_idesc(fmt, 128, 32, 0, 1);
      for (uint32_t k = 0; k < 4; ++k) {
        const uint64_t ad = make_smem_desc(a_smem + k * 32u, 16, 1024, kSw128);
        const uint64_t bd = make_smem_desc(b_smem + k * 1024u, 512, 512, kSw64);
        mma_ss(tmem + d_cols, ad, bd, idesc, k > 0);
      }
    } else if (mode == 2) {
      const uint32_t idesc = make_idesc(fmt, 128, 32, 0, 1);
      for (uint32_t k = 0; k < 4; ++k) {
        const uint64_t bd = make_smem_desc(b_smem + k * 1024u, 512, 512, kSw64);
        mma_ts(tmem + d_cols, tmem + a_cols + k * 8u, bd, idesc, k > 0);
      }
    } else {
      const uint32_t idesc = make_idesc(fmt, 128, 32, 1, 1);
      for (uint32_t k = 0; k < 8; ++k) {
        const uint64_t ad = make_smem_desc(a_smem + k * 2048u, 16384, 1024, kSw128);
        const uint64_t bd = make_smem_desc(b_smem + k * 1024u, 512, 512, kSw64);
        mma_ss(tmem + d_cols, ad, bd, idesc, k > 0);
      }
    }
    mma_commit(smem_u32(&bar));
  }
  WaitCtx ctx{&abort_flag, status};
  const bool ok = mbar_wait(smem_u32(&bar), 0, ctx, 1);
  tc_fence_after();
  __syncwarp();
  if (ok) {
    const uint32_t ncols = (mode == 0) ? 64u : 32u;
    uint32_t r[32];
    for (uint32_t c0 = 0; c0 < ncols; c0 += 32) {
      tmem_ld32(tmem + lane_base + d_cols + c0, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) d[tid * ncols + c0 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

// Issue / completion cost of short tcgen05.mma sequences (kind::f16, M = 128, K = 16 each).
//   n:        N of every MMA
//   a_tmem:   1 = A operand from tensor memory, 0 = from shared memory
//   chains:   1, 2 or 4 independent accumulators the sequence alternates between (one thread
//             issues); 8 = the whole warp runs the loop and an elected lane issues
//   count:    MMAs in the sequence
// out[0] = cycles to issue the sequence, out[1] = cycles until the commit barrier fires.
__global__ void __launch_bounds__(128, 1)
mma_timing_kernel(int n, int a_tmem, int chains, int count, float* __restrict__ out,
                  DeviceStatus* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint32_t tmem_base_slot;
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t abort_flag;
  const uint32_t tid = threadIdx.x, warp = tid >> 5;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // zero the operand area so that the arithmetic is well defined
  for (uint32_t i = tid; i < (65536u + 1024u) / 16u; i += 128) {
    const uint32_t z[4] = {0u, 0u, 0u, 0u};
    if (smem_u32(smem_raw) + i * 16u + 16u <= base + 65536u) sts128(smem_u32(smem_raw) + i * 16u, z);
  }
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_slot), 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;
  long long t0 = 0, t1 = 0;
  const bool uniform_style = chains >= 8;   // chains = 8: whole warp runs the loop, one elected lane issues
  if (uniform_style) {
    if (warp == 0) {
      const uint32_t idesc = make_idesc(1, 128, static_cast<uint32_t>(n), 0, 0);
      const DescBase db = make_desc_base(base + 32768u, 16, 512, kSw64);
      const DescBase da = make_desc_base(base, 16, 512, kSw64);
      t0 = clock64();
#pragma unroll 8
      for (int i = 0; i < count; ++i) {
        const uint64_t bd = desc_at(db, (i & 1) * 32u);
        const uint64_t ad = desc_at(da, (i & 1) * 32u);
        const uint32_t d = tmem + (static_cast<uint32_t>(i) & 1u) * 64u;
        if (elect_one()) {
          if (a_tmem) mma_ts(d, tmem + 256u + (i & 3) * 8u, bd, idesc, i > 1);
          else mma_ss(d, ad, bd, idesc, i > 1);
        }
        __syncwarp();
      }
      t1 = clock64();
      if (elect_one()) mma_commit(smem_u32(&bar));
      __syncwarp();
    }
  } else if (tid == 0) {
    const uint32_t idesc = make_idesc(1, 128, static_cast<uint32_t>(n), 0, 0);
    const DescBase da = make_desc_base(base, 16, 512, kSw64);
    const DescBase db = make_desc_base(base + 32768u, 16, 512, kSw64);
    const uint32_t cmask = static_cast<uint32_t>(chains) - 1u;   // chains is 1, 2 or 4
    t0 = clock64();
    if (a_tmem) {
#pragma unroll 8
      for (int i = 0; i < count; ++i)
        mma_ts(tmem + (static_cast<uint32_t>(i) & cmask) * 64u, tmem + 256u + (i & 3) * 8u,
               desc_at(db, (i & 1) * 32u), idesc, static_cast<uint32_t>(i) > cmask);
    } else {
#pragma unroll 8
      for (int i = 0; i < count; ++i)
        mma_ss(tmem + (static_cast<uint32_t>(i) & cmask) * 64u, desc_at(da, (i & 1) * 32u),
               desc_at(db, (i & 1) * 32u), idesc, static_cast<uint32_t>(i) > cmask);
    }
    t1 = clock64();
    mma_commit(smem_u32(&bar));
  }
  WaitCtx ctx{&abort_flag, status};
  mbar_wait(smem_u32(&bar), 0, ctx, 2);
  if (tid == 0) {
    const long long t2 = clock64();
    out[0] = static_cast<float>(t1 - t0);
    out[1] = static_cast<float>(t2 - t0);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace fwa2

// (development builds only: a micro-benchmark of the tcgen05.mma issue rate)
#ifdef FWA2_DEVELOPER
extern "C" int fwa2_selftest_mma_timing(int n, int a_tmem, int chains, int count, float* out,
                                        void* status, void* stream) {
  using namespace fwa2;
  if (n < 16 || n > 256 || (n % 16) != 0 || (chains != 1 && chains != 2 && chains != 4 && chains != 8) || count < 1 || count > 4096) return -1;
  const size_t smem = 65536 + 2048;
  cudaError_t e = cudaFuncSetAttribute(mma_timing_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return -100 - static_cast<int>(e);
  mma_timing_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      n, a_tmem, chains, count, out, static_cast<DeviceStatus*>(status));
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}

#endif  // FWA2_DEVELOPER

extern "C" int fwa2_selftest_mma(int mode, int dtype, const void* a, const void* b, float* d,
                                 void* status, void* stream) {
  using namespace fwa2;
  if (a == nullptr || b == nullptr || d == nullptr) return -1;   // FWA2_ERR_NULL: never reaches the device
  if (mode < 0 || mode > 3 || (dtype != 0 && dtype != 1)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = 32768 + 8192 + 1024;
  cudaError_t e;
  if (dtype == 1) {
    e = cudaFuncSetAttribute(selftest_kernel<__nv_bfloat16>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return -100 - static_cast<int>(e);
    selftest_kernel<__nv_bfloat16><<<1, 128, smem, st>>>(
        mode, static_cast<const uint16_t*>(a), static_cast<const uint16_t*>(b), d,
        static_cast<DeviceStatus*>(status));
  } else {
    e = cudaFuncSetAttribute(selftest_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem));
    if (e != cudaSuccess) return -100 - static_cast<int>(e);
    selftest_kernel<__half><<<1, 128, smem, st>>>(mode, static_cast<const uint16_t*>(a),
                                                  static_cast<const uint16_t*>(b), d,
                                                  static_cast<DeviceStatus*>(status));
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -100 - static_cast<int>(e);
}
