// Small kernels around the backward pass:
//   * transpose_tables: bias (H,N,N) and mask (nW,N,N) -> (planes, key, query) copies in the
//     workspace, which is the orientation the transposed backward kernel reads;
//   * reduce_partials: second stage of the deterministic dBias / dLogitScale reduction: sums the
//     per-CTA partial buffers in a fixed order, transposes back, and either casts to the output
//     dtype or leaves fp32 sums for a cross-GPU all-reduce;
//   * finalize: cast of an (all-reduced) fp32 buffer to the output dtype with the clamp gate on
//     dLogitScale (flash_win_attn_v2/kernels/attn_kernel_backward.py:703-711).
#include "fwa2_common.cuh"

namespace fwa2 {

template <typename T>
__device__ __forceinline__ uint16_t to_raw16(float x);
template <>
__device__ __forceinline__ uint16_t to_raw16<__nv_bfloat16>(float x) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}
template <>
__device__ __forceinline__ uint16_t to_raw16<__half>(float x) {
  return __half_as_ushort(__float2half_rn(x));
}

// 1[g <= ln 100], the comparison done in the parameter's own dtype like the reference does.
template <typename T>
__device__ __forceinline__ float clamp_gate(const void* logit_scale, int h) {
  const uint16_t raw = static_cast<const uint16_t*>(logit_scale)[h];
  const float g = Elem<T>::from_raw(raw);
  const float lim = Elem<T>::from_raw(to_raw16<T>(kLn100));
  return g <= lim ? 1.f : 0.f;
}

// dst[plane][j][i] = src[plane][i][j]; planes [0, n_bias) come from bias, the rest from mask.
__global__ void __launch_bounds__(256) transpose_tables_kernel(
    const uint16_t* __restrict__ bias, long long bias_pitch, uint16_t* __restrict__ bias_t,
    const uint16_t* __restrict__ mask, long long mask_pitch, uint16_t* __restrict__ mask_t,
    int n_bias, int n, int dst_pitch) {
  __shared__ uint16_t tile[32][33];
  const int plane = blockIdx.z;
  const uint16_t* src;
  uint16_t* dst;
  long long sp;
  if (plane < n_bias) {
    src = bias + static_cast<long long>(plane) * n * bias_pitch;
    dst = bias_t + static_cast<long long>(plane) * n * dst_pitch;
    sp = bias_pitch;
  } else {
    src = mask + static_cast<long long>(plane - n_bias) * n * mask_pitch;
    dst = mask_t + static_cast<long long>(plane - n_bias) * n * dst_pitch;
    sp = mask_pitch;
  }
  const int i0 = blockIdx.y * 32, j0 = blockIdx.x * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = i0 + ty + 8 * r, j = j0 + tx;
    tile[ty + 8 * r][tx] = (i < n && j < n) ? src[i * sp + j] : static_cast<uint16_t>(0);
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int j = j0 + ty + 8 * r, i = i0 + tx;
    if (j < n && i < dst_pitch) dst[static_cast<long long>(j) * dst_pitch + i] = (i < n) ? tile[tx][ty + 8 * r] : static_cast<uint16_t>(0);
  }
}

// Number of units CTA slot `s` (and, in pair mode, warpgroup w of it) accumulated.
__device__ __forceinline__ int units_of(const ReduceParams& p, int s, int w) {
  if (s >= p.BW) return 0;
  const int count = (p.BW - s + p.nslots - 1) / p.nslots;
  if (!p.pair) return count;
  return w == 0 ? (count + 1) / 2 : count / 2;
}

// One block sums an 8 (query) x 32 (key) patch of every partial buffer of its head; the partials
// are (query, key) like the result, so there is nothing to transpose.  The buffer list is dealt
// round-robin to kReduceLanes thread rows (threadIdx.y), each of which adds its buffers in
// ascending order; the sub-sums are then added in ascending order as well, so the result does not
// depend on timing.  Many thread rows keep the chain of dependent loads per thread short: the
// kernel is a few microseconds of latency, not bandwidth.
constexpr int kReduceLanes = 32;
template <typename T>
__global__ void __launch_bounds__(32 * kReduceLanes) reduce_partials_kernel(const ReduceParams p) {
  __shared__ float part[kReduceLanes][8][33];   // [buffer lane][query][key]
  const int h = blockIdx.z;
  const int j0 = blockIdx.x * 32, i0 = blockIdx.y * 8;
  const int tx = threadIdx.x, ty = threadIdx.y;
  if (p.db_partial != nullptr) {
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.f;
    const int nw = p.pair ? 2 : 1;
    const int nbuf = p.nslots * nw;
    const int j = j0 + tx;
    for (int b = ty; b < nbuf; b += kReduceLanes) {
      const int s = b / nw, w = b - s * nw;
      if (units_of(p, s, w) == 0) continue;
      const long long buf = static_cast<long long>(s * p.H + h) * nw + w;
      const float* src = p.db_partial + buf * p.buf_stride;
      if (j < p.N) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int i = i0 + r;
          if (i < p.N) acc[r] += src[static_cast<long long>(i) * p.pitch + j];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) part[ty][r][tx] = acc[r];
    __syncthreads();
    // thread (tx, ty < 8) finishes query i0 + ty, key j0 + tx
    if (ty < 8) {
      float v = 0.f;
#pragma unroll
      for (int l = 0; l < kReduceLanes; ++l) v += part[l][ty][tx];
      const int qi = i0 + ty, kj = j0 + tx;
      if (qi < p.N && kj < p.N) {
        const long long idx = (static_cast<long long>(h) * p.N + qi) * p.N + kj;
        if (p.out_f32 != nullptr) p.out_f32[idx] = v;
        else if (p.dbias != nullptr) static_cast<uint16_t*>(p.dbias)[idx] = to_raw16<T>(v);
      }
    }
  }
  // dLogitScale of head h: one warp, lane l adds slots l, l + 32, ... in ascending order, then a fixed
  // shuffle tree (all the loads of a lane are in flight together: a single thread walking the
  // list was the longest dependency chain of this kernel)
  if (blockIdx.x == 0 && blockIdx.y == 0 && ty == 0 && p.dscale_partial != nullptr) {
    float s = 0.f;
    for (int sl = tx; sl < p.dscale_slots; sl += 32) s += p.dscale_partial[sl * p.H + h];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
    if (tx != 0) {
      // lane 0 writes
    } else if (p.out_f32 != nullptr) {
      p.out_f32[static_cast<long long>(p.H) * p.N * p.N + h] = s;
    } else if (p.dscale != nullptr) {
      static_cast<uint16_t*>(p.dscale)[h] = to_raw16<T>(s * clamp_gate<T>(p.logit_scale, h));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) finalize_kernel(const float* __restrict__ partial, int H, int N,
                                                       const void* logit_scale, void* dbias,
                                                       void* dscale) {
  const long long total = static_cast<long long>(H) * N * N;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  if (dbias != nullptr) {
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
      static_cast<uint16_t*>(dbias)[i] = to_raw16<T>(partial[i]);
  }
  if (dscale != nullptr && blockIdx.x == 0 && threadIdx.x < H) {
    const int h = threadIdx.x;
    static_cast<uint16_t*>(dscale)[h] = to_raw16<T>(partial[total + h] * clamp_gate<T>(logit_scale, h));
  }
}

// cuTensorMapEncodeTiled is a driver call and needs the device's primary context current on the
// calling thread; a thread that has made no runtime call that touches the device yet (an autograd
// worker entering the backward pass) may not have it.  Looking up a kernel's attributes binds it.
cudaError_t ensure_context() {
  cudaFuncAttributes attr;
  return cudaFuncGetAttributes(&attr, transpose_tables_kernel);
}

cudaError_t launch_transpose_tables(const void* bias, long long bias_pitch, void* bias_t,
                                    const void* mask, long long mask_pitch, void* mask_t, int n_bias,
                                    int n_mask, int n, int dst_pitch, cudaStream_t stream) {
  if (n_bias + n_mask == 0) return cudaSuccess;
  dim3 grid((n + 31) / 32, (dst_pitch + 31) / 32, n_bias + n_mask), block(32, 8);
  transpose_tables_kernel<<<grid, block, 0, stream>>>(
      static_cast<const uint16_t*>(bias), bias_pitch, static_cast<uint16_t*>(bias_t),
      static_cast<const uint16_t*>(mask), mask_pitch, static_cast<uint16_t*>(mask_t), n_bias, n, dst_pitch);
  return cudaGetLastError();
}

cudaError_t launch_reduce_partials(const ReduceParams& p, int dtype_is_bf16, cudaStream_t stream) {
  dim3 grid(1, 1, p.H), block(32, kReduceLanes);
  if (p.db_partial != nullptr) {
    grid.x = (p.N + 31) / 32;
    grid.y = (p.N + 7) / 8;
  }
  if (dtype_is_bf16) reduce_partials_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(p);
  else reduce_partials_kernel<__half><<<grid, block, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_finalize(const float* partial, int dtype_is_bf16, int H, int N,
                            const void* logit_scale, void* dbias, void* dscale, cudaStream_t stream) {
  const long long total = static_cast<long long>(H) * N * N;
  int blocks = static_cast<int>((total + 255) / 256);
  if (blocks > 1184) blocks = 1184;
  if (blocks < 1) blocks = 1;
  if (dtype_is_bf16)
    finalize_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(partial, H, N, logit_scale, dbias, dscale);
  else
    finalize_kernel<__half><<<blocks, 256, 0, stream>>>(partial, H, N, logit_scale, dbias, dscale);
  return cudaGetLastError();
}

}  // namespace fwa2
