// Relative-position bias preparation of Swin-V2 and its backward, the step in front of the
// attention operator:  bias[h, i, j] = 16 * sigmoid(table[index[i, j], h])
// (flash_win_attn_v2/swin_transformer_v2.py:283-287: gather from the continuous-position-bias
// table, permute to (H, N, N), 16 * sigmoid).
//
// The backward takes the window-summed dBias in fp32, exactly as the attention backward leaves it
// in its `partial_out` buffer, so the gradient never passes through a 16-bit (H, N, N) tensor:
//   dtable[r, h] = 16 s (1 - s) * sum over {(i, j): index[i, j] = r} of dbias[h, i, j],  s = sigmoid(table[r, h]).
// The sum over the positions of a table row runs in a fixed order (inverse index in CSR form, built
// once by the caller), so the result is bitwise reproducible.  Both kernels are a few hundred
// thousand elements: bound by launch latency, not by any unit.
#include "../../include/fwa2.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace {

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float sigmoidf(float t) { return 1.f / (1.f + __expf(-t)); }

// One thread per (i, j): the index is read once, the H table values of its row are contiguous.
// The reference rounds sigmoid(t) to the table's dtype and then multiplies by 16 (exact).
template <typename TT, typename TO>
__global__ void __launch_bounds__(256) cpb_bias_fwd_kernel(const TT* __restrict__ table,
                                                           const int32_t* __restrict__ index, int nn, int heads,
                                                           int rows, TO* __restrict__ bias) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= nn) return;
  int r = index[e];
  r = r < 0 ? 0 : (r >= rows ? rows - 1 : r);
  const TT* trow = table + static_cast<long long>(r) * heads;
  for (int h = 0; h < heads; ++h) {
    const float s = to_f32(from_f32<TO>(sigmoidf(to_f32<TT>(trow[h]))));
    bias[static_cast<long long>(h) * nn + e] = from_f32<TO>(16.f * s);
  }
}

// One warp per table row: lane l adds positions l, l + 32, ... of the row's list in order, the 32
// sub-sums are combined by a fixed shuffle tree.
template <typename TT>
__global__ void __launch_bounds__(256) cpb_bias_bwd_kernel(const float* __restrict__ dbias,
                                                           const TT* __restrict__ table,
                                                           const int32_t* __restrict__ offsets,
                                                           const int32_t* __restrict__ positions, int nn,
                                                           int heads, int rows, float* __restrict__ dtable) {
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  // a malformed inverse index must not become an out-of-range read: offsets are clamped to the
  // list, positions outside the (n, n) table are skipped
  const int beg = max(0, min(offsets[r], nn)), end = max(beg, min(offsets[r + 1], nn));
  for (int h = 0; h < heads; ++h) {
    const float* src = dbias + static_cast<long long>(h) * nn;
    float acc = 0.f;
    for (int p = beg + lane; p < end; p += 32) {
      const int pos = positions[p];
      if (static_cast<unsigned>(pos) < static_cast<unsigned>(nn)) acc += src[pos];
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    if (lane == 0) {
      const float s = sigmoidf(to_f32<TT>(table[static_cast<long long>(r) * heads + h]));
      dtable[static_cast<long long>(r) * heads + h] = 16.f * s * (1.f - s) * acc;
    }
  }
}

}  // namespace
namespace fwa2 { void set_last_cuda_error(int e); }
namespace {

}  // namespace

extern "C" int fwa2_cpb_bias_forward(const void* table, int32_t table_is_f32, const int32_t* index, int32_t dtype,
                                     int32_t n, int32_t heads, int32_t rows, void* bias, void* stream) {
  if (table == nullptr || index == nullptr || bias == nullptr) return FWA2_ERR_NULL;
  if (dtype != FWA2_F16 && dtype != FWA2_BF16) return FWA2_ERR_DTYPE;
  if (n <= 0 || heads <= 0 || rows <= 0) return FWA2_ERR_SHAPE;
  const int nn = n * n;
  const dim3 grid((nn + 255) / 256), block(256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == FWA2_F16) {
    if (table_is_f32)
      cpb_bias_fwd_kernel<float, __half><<<grid, block, 0, st>>>(static_cast<const float*>(table), index, nn, heads,
                                                                 rows, static_cast<__half*>(bias));
    else
      cpb_bias_fwd_kernel<__half, __half><<<grid, block, 0, st>>>(static_cast<const __half*>(table), index, nn,
                                                                  heads, rows, static_cast<__half*>(bias));
  } else {
    if (table_is_f32)
      cpb_bias_fwd_kernel<float, __nv_bfloat16><<<grid, block, 0, st>>>(
          static_cast<const float*>(table), index, nn, heads, rows, static_cast<__nv_bfloat16*>(bias));
    else
      cpb_bias_fwd_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, block, 0, st>>>(
          static_cast<const __nv_bfloat16*>(table), index, nn, heads, rows, static_cast<__nv_bfloat16*>(bias));
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { fwa2::set_last_cuda_error(static_cast<int>(e)); return FWA2_ERR_LAUNCH; }
  return FWA2_OK;
}

extern "C" int fwa2_cpb_bias_backward(const float* dbias_f32, const void* table, int32_t table_is_f32,
                                      int32_t dtype, const int32_t* row_offsets, const int32_t* positions,
                                      int32_t n, int32_t heads, int32_t rows, float* dtable_f32, void* stream) {
  if (dbias_f32 == nullptr || table == nullptr || row_offsets == nullptr || positions == nullptr ||
      dtable_f32 == nullptr)
    return FWA2_ERR_NULL;
  if (dtype != FWA2_F16 && dtype != FWA2_BF16) return FWA2_ERR_DTYPE;
  if (n <= 0 || heads <= 0 || rows <= 0) return FWA2_ERR_SHAPE;
  const int nn = n * n;
  const dim3 grid((rows * 32 + 255) / 256), block(256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (table_is_f32)
    cpb_bias_bwd_kernel<float><<<grid, block, 0, st>>>(dbias_f32, static_cast<const float*>(table), row_offsets,
                                                       positions, nn, heads, rows, dtable_f32);
  else if (dtype == FWA2_F16)
    cpb_bias_bwd_kernel<__half><<<grid, block, 0, st>>>(dbias_f32, static_cast<const __half*>(table), row_offsets,
                                                        positions, nn, heads, rows, dtable_f32);
  else
    cpb_bias_bwd_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(dbias_f32, static_cast<const __nv_bfloat16*>(table),
                                                               row_offsets, positions, nn, heads, rows, dtable_f32);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { fwa2::set_last_cuda_error(static_cast<int>(e)); return FWA2_ERR_LAUNCH; }
  return FWA2_OK;
}
