// Host side of the C ABI: argument checks, TMA descriptor construction, shared-memory layout
// decisions and kernel launches.  Allocates nothing on the device and never synchronises.
#include "../../include/fwa2.h"

#include <cuda_runtime.h>

#include <cstring>

#include "fwa2_common.cuh"

namespace fwa2 {

cudaError_t launch_fwd(const FwdParams& p, int dtype_is_bf16, int p_in_tmem, int grid,
                       cudaStream_t stream);

namespace {

thread_local int g_last_cuda_error = 0;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is fetched through the runtime so that the library has no link-time
// dependency on libcuda and loads on machines without a GPU.
EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) {
      g_last_cuda_error = static_cast<int>(e);
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct DeviceInfo {
  int sm_count = 0;
  int max_smem_optin = 0;
  bool ok = false;
};

DeviceInfo device_info() {
  DeviceInfo d;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return d;
  if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return d;
  if (cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
    return d;
  d.ok = true;
  return d;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// (BW, H, N, 32) tensor of 16-bit elements -> 4-D map (d, N, H, BW), box (32, 64, 1, 1).
int encode_rows4(CUtensorMap* m, const fwa2_tensor4& t, int dtype, int bw, int h, int n) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return FWA2_ERR_DRIVER;
  if (t.ptr == nullptr) return FWA2_ERR_NULL;
  if (!aligned16(t.ptr)) return FWA2_ERR_ALIGN;
  const int64_t s[3] = {t.stride_n, t.stride_h, t.stride_bw};
  const int64_t ext[3] = {n, h, bw};
  for (int i = 0; i < 3; ++i) {
    // a dimension of extent 1 never uses its stride; give it a harmless legal value
    if (ext[i] > 1 && (s[i] <= 0 || (s[i] % 8) != 0)) return FWA2_ERR_STRIDE;
  }
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(n),
                        static_cast<cuuint64_t>(h), static_cast<cuuint64_t>(bw)};
  cuuint64_t strides[3];
  for (int i = 0; i < 3; ++i) {
    const int64_t se = (ext[i] > 1) ? s[i] : static_cast<int64_t>(kHeadDim);
    strides[i] = static_cast<cuuint64_t>(se) * 2u;
  }
  cuuint32_t box[4] = {static_cast<cuuint32_t>(kHeadDim), static_cast<cuuint32_t>(kBoxRows), 1u, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = enc(m, dtype == FWA2_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   4, t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return FWA2_ERR_TENSOR_MAP;
  }
  return FWA2_OK;
}

// (planes, rows, row_stride) table of 16-bit elements -> 3-D map (cols, rows, planes),
// box (32, 64, 1).
int encode_table3(CUtensorMap* m, const void* ptr, int dtype, int planes, int rows, int cols,
                  int64_t row_stride) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return FWA2_ERR_DRIVER;
  if (ptr == nullptr) return FWA2_ERR_NULL;
  if (!aligned16(ptr)) return FWA2_ERR_ALIGN;
  if (row_stride < cols || (row_stride % 8) != 0) return FWA2_ERR_STRIDE;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(planes)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_stride) * 2u,
                           static_cast<cuuint64_t>(row_stride) * 2u * static_cast<cuuint64_t>(rows)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kChunkCols), static_cast<cuuint32_t>(kBoxRows), 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = enc(m, dtype == FWA2_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return FWA2_ERR_TENSOR_MAP;
  }
  return FWA2_OK;
}

int check_common(int dtype, int bw, int heads, int n, int head_dim, int n_windows, bool has_mask) {
  if (dtype != FWA2_F16 && dtype != FWA2_BF16) return FWA2_ERR_DTYPE;
  if (head_dim != kHeadDim) return FWA2_ERR_HEAD_DIM;
  if (bw <= 0 || heads <= 0 || n <= 0 || n > 640) return FWA2_ERR_SHAPE;
  if (has_mask && (n_windows <= 0 || (bw % n_windows) != 0)) return FWA2_ERR_SHAPE;
  return FWA2_OK;
}

constexpr uint32_t kCtrlBytes = 512;

}  // namespace
}  // namespace fwa2

using namespace fwa2;

extern "C" int fwa2_abi_version(void) { return FWA2_ABI_VERSION; }

extern "C" int fwa2_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" const char* fwa2_strerror(int code) {
  switch (code) {
    case FWA2_OK: return "ok";
    case FWA2_ERR_NULL: return "a required pointer is null";
    case FWA2_ERR_DTYPE: return "dtype must be f16 or bf16";
    case FWA2_ERR_HEAD_DIM: return "only head dimension 32 is supported";
    case FWA2_ERR_SHAPE: return "invalid problem shape";
    case FWA2_ERR_STRIDE: return "stride not expressible by TMA (needs multiples of 8 elements)";
    case FWA2_ERR_ALIGN: return "base pointer not 16-byte aligned";
    case FWA2_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case FWA2_ERR_DRIVER: return "cuTensorMapEncodeTiled driver entry point unavailable";
    case FWA2_ERR_TENSOR_MAP: return "tensor map encoding failed";
    case FWA2_ERR_ABI: return "struct_size / abi_version mismatch";
    case FWA2_ERR_LAUNCH: return "kernel launch failed";
    default: return "unknown error";
  }
}

extern "C" int fwa2_forward(const fwa2_fwd_args* a, void* stream) {
  if (a == nullptr) return FWA2_ERR_NULL;
  if (a->struct_size != sizeof(fwa2_fwd_args) || a->abi_version != FWA2_ABI_VERSION) return FWA2_ERR_ABI;
  const bool has_bias = a->bias != nullptr, has_mask = a->mask != nullptr;
  int rc = check_common(a->dtype, a->bw, a->heads, a->n, a->head_dim, a->n_windows, has_mask);
  if (rc != FWA2_OK) return rc;
  if (a->o.ptr == nullptr || a->lse == nullptr || a->logit_scale == nullptr) return FWA2_ERR_NULL;
  if (!aligned16(a->o.ptr)) return FWA2_ERR_ALIGN;
  if ((a->o.stride_n % 8) != 0 || (a->o.stride_h % 8) != 0 || (a->o.stride_bw % 8) != 0) return FWA2_ERR_STRIDE;

  FwdParams p;
  std::memset(&p, 0, sizeof(p));
  if ((rc = encode_rows4(&p.tm_q, a->q, a->dtype, a->bw, a->heads, a->n)) != FWA2_OK) return rc;
  if ((rc = encode_rows4(&p.tm_k, a->k, a->dtype, a->bw, a->heads, a->n)) != FWA2_OK) return rc;
  if ((rc = encode_rows4(&p.tm_v, a->v, a->dtype, a->bw, a->heads, a->n)) != FWA2_OK) return rc;
  if (has_bias &&
      (rc = encode_table3(&p.tm_bias, a->bias, a->dtype, a->heads, a->n, a->n, a->bias_row_stride)) != FWA2_OK)
    return rc;
  if (has_mask &&
      (rc = encode_table3(&p.tm_mask, a->mask, a->dtype, a->n_windows, a->n, a->n, a->mask_row_stride)) != FWA2_OK)
    return rc;

  const DeviceInfo dev = device_info();
  if (!dev.ok) return FWA2_ERR_LAUNCH;

  p.o = a->o.ptr;
  p.o_sbw = a->o.stride_bw; p.o_sh = a->o.stride_h; p.o_sn = a->o.stride_n;
  p.lse = a->lse; p.lse_sbw = a->lse_stride_bw; p.lse_sh = a->lse_stride_h;
  p.scale = a->logit_scale; p.scale_is_tensor = a->scale_is_tensor;
  p.BW = a->bw; p.H = a->heads; p.N = a->n; p.nW = has_mask ? a->n_windows : 1;
  p.has_bias = has_bias; p.has_mask = has_mask;
  p.pair_mode = a->n <= 64;
  const int units = a->bw * a->heads;
  p.n_jobs = p.pair_mode ? (units + 1) / 2 : units;
  p.status = static_cast<DeviceStatus*>(a->status);

  // ---- shared memory layout: prefer two CTAs per SM ----
  const bool p_in_tmem = a->variant != 1;
  const uint32_t rows_kv = p.pair_mode ? 128u : static_cast<uint32_t>((a->n + 63) / 64) * 64u;
  p.kv_stage_bytes = 2u * rows_kv * kRowBytes;
  const uint32_t p_bytes = p_in_tmem ? 0u : (p.pair_mode ? 32768u : 16384u);
  const uint32_t bm_stage = 2u * kTableTileBytes;
  auto total = [&](uint32_t nkv, uint32_t nbm) {
    return nkv * p.kv_stage_bytes + 2u * 2u * kBoxBytes + nbm * bm_stage + p_bytes + kCtrlBytes;
  };
  const uint32_t budget_two = static_cast<uint32_t>(dev.max_smem_optin + 1024) / 2u - 1024u;
  const uint32_t budget_one = static_cast<uint32_t>(dev.max_smem_optin);
  uint32_t nkv = 2, nbm = 3;
  int ctas_per_sm = 2;
  if (total(2, 3) <= budget_two) { nkv = 2; nbm = 3; }
  else if (total(2, 2) <= budget_two) { nkv = 2; nbm = 2; }
  else if (total(1, 2) <= budget_two) { nkv = 1; nbm = 2; }
  else {
    ctas_per_sm = 1;
    if (total(2, 4) <= budget_one) { nkv = 2; nbm = 4; }
    else if (total(1, 4) <= budget_one) { nkv = 1; nbm = 4; }
    else if (total(1, 2) <= budget_one) { nkv = 1; nbm = 2; }
    else return FWA2_ERR_SHAPE;
  }
  p.n_kv_stages = static_cast<int>(nkv);
  p.n_bm_stages = static_cast<int>(nbm);
  p.off_kv = 0;
  p.off_q = p.off_kv + nkv * p.kv_stage_bytes;
  p.off_bm = p.off_q + 2u * 2u * kBoxBytes;
  p.off_p = p.off_bm + nbm * bm_stage;
  p.off_ctrl = p.off_p + p_bytes;
  p.smem_bytes = p.off_ctrl + kCtrlBytes;

  int grid = dev.sm_count * ctas_per_sm;
  if (a->max_ctas > 0 && grid > a->max_ctas) grid = a->max_ctas;
  if (grid > p.n_jobs) grid = p.n_jobs;
  cudaError_t e = launch_fwd(p, a->dtype == FWA2_BF16, p_in_tmem ? 1 : 0, grid,
                             static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return FWA2_ERR_LAUNCH;
  }
  return FWA2_OK;
}
