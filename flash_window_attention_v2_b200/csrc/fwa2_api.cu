// Host side of the C ABI: argument checks, TMA descriptor construction, shared-memory layout
// decisions and kernel launches.  Allocates nothing on the device and never synchronises.
#include "../../include/fwa2.h"

#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "fwa2_common.cuh"

namespace fwa2 {

cudaError_t launch_fwd(const FwdParams& p, int dtype_is_bf16, int p_in_tmem, int grid,
                       cudaStream_t stream);
cudaError_t launch_fwd_duo(const FwdParams& p, int dtype_is_bf16, int grid, cudaStream_t stream);
cudaError_t launch_combine_tables(const void* bias, long long bias_pitch, const void* mask, long long mask_pitch,
                                  float* out, int n, int heads, int n_windows, int pitch, int dtype_is_bf16,
                                  cudaStream_t stream);
cudaError_t launch_bwd(const BwdParams& p, int dtype_is_bf16, int grid, cudaStream_t stream);
cudaError_t launch_bwd_quad(const QuadParams& p, int dtype_is_bf16, int grid, cudaStream_t stream);
int quad_max_active_clusters(int dtype_is_bf16, int cluster, uint32_t smem_bytes);
cudaError_t launch_transpose_tables(const void* bias, long long bias_pitch, void* bias_t,
                                    const void* mask, long long mask_pitch, void* mask_t, int n_bias,
                                    int n_mask, int n, int dst_pitch, cudaStream_t stream);
cudaError_t launch_reduce_partials(const ReduceParams& p, int dtype_is_bf16, cudaStream_t stream);
cudaError_t ensure_context();
cudaError_t launch_finalize(const float* partial, int dtype_is_bf16, int H, int N,
                            const void* logit_scale, void* dbias, void* dscale, cudaStream_t stream);

namespace {

// development builds only: leave dBias out of the backward (timing experiments)
#ifdef FWA2_DEVELOPER
constexpr int kSkipDbias = 8;
#else
constexpr int kSkipDbias = 0;
#endif

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
int encode_rows4(CUtensorMap* m, const fwa2_tensor4& t, int dtype, int bw, int h, int n, int box_rows = kBoxRows) {
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
  cuuint32_t box[4] = {static_cast<cuuint32_t>(kHeadDim), static_cast<cuuint32_t>(box_rows), 1u, 1u};
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

// (planes, rows, pitch) fp32 table -> 3-D map (cols, rows, planes), box (32, 128, 1): rows of 128
// bytes, 128-byte swizzle.
int encode_comb3(CUtensorMap* m, const void* ptr, int planes, int rows, int cols, int pitch) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return FWA2_ERR_DRIVER;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(planes)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(pitch) * 4u,
                           static_cast<cuuint64_t>(pitch) * 4u * static_cast<cuuint64_t>(rows)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(kChunkCols), static_cast<cuuint32_t>(kTileRows), 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return FWA2_ERR_TENSOR_MAP;
  }
  return FWA2_OK;
}

// The forward kernel for windows of 129 to 256 tokens can read ONE fp32 table, bias + mask, per
// (window type, head) instead of the two 16-bit tables: two conversions and an addition less per
// score.  Building that table costs a pass of its own (4 * nW * H * N * pitch bytes written), which
// pays once every table is used by enough units, i.e. images.
constexpr int kCombMinImages = 24;
int comb_pitch(int n) { return ((n + 31) / 32) * 32; }
bool comb_applies(int bw, int n, int n_windows, bool has_bias, bool has_mask, int variant) {
  if (!has_bias || !has_mask || n <= 128 || n > 256 || n_windows <= 0 || (bw % n_windows) != 0) return false;
  if (variant & (FWA2_FWD_SEPARATE_TABLES | FWA2_FWD_GENERAL_KERNEL | FWA2_FWD_P_IN_SMEM)) return false;
  return (variant & FWA2_FWD_COMBINE_TABLES) != 0 || bw / n_windows >= kCombMinImages;
}

int check_common(int dtype, int bw, int heads, int n, int head_dim, int n_windows, bool has_mask) {
  if (dtype != FWA2_F16 && dtype != FWA2_BF16) return FWA2_ERR_DTYPE;
  if (head_dim != kHeadDim) return FWA2_ERR_HEAD_DIM;
  if (bw <= 0 || heads <= 0 || heads > 192 || n <= 0 || n > 640) return FWA2_ERR_SHAPE;
  if (has_mask && (n_windows <= 0 || (bw % n_windows) != 0)) return FWA2_ERR_SHAPE;
  return FWA2_OK;
}

constexpr uint32_t kCtrlBytes = 1024;   // mbarriers + control words [0, 256), per-head scales [256, 1024)

size_t align256(size_t x) { return (x + 255u) & ~static_cast<size_t>(255u); }

// How the backward pass carves up its workspace and its grid.
struct BwdPlan {
  int pair, quad, cluster, nslots, grid, n_bufs, table_pitch, db_pitch;
  size_t off_bias_t, off_mask_t, off_db, off_dscale, total;
};

// Windows of 65 to 256 tokens go to the cluster kernel (fwa2_bwd_quad.cu) unless the caller asks
// for the general one.
bool wants_quad(int n, int variant) { return n > 64 && n <= 256 && (variant & FWA2_BWD_GENERAL_KERNEL) == 0; }

BwdPlan make_bwd_plan(int bw, int heads, int n, int n_windows, bool has_bias, bool has_mask,
                      int sm_count, bool quad) {
  BwdPlan pl;
  pl.pair = n <= 64;
  pl.quad = quad ? 1 : 0;
  pl.cluster = quad ? (n > kTileRows ? 4 : 1) : 1;
  const int groups = sm_count / pl.cluster;   // CTAs, or clusters, that can be resident
  const int per_head = groups / heads > 0 ? groups / heads : 1;
  const int jobs = pl.pair ? (bw + 1) / 2 : bw;
  pl.nslots = per_head < jobs ? per_head : jobs;
  pl.grid = pl.nslots * heads * pl.cluster;
  pl.n_bufs = pl.nslots * heads * (pl.pair ? 2 : 1);
  pl.table_pitch = ((n + 7) / 8) * 8;
  pl.db_pitch = ((n + 31) / 32) * 32;
  size_t off = 0;
  pl.off_bias_t = off;
  if (has_bias) off += align256(static_cast<size_t>(heads) * n * pl.table_pitch * 2u);
  pl.off_mask_t = off;
  if (has_mask) off += align256(static_cast<size_t>(n_windows) * n * pl.table_pitch * 2u);
  pl.off_db = off;
  if (has_bias) off += align256(static_cast<size_t>(pl.n_bufs) * pl.db_pitch * pl.db_pitch * 4u);
  pl.off_dscale = off;
  off += align256(static_cast<size_t>(pl.nslots) * heads * pl.cluster * 4u);
  pl.total = off;
  return pl;
}

// Shared-memory layout of the cluster kernel; false if it does not fit.
bool quad_smem_plan(QuadParams& p, uint32_t budget) {
  const uint32_t mask_b = p.has_mask ? 2u * 32768u : 0u;
  const uint32_t recv_b = p.cluster > 1 ? 3u * 64u * 128u : 0u;
  auto total = [&](uint32_t ns) {
    return ns * 32768u + mask_b + 32768u + recv_b + 4096u + ns * 1024u + kCtrlBytes;
  };
  uint32_t ns = 3;
  if (total(ns) > budget) ns = 2;
  if (total(ns) > budget) return false;
  p.n_stages = static_cast<int>(ns);
  p.n_mask_stages = 2;
  p.off_stage = 0;
  p.off_mask = p.off_stage + ns * 32768u;
  p.off_ds = p.off_mask + mask_b;
  p.off_recv = p.off_ds + 32768u;
  p.off_ident = p.off_recv + recv_b;
  p.off_rowstats = p.off_ident + 4096u;
  p.off_ctrl = p.off_rowstats + ns * 1024u;
  p.smem_bytes = p.off_ctrl + kCtrlBytes;
  return true;
}

// Resident clusters per device for the cluster kernel, looked up once per
// (device, dtype, cluster size, shared-memory size).
int cached_max_clusters(int dtype_is_bf16, int cluster, uint32_t smem_bytes) {
  struct Entry { int dev, bf16, cluster; uint32_t smem; int value; };
  static std::mutex mu;
  static Entry cache[32];
  static int used = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used; ++i)
    if (cache[i].dev == dev && cache[i].bf16 == dtype_is_bf16 && cache[i].cluster == cluster && cache[i].smem == smem_bytes)
      return cache[i].value;
  const int v = quad_max_active_clusters(dtype_is_bf16, cluster, smem_bytes);
  if (v > 0 && used < 32) cache[used++] = Entry{dev, dtype_is_bf16, cluster, smem_bytes, v};
  return v;
}

}  // namespace
}  // namespace fwa2

namespace fwa2 {
// for the other translation units of the library: what fwa2_last_cuda_error() reports
void set_last_cuda_error(int e) { g_last_cuda_error = e; }
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
    case FWA2_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the built-in static array holds";
    default: return "unknown error";
  }
}

extern "C" size_t fwa2_fwd_workspace_bytes(int32_t bw, int32_t heads, int32_t n, int32_t n_windows,
                                           int32_t has_bias, int32_t has_mask, int32_t variant) {
  if (bw <= 0 || heads <= 0 || heads > 192 || n <= 0) return 0;
  if (!comb_applies(bw, n, n_windows, has_bias != 0, has_mask != 0, variant)) return 0;
  return align256(static_cast<size_t>(n_windows) * heads * n * comb_pitch(n) * 4u);
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

  {
    const cudaError_t ce = ensure_context();   // the tensor maps below are encoded by a driver call
    if (ce != cudaSuccess) { g_last_cuda_error = static_cast<int>(ce); return FWA2_ERR_LAUNCH; }
  }
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
  p.trace.buf = reinterpret_cast<unsigned long long*>(a->developer0);
  p.trace.cap = a->developer0 != nullptr ? a->developer1 : 0;

  const bool p_in_tmem = (a->variant & FWA2_FWD_P_IN_SMEM) == 0;
  const uint32_t budget_two = static_cast<uint32_t>(dev.max_smem_optin + 1024) / 2u - 1024u;

  // ---- windows of 129 to 256 tokens: two softmax warpgroups per CTA, one per tile of the unit ----
  if (a->n > 128 && a->n <= 256 && p_in_tmem && (a->variant & FWA2_FWD_GENERAL_KERNEL) == 0) {
    const uint32_t rows = static_cast<uint32_t>((a->n + 63) / 64) * 64u;
    p.kv_stage_bytes = rows * kRowBytes;
    // K and Q have one buffer each.  Four table stages (two per tile) matter more than a second
    // V buffer: the next unit's V is not needed before its first step is through the softmax.
    const bool tables = has_bias || has_mask;
    const uint32_t fixed = rows * kRowBytes + 4u * kBoxBytes + kCtrlBytes;
    const uint32_t t_stage = 2u * kTableTileBytes;
    uint32_t nv = 2, nt = tables ? 4u : 0u;
    if (fixed + nv * rows * kRowBytes + nt * t_stage > budget_two) nv = 1;
    if (fixed + nv * rows * kRowBytes + nt * t_stage > budget_two) nt = 3;
    p.n_kv_stages = static_cast<int>(nv);               // of V
    p.n_bm_stages = static_cast<int>(tables ? nt : 3u);
    p.off_kv = 0;                                       // K
    p.off_q = p.off_kv + rows * kRowBytes;              // Q: 256 rows
    p.off_p = p.off_q + 4u * kBoxBytes;                 // V
    p.off_bm = p.off_p + nv * rows * kRowBytes;         // table chunks: stages of [bias | mask]
    p.off_ctrl = p.off_bm + nt * t_stage;
    p.smem_bytes = p.off_ctrl + kCtrlBytes;
    if (p.smem_bytes <= budget_two) {
      int grid = dev.sm_count * 2;
      if (a->max_ctas > 0 && grid > a->max_ctas) grid = a->max_ctas;
      if (grid > p.n_jobs) grid = p.n_jobs;
      // ---- one fp32 table (bias + mask) per (window type, head), when it pays ----
      const size_t comb_bytes = fwa2_fwd_workspace_bytes(a->bw, a->heads, a->n, a->n_windows, has_bias, has_mask,
                                                         a->variant);
      if (comb_bytes != 0) {
        const bool usable = a->workspace != nullptr && a->workspace_bytes >= comb_bytes &&
                            (reinterpret_cast<uintptr_t>(a->workspace) & 255u) == 0;
        if (!usable && (a->variant & FWA2_FWD_COMBINE_TABLES)) return FWA2_ERR_WORKSPACE;
        if (usable) {
          const int pitch = comb_pitch(a->n);
          if ((rc = encode_comb3(&p.tm_bias, a->workspace, a->n_windows * a->heads, a->n, a->n, pitch)) != FWA2_OK)
            return rc;
          const cudaError_t ce = launch_combine_tables(a->bias, a->bias_row_stride, a->mask, a->mask_row_stride,
                                                       static_cast<float*>(a->workspace), a->n, a->heads,
                                                       a->n_windows, pitch, a->dtype == FWA2_BF16,
                                                       static_cast<cudaStream_t>(stream));
          if (ce != cudaSuccess) {
            g_last_cuda_error = static_cast<int>(ce);
            return FWA2_ERR_LAUNCH;
          }
          p.comb = 1;
          p.n_img = a->bw / a->n_windows;
        }
      }
      const cudaError_t e = launch_fwd_duo(p, a->dtype == FWA2_BF16, grid, static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) {
        g_last_cuda_error = static_cast<int>(e);
        return FWA2_ERR_LAUNCH;
      }
      return FWA2_OK;
    }
  }

  // ---- shared memory layout: prefer two CTAs per SM ----
  const uint32_t rows_kv = p.pair_mode ? 128u : static_cast<uint32_t>((a->n + 63) / 64) * 64u;
  p.kv_stage_bytes = 2u * rows_kv * kRowBytes;
  const uint32_t p_bytes = p_in_tmem ? 0u : (p.pair_mode ? 32768u : 16384u);
  const uint32_t bm_stage = 2u * kTableTileBytes;
  auto total = [&](uint32_t nkv, uint32_t nbm) {
    return nkv * p.kv_stage_bytes + 2u * 2u * kBoxBytes + nbm * bm_stage + p_bytes + kCtrlBytes;
  };
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

extern "C" size_t fwa2_bwd_workspace_bytes(int32_t bw, int32_t heads, int32_t n, int32_t n_windows,
                                           int32_t has_bias, int32_t has_mask) {
  if (bw <= 0 || heads <= 0 || n <= 0 || n > 640 || (has_mask && n_windows <= 0)) return 0;
  const DeviceInfo dev = device_info();
  const int sms = dev.ok ? dev.sm_count : 148;
  // enough for either kernel that serves this window size
  size_t need = make_bwd_plan(bw, heads, n, n_windows, has_bias != 0, has_mask != 0, sms, false).total;
  if (wants_quad(n, 0)) {
    const size_t q = make_bwd_plan(bw, heads, n, n_windows, has_bias != 0, has_mask != 0, sms, true).total;
    if (q > need) need = q;
  }
  return need;
}

extern "C" int fwa2_backward(const fwa2_bwd_args* a, void* stream_v) {
  if (a == nullptr) return FWA2_ERR_NULL;
  if (a->struct_size != sizeof(fwa2_bwd_args) || a->abi_version != FWA2_ABI_VERSION) return FWA2_ERR_ABI;
  const bool has_bias = a->bias != nullptr, has_mask = a->mask != nullptr;
  int rc = check_common(a->dtype, a->bw, a->heads, a->n, a->head_dim, a->n_windows, has_mask);
  if (rc != FWA2_OK) return rc;
  if (a->lse == nullptr || a->logit_scale == nullptr) return FWA2_ERR_NULL;
  const fwa2_tensor4* plain[] = {&a->q, &a->k, &a->o, &a->dq, &a->dk, &a->dv};
  for (const fwa2_tensor4* t : plain) {
    if (t->ptr == nullptr) return FWA2_ERR_NULL;
    if (!aligned16(t->ptr)) return FWA2_ERR_ALIGN;
    if ((t->stride_n % 8) != 0 || (t->stride_h % 8) != 0 || (t->stride_bw % 8) != 0) return FWA2_ERR_STRIDE;
  }
  if (has_bias && a->dbias == nullptr && a->partial_out == nullptr) return FWA2_ERR_NULL;
  if (has_bias && (a->bias_row_stride < a->n)) return FWA2_ERR_STRIDE;
  if (has_mask && (a->mask_row_stride < a->n)) return FWA2_ERR_STRIDE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int is_bf16 = a->dtype == FWA2_BF16;

  const DeviceInfo dev = device_info();
  if (!dev.ok) return FWA2_ERR_LAUNCH;
  {
    const cudaError_t ce = ensure_context();   // the tensor maps below are encoded by a driver call
    if (ce != cudaSuccess) { g_last_cuda_error = static_cast<int>(ce); return FWA2_ERR_LAUNCH; }
  }
  const bool quad = wants_quad(a->n, a->variant);
  BwdPlan pl = make_bwd_plan(a->bw, a->heads, a->n, a->n_windows, has_bias, has_mask, dev.sm_count, quad);
  if (a->workspace == nullptr || a->workspace_bytes < pl.total ||
      (reinterpret_cast<uintptr_t>(a->workspace) & 255u) != 0)
    return FWA2_ERR_WORKSPACE;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  void* bias_t = ws + pl.off_bias_t;
  void* mask_t = ws + pl.off_mask_t;
  float* db_partial = (has_bias && (a->variant & kSkipDbias) == 0) ? reinterpret_cast<float*>(ws + pl.off_db) : nullptr;
  float* dscale_partial = reinterpret_cast<float*>(ws + pl.off_dscale);

  // Everything that can fail is checked and every descriptor is encoded before the first launch:
  // a rejected call leaves the workspace and the outputs untouched.
  BwdParams p;
  QuadParams qp;
  std::memset(&p, 0, sizeof(p));
  std::memset(&qp, 0, sizeof(qp));
  if (quad) {
    if ((rc = encode_rows4(&qp.tm_q, a->q, a->dtype, a->bw, a->heads, a->n)) != FWA2_OK) return rc;
    if ((rc = encode_rows4(&qp.tm_k, a->k, a->dtype, a->bw, a->heads, a->n)) != FWA2_OK) return rc;
    if ((rc = encode_rows4(&qp.tm_v, a->v, a->dtype, a->bw, a->heads, a->n)) != FWA2_OK) return rc;
    if ((rc = encode_rows4(&qp.tm_do, a->dout, a->dtype, a->bw, a->heads, a->n)) != FWA2_OK) return rc;
    qp.bias_t = has_bias ? bias_t : nullptr;
    qp.table_pitch = pl.table_pitch;
    if (has_mask &&
        (rc = encode_table3(&qp.tm_maskT, mask_t, a->dtype, a->n_windows, a->n, a->n, pl.table_pitch)) != FWA2_OK)
      return rc;
    qp.q = a->q.ptr; qp.q_sbw = a->q.stride_bw; qp.q_sh = a->q.stride_h; qp.q_sn = a->q.stride_n;
    qp.k = a->k.ptr; qp.k_sbw = a->k.stride_bw; qp.k_sh = a->k.stride_h; qp.k_sn = a->k.stride_n;
    qp.o = a->o.ptr; qp.o_sbw = a->o.stride_bw; qp.o_sh = a->o.stride_h; qp.o_sn = a->o.stride_n;
    qp.dq = a->dq.ptr; qp.dq_sbw = a->dq.stride_bw; qp.dq_sh = a->dq.stride_h; qp.dq_sn = a->dq.stride_n;
    qp.dk = a->dk.ptr; qp.dk_sbw = a->dk.stride_bw; qp.dk_sh = a->dk.stride_h; qp.dk_sn = a->dk.stride_n;
    qp.dv = a->dv.ptr; qp.dv_sbw = a->dv.stride_bw; qp.dv_sh = a->dv.stride_h; qp.dv_sn = a->dv.stride_n;
    qp.lse = a->lse; qp.lse_sbw = a->lse_stride_bw; qp.lse_sh = a->lse_stride_h;
    qp.scale = a->logit_scale; qp.scale_is_tensor = a->scale_is_tensor;
    qp.db_partial = db_partial;
    qp.db_pitch = pl.db_pitch;
    qp.db_buf_stride = static_cast<long long>(pl.db_pitch) * pl.db_pitch;
    qp.dscale_partial = dscale_partial;
    qp.BW = a->bw; qp.H = a->heads; qp.N = a->n; qp.nW = has_mask ? a->n_windows : 1;
    qp.has_bias = has_bias; qp.has_mask = has_mask;
    qp.cluster = pl.cluster;
    qp.status = static_cast<DeviceStatus*>(a->status);
    qp.prof = (a->developer0 != nullptr && a->developer1 >= 64) ? reinterpret_cast<unsigned long long*>(a->developer0) : nullptr;
    if (!quad_smem_plan(qp, static_cast<uint32_t>(dev.max_smem_optin))) return FWA2_ERR_SHAPE;
    // no more clusters than the device holds at once (fewer clusters use a prefix of the
    // workspace's partial buffers)
    int max_clusters = cached_max_clusters(is_bf16, pl.cluster, qp.smem_bytes);
    if (max_clusters <= 0) return FWA2_ERR_LAUNCH;
    if (a->max_ctas > 0 && a->max_ctas / pl.cluster < max_clusters) max_clusters = a->max_ctas / pl.cluster;
    int ns = max_clusters / a->heads;
    if (ns < 1) ns = 1;
    if (ns < pl.nslots) { pl.nslots = ns; pl.grid = ns * a->heads * pl.cluster; }
    qp.nslots = pl.nslots;
  } else {
    if (a->max_ctas > 0 && pl.grid > a->max_ctas) {
      // a smaller grid keeps the same workspace layout (it only uses a prefix of it)
      int ns = a->max_ctas / a->heads;
      if (ns < 1) ns = 1;
      if (ns < pl.nslots) { pl.nslots = ns; pl.grid = ns * a->heads; }
    }
    // pair mode loads Q and dO in boxes of 32 rows, so that the queries of the two units can be
    // interleaved in shared memory (see the kernel)
    const int q_box_rows = pl.pair ? 32 : kBoxRows;
    if ((rc = encode_rows4(&p.tm_q, a->q, a->dtype, a->bw, a->heads, a->n, q_box_rows)) != FWA2_OK) return rc;
    if ((rc = encode_rows4(&p.tm_k, a->k, a->dtype, a->bw, a->heads, a->n)) != FWA2_OK) return rc;
    if ((rc = encode_rows4(&p.tm_v, a->v, a->dtype, a->bw, a->heads, a->n)) != FWA2_OK) return rc;
    if ((rc = encode_rows4(&p.tm_do, a->dout, a->dtype, a->bw, a->heads, a->n, q_box_rows)) != FWA2_OK) return rc;
    if (has_bias &&
        (rc = encode_table3(&p.tm_biasT, bias_t, a->dtype, a->heads, a->n, a->n, pl.table_pitch)) != FWA2_OK)
      return rc;
    if (has_mask &&
        (rc = encode_table3(&p.tm_maskT, mask_t, a->dtype, a->n_windows, a->n, a->n, pl.table_pitch)) != FWA2_OK)
      return rc;

    p.q = a->q.ptr; p.q_sbw = a->q.stride_bw; p.q_sh = a->q.stride_h; p.q_sn = a->q.stride_n;
    p.k = a->k.ptr; p.k_sbw = a->k.stride_bw; p.k_sh = a->k.stride_h; p.k_sn = a->k.stride_n;
    p.o = a->o.ptr; p.o_sbw = a->o.stride_bw; p.o_sh = a->o.stride_h; p.o_sn = a->o.stride_n;
    p.dq = a->dq.ptr; p.dq_sbw = a->dq.stride_bw; p.dq_sh = a->dq.stride_h; p.dq_sn = a->dq.stride_n;
    p.dk = a->dk.ptr; p.dk_sbw = a->dk.stride_bw; p.dk_sh = a->dk.stride_h; p.dk_sn = a->dk.stride_n;
    p.dv = a->dv.ptr; p.dv_sbw = a->dv.stride_bw; p.dv_sh = a->dv.stride_h; p.dv_sn = a->dv.stride_n;
    p.lse = a->lse; p.lse_sbw = a->lse_stride_bw; p.lse_sh = a->lse_stride_h;
    p.scale = a->logit_scale; p.scale_is_tensor = a->scale_is_tensor;
    p.db_partial = db_partial;
    p.db_pitch = pl.db_pitch;
    p.db_buf_stride = static_cast<long long>(pl.db_pitch) * pl.db_pitch;
    p.dscale_partial = dscale_partial;
    p.BW = a->bw; p.H = a->heads; p.N = a->n; p.nW = has_mask ? a->n_windows : 1;
    p.has_bias = has_bias; p.has_mask = has_mask;
    p.pair_mode = pl.pair;
    p.nslots = pl.nslots;
    p.status = static_cast<DeviceStatus*>(a->status);
    p.trace.buf = reinterpret_cast<unsigned long long*>(a->developer0);
    p.trace.cap = a->developer0 != nullptr ? a->developer1 : 0;

    // ---- shared memory layout (one CTA per SM) ----
    p.rows_kv = pl.pair ? 128 : ((a->n + 127) / 128) * 128;
    p.kv_stage_bytes = 2u * static_cast<uint32_t>(p.rows_kv) * kRowBytes;
    const uint32_t qdo_bytes = 3u * 4u * kBoxBytes;
    const uint32_t bm_stage = 2u * kTableTileBytes;
    const bool any_table = has_bias || has_mask;
    auto total = [&](uint32_t nkv, uint32_t nds, uint32_t nbm) {
      return nkv * p.kv_stage_bytes + qdo_bytes + nds * 32768u + (any_table ? 2u * nbm * bm_stage : 0u) +
             4096u + nkv * static_cast<uint32_t>(p.rows_kv) * 4u + 3u * 1024u + kCtrlBytes;
    };
    const uint32_t budget = static_cast<uint32_t>(dev.max_smem_optin);
    // Preference order.  Jobs of a single tile (windows of at most 128 tokens) release their
    // K/V stage only in the epilogue that runs one tile late, so they want four stages to keep a
    // whole tile of lead for the next load (see bwd_num_sets() in the kernel).
    const uint32_t opts[][3] = {{4, 2, 2}, {4, 2, 1}, {4, 1, 2}, {3, 2, 2}, {3, 1, 2}, {2, 2, 2}, {2, 1, 2},
                                {1, 2, 2}, {1, 1, 2}, {1, 1, 1}};
    uint32_t nkv = 0, nds = 0, nbm = 0;
    for (const auto& o : opts) {
      if (o[0] >= 3 && p.rows_kv > 128) continue;
      // one table stage per warpgroup is enough only in pair mode (one chunk per tile and warpgroup)
      if (o[0] == 4 && o[2] == 1 && !pl.pair) continue;
      if (total(o[0], o[1], o[2]) <= budget) { nkv = o[0]; nds = o[1]; nbm = o[2]; break; }
    }
    if (nkv == 0) return FWA2_ERR_SHAPE;
    p.n_kv_stages = static_cast<int>(nkv);
    p.n_ds_bufs = static_cast<int>(nds);
    p.n_bm_stages = static_cast<int>(nbm);
    p.off_kv = 0;
    p.off_qdo = p.off_kv + nkv * p.kv_stage_bytes;
    p.off_ds = p.off_qdo + qdo_bytes;
    p.off_bm = p.off_ds + nds * 32768u;
    p.off_ident = p.off_bm + (any_table ? 2u * nbm * bm_stage : 0u);
    p.off_rk = p.off_ident + 4096u;
    p.off_rowstats = p.off_rk + nkv * static_cast<uint32_t>(p.rows_kv) * 4u;
    p.off_ctrl = p.off_rowstats + 3u * 1024u;
    p.smem_bytes = p.off_ctrl + kCtrlBytes;
  }

  cudaError_t e = cudaSuccess;
  if ((a->variant & FWA2_BWD_SKIP_TABLES) == 0) {
    e = launch_transpose_tables(a->bias, a->bias_row_stride, bias_t, a->mask, a->mask_row_stride,
                                mask_t, has_bias ? a->heads : 0, has_mask ? a->n_windows : 0, a->n,
                                pl.table_pitch, stream);
    if (e != cudaSuccess) { g_last_cuda_error = static_cast<int>(e); return FWA2_ERR_LAUNCH; }
  }

  e = quad ? launch_bwd_quad(qp, is_bf16, pl.grid, stream) : launch_bwd(p, is_bf16, pl.grid, stream);
  if (e != cudaSuccess) { g_last_cuda_error = static_cast<int>(e); return FWA2_ERR_LAUNCH; }

  if ((has_bias || a->scale_is_tensor) && (a->variant & FWA2_BWD_SKIP_REDUCE) == 0) {
    ReduceParams r;
    std::memset(&r, 0, sizeof(r));
    r.db_partial = db_partial;
    r.buf_stride = static_cast<long long>(pl.db_pitch) * pl.db_pitch;
    r.pitch = pl.db_pitch;
    r.dscale_partial = a->scale_is_tensor ? dscale_partial : nullptr;
    r.H = a->heads; r.N = a->n; r.BW = a->bw; r.nslots = pl.nslots; r.pair = pl.pair;
    r.dscale_slots = pl.nslots * pl.cluster;
    r.out_f32 = a->partial_out;
    r.dbias = a->dbias;
    r.dscale = a->dscale;
    r.logit_scale = a->logit_scale;
    e = launch_reduce_partials(r, is_bf16, stream);
    if (e != cudaSuccess) { g_last_cuda_error = static_cast<int>(e); return FWA2_ERR_LAUNCH; }
  }
  return FWA2_OK;
}

extern "C" int fwa2_finalize_grads(const float* partial, int32_t dtype, int32_t heads, int32_t n,
                                   const void* logit_scale, void* dbias, void* dscale, void* stream) {
  if (partial == nullptr) return FWA2_ERR_NULL;
  if (dtype != FWA2_F16 && dtype != FWA2_BF16) return FWA2_ERR_DTYPE;
  if (heads <= 0 || heads > 256 || n <= 0) return FWA2_ERR_SHAPE;
  if (dscale != nullptr && logit_scale == nullptr) return FWA2_ERR_NULL;
  cudaError_t e = launch_finalize(partial, dtype == FWA2_BF16, heads, n, logit_scale, dbias, dscale,
                                  static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { g_last_cuda_error = static_cast<int>(e); return FWA2_ERR_LAUNCH; }
  return FWA2_OK;
}
