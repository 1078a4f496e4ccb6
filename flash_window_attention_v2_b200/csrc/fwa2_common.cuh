// Kernel parameter blocks and launch-time layout decisions shared by the host API and the
// device code.  A "unit" is one (window, head) pair; a "tile" is 128 query rows; a "step" is 64
// key columns of a tile.  Windows of at most 64 tokens are processed two units per tile ("pair
// mode": the tile's rows and its 128 key columns are [unit A | unit B], and each row only ever
// looks at the 64 columns of its own unit).
#pragma once

#include <cuda.h>
#include <cstdint>

#include "fwa2_ptx.cuh"

namespace fwa2 {

constexpr int kHeadDim = 32;          // the only head dimension these kernels are built for
constexpr int kRowBytes = 64;         // one row of a q/k/v/do tile: 32 x 16 bit
constexpr int kBoxRows = 64;          // every TMA box is 64 rows tall
constexpr int kBoxBytes = kBoxRows * kRowBytes;   // 4 KiB
constexpr int kTileRows = 128;
constexpr int kStepCols = 64;
constexpr int kChunkCols = 32;        // bias / mask tables are staged 32 columns at a time
constexpr int kTableTileBytes = kTileRows * kChunkCols * 2;   // 8 KiB per table per chunk
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kLn100 = 4.605170185988092f;

// Optional timeline of CTA 0: each role appends (clock64 << 8 | event) words to its own region.
// Only compiled in with -DFWA2_TRACE=2 (-DFWA2_TRACE=1: only per-CTA times and the cycles spent in
// waits; a development aid: the extra code costs instruction-cache
// space that the kernels cannot spare); otherwise the trace arguments are accepted and ignored.
#ifndef FWA2_TRACE
#define FWA2_TRACE 0
#endif
struct Trace {
  unsigned long long* buf;
  int cap;
};
struct TraceCursor {
  unsigned long long* p;
  int left;
};
__device__ __forceinline__ TraceCursor trace_begin(const Trace& t, int role) {
  TraceCursor c{nullptr, 0};
#if FWA2_TRACE >= 2
  if (t.buf != nullptr && blockIdx.x == 0) {
    c.p = t.buf + static_cast<long long>(role) * t.cap;
    c.left = t.cap;
  }
#endif
  return c;
}
__device__ __forceinline__ void trace_ev(TraceCursor& c, unsigned int id) {
#if FWA2_TRACE >= 2
  if (c.left > 0) {
    *c.p++ = (static_cast<unsigned long long>(clock64()) << 8) | id;
    --c.left;
  }
#endif
}

struct FwdParams {
  CUtensorMap tm_q, tm_k, tm_v;   // 4-D (d, N, H, BW), box (32, 64, 1, 1), 64-byte swizzle
  CUtensorMap tm_bias;            // 3-D (N, N, H),  box (32, 64, 1)
  CUtensorMap tm_mask;            // 3-D (N, N, nW), box (32, 64, 1)
  void* o;
  long long o_sbw, o_sh, o_sn;    // element strides of o
  float* lse;
  long long lse_sbw, lse_sh;
  const void* scale;              // scalar mode: one fp32; tensor mode: H values of the input dtype
  int scale_is_tensor;
  int BW, H, N, nW;
  int has_bias, has_mask;
  int pair_mode;
  int comb;                       // tm_bias describes the fp32 table bias + mask, (N, N, nW * H), box
                                  // (32, 128, 1), 128-byte swizzle, and the units are walked table by
                                  // table: job = (window type * H + head) * n_img + image
  int n_img;                      // BW / nW
  int n_jobs;                     // units, or pairs of units in pair mode
  int n_kv_stages;                // 1 or 2
  int n_bm_stages;
  uint32_t off_kv, kv_stage_bytes;   // stage = [K rows | V rows]
  uint32_t off_q;                    // 2 stages of 8 KiB
  uint32_t off_bm;                   // stage = [bias tile 8 KiB | mask tile 8 KiB]
  uint32_t off_p;                    // P tile in shared memory (only when P is not kept in TMEM)
  uint32_t off_ctrl;                 // mbarriers, TMEM base slot, abort flag (512 bytes)
  uint32_t smem_bytes;
  DeviceStatus* status;
  Trace trace;
};

#ifndef FWA2_NORMALISE_ROLLED
#define FWA2_NORMALISE_ROLLED 1
#endif
#if FWA2_NORMALISE_ROLLED
// Normalise one 32-element row of a 64-byte-swizzled tile in place; returns 1 / max(|x|, 1e-12).
// Two rolled passes over the four 16-byte pieces of the row (small code matters more than the
// second read of 64 bytes of shared memory).
template <typename T>
__device__ __forceinline__ float normalise_row(uint32_t tile_base, uint32_t row) {
  const uint32_t row_base = tile_base + row * 64u, sw = (row >> 1) & 3u;
  float ss = 0.f;
#pragma unroll 1
  for (uint32_t ch = 0; ch < 4u; ++ch) {
    uint32_t w[4];
    lds128(row_base + ((ch ^ sw) << 4), w);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = Elem<T>::lo(w[i]), b = Elem<T>::hi(w[i]);
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
  }
  const float rn = rsqrtf(fmaxf(ss, 1e-24f));
#pragma unroll 1
  for (uint32_t ch = 0; ch < 4u; ++ch) {
    uint32_t w[4];
    lds128(row_base + ((ch ^ sw) << 4), w);
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = Elem<T>::pack(Elem<T>::lo(w[i]) * rn, Elem<T>::hi(w[i]) * rn);
    sts128(row_base + ((ch ^ sw) << 4), w);
  }
  return rn;
}

#else
// Normalise one 32-element row of a 64-byte-swizzled tile in place; returns 1 / max(|x|, 1e-12).
template <typename T>
__device__ __forceinline__ float normalise_row(uint32_t tile_base, uint32_t row) {
  uint32_t w[4][4];
  float ss = 0.f;
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    lds128(tile_base + sw64_offset(row, ch), w[ch]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = Elem<T>::lo(w[ch][i]), b = Elem<T>::hi(w[ch][i]);
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
  }
  const float rn = rsqrtf(fmaxf(ss, 1e-24f));
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[ch][i] = Elem<T>::pack(Elem<T>::lo(w[ch][i]) * rn, Elem<T>::hi(w[ch][i]) * rn);
    sts128(tile_base + sw64_offset(row, ch), w[ch]);
  }
  return rn;
}

#endif
// Multiplier of the cosine scores: exp(min(g_h, ln 100)) in tensor mode, the given fp32 constant
// in scalar mode.
template <typename T>
__device__ __forceinline__ float load_scale(const void* scale, int is_tensor, int h) {
  if (!is_tensor) return *static_cast<const float*>(scale);
  const float g = Elem<T>::from_raw(static_cast<const uint16_t*>(scale)[h]);
  return __expf(fminf(g, kLn100));
}

// Backward.  CTA c works on head (c mod H) only, on the windows slot, slot + nslots, ... with
// slot = c / H, so that its window-summed dBias partial has a single writer per address.
struct BwdParams {
  CUtensorMap tm_q, tm_k, tm_v, tm_do;   // 4-D (d, N, H, BW), box (32, 64, 1, 1)
  CUtensorMap tm_biasT, tm_maskT;        // 3-D transposed tables (N_pad, N, planes), box (32, 64, 1)
  const void* q;  long long q_sbw, q_sh, q_sn;
  const void* k;  long long k_sbw, k_sh, k_sn;
  const void* o;  long long o_sbw, o_sh, o_sn;
  void* dq;       long long dq_sbw, dq_sh, dq_sn;
  void* dk;       long long dk_sbw, dk_sh, dk_sn;
  void* dv;       long long dv_sbw, dv_sh, dv_sn;
  const float* lse;
  long long lse_sbw, lse_sh;
  const void* scale;
  int scale_is_tensor;
  float* db_partial;          // [n_bufs][db_pitch][db_pitch] fp32: (query, key)
  long long db_buf_stride;    // db_pitch * db_pitch
  int db_pitch;               // N rounded up to 32
  float* dscale_partial;      // [grid]
  int BW, H, N, nW;
  int has_bias, has_mask;
  int pair_mode;
  int nslots;                 // grid = nslots * H
  int n_kv_stages, n_ds_bufs, n_bm_stages;
  int rows_kv;                // K/V rows held per stage (N rounded up to 128; 128 in pair mode)
  uint32_t off_kv, kv_stage_bytes;   // stage = [K rows | V rows]
  uint32_t off_qdo;                  // 2 stages of [Q tile 8 KiB | dO tile 8 KiB]
  uint32_t off_ds;                   // n_ds_bufs tiles of 32 KiB (two 64-query slabs)
  uint32_t off_bm;                   // [warpgroup][stage] of [bias^T 8 KiB | mask^T 8 KiB]
  uint32_t off_ident;                // two 32 x 32 identity tiles (16 bit, MN-major rows of 64 bytes, swizzled)
  uint32_t off_rk;                   // n_kv_stages x rows_kv floats: 1 / |k|
  uint32_t off_rowstats;             // 2 stages x (128 lse*log2e, 128 delta) floats
  uint32_t off_ctrl;
  uint32_t smem_bytes;
  DeviceStatus* status;
  Trace trace;
};

// Backward for windows of 65 to 256 tokens ("quad" kernel).  The N x N score matrix of a unit is
// cut into 128 x 128 tiles (key block a, query tile b); a cluster of `cluster` CTAs (4, or 1 for
// windows of at most 128 tokens) works on one unit at a time, CTA rank 2 a + b on tile (a, b).
// Cluster c works on head (c mod H) only, on the windows slot, slot + nslots, ... (slot = c / H),
// so each CTA keeps its tile of the window-summed dBias in tensor memory for the whole kernel.
struct QuadParams {
  CUtensorMap tm_q, tm_k, tm_v, tm_do;   // 4-D (d, N, H, BW), box (32, 64, 1, 1)
  CUtensorMap tm_maskT;                  // 3-D transposed mask (N_pad, N, nW), box (32, 64, 1)
  const void* bias_t;                    // transposed bias (H, key, table_pitch queries), 16 bit
  int table_pitch;
  const void* q;  long long q_sbw, q_sh, q_sn;
  const void* k;  long long k_sbw, k_sh, k_sn;
  const void* o;  long long o_sbw, o_sh, o_sn;
  void* dq;       long long dq_sbw, dq_sh, dq_sn;
  void* dk;       long long dk_sbw, dk_sh, dk_sn;
  void* dv;       long long dv_sbw, dv_sh, dv_sn;
  const float* lse;
  long long lse_sbw, lse_sh;
  const void* scale;
  int scale_is_tensor;
  float* db_partial;          // [clusters][db_pitch][db_pitch] fp32: (query, key); nullptr = no dBias
  long long db_buf_stride;
  int db_pitch;
  float* dscale_partial;      // [(slot * cluster + rank) * H + h]
  int BW, H, N, nW;
  int has_bias, has_mask;
  int cluster;                // CTAs per cluster: 1 or 4
  int nslots;                 // clusters = nslots * H
  int n_stages, n_mask_stages;
  uint32_t off_stage;         // n_stages x [K | V | Q | dO], 8 KiB each
  uint32_t off_mask;          // n_mask_stages x four chunks of (128 keys x 32 queries) mask^T
  uint32_t off_ds;            // dS tile, 32 KiB (two slabs of 64 queries)
  uint32_t off_recv;          // three partial accumulators of 64 rows x 32 fp32 pushed by peers
  uint32_t off_ident;         // two 32 x 32 identity tiles
  uint32_t off_rowstats;      // n_stages x (128 x -lse*log2e, 128 x -delta) floats
  uint32_t off_ctrl;
  uint32_t smem_bytes;
  DeviceStatus* status;
  unsigned long long* prof;   // development builds (-DFWA2_TRACE=1): cycles waited per site, CTA 0
};

// Second stage of the dBias / dLogitScale reduction.
struct ReduceParams {
  const float* db_partial;     // [n_bufs][pitch][pitch] (query, key)
  long long buf_stride;
  int pitch;
  const float* dscale_partial; // [grid]
  int H, N, BW, nslots, pair;
  int dscale_slots;            // dLogitScale partials per head (laid out [slot][H])
  float* out_f32;              // (H*N*N + H) or nullptr
  void* dbias;                 // (H, N, N) output dtype or nullptr
  void* dscale;                // H values or nullptr
  const void* logit_scale;     // for the gate (tensor mode) or nullptr
};

}  // namespace fwa2
