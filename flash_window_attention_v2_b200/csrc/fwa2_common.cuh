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
};

}  // namespace fwa2
