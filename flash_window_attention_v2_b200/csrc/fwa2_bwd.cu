// Backward kernel: recomputes the scores and produces dQ, dK, dV (through the L2-normalisation
// Jacobian), per-CTA partial sums of dBias and of dLogitScale, with no contended atomics.
//
// Everything is computed TRANSPOSED: S^T = K^ Q^^T and dP^T = V dO^T put keys on the 128 TMEM
// lanes, so that P^T and dS^T (written back over S^T / dP^T as packed 16-bit pairs) are directly
// the tensor-memory A operands of dV += P^T dO and dK^ += dS^T Q^.  Only dS takes a trip
// through shared memory, as the A operand of dQ^ += dS K^.
//
// One persistent CTA per SM.  A tile is 128 keys x 128 queries; its two 64-query halves
// ("steps") are processed concurrently by two warpgroups.  Roles:
//   warps 0-3   compute warpgroup 0: thread t owns key t of the tile, queries [0, 64)
//   warps 4-7   compute warpgroup 1: same keys, queries [64, 128)
//   warps 12-15 preparing warpgroup: normalises K and Q, computes delta, one tile ahead
//   warp  8     issues every tcgen05.mma (one thread)
//   warp  9     TMA producer of K/V and Q/dO (one thread)
//   warps 10-11 TMA producers of the bias / mask tables of warpgroup 0 / 1 (one thread each)
// Replaces flash_win_attn_v2/kernels/attn_kernel_backward.py:6-51 (delta pre-pass) and
// :84-564 (`_bwd_kernel`).
#ifndef FWA2_BWD_NORMALISE_ROLLED
#define FWA2_BWD_NORMALISE_ROLLED 1
#endif
#ifndef FWA2_BWD_WAIT_INLINE
#define FWA2_BWD_WAIT_INLINE 1   // register reallocation (setmaxnreg) does not go with calls
#endif
#define FWA2_NORMALISE_ROLLED FWA2_BWD_NORMALISE_ROLLED
#define FWA2_WAIT_INLINE FWA2_BWD_WAIT_INLINE
#include "fwa2_common.cuh"

namespace fwa2 {

constexpr int kBwdThreads = 512;
constexpr uint32_t kBwdTmemCols = 512;
constexpr uint32_t kTmST = 0;       // S^T of warpgroup w at 128 w (64 columns), P^T written over it
constexpr uint32_t kTmDPT = 64;     // dP^T of warpgroup w at 128 w + 64, dS^T written over it
// Accumulators.  Windows of at most 256 tokens (two query tiles) get TWO sets, so that the
// epilogue of one key block / job can run one tile late while the tensor core already fills the
// other set; larger windows have room for one set only.
//   two sets:  dV[s] 256 + 64 s, dK[s] 288 + 64 s, dQ[s][i] 384 + 64 s + 32 i   (i < 2)
//   one set:   dV 256, dK 288, dQ[i] 320 + 32 i                                  (i < 5)
__device__ __forceinline__ uint32_t tm_dv(uint32_t set) { return 256u + 64u * set; }
__device__ __forceinline__ uint32_t tm_dk(uint32_t set) { return 288u + 64u * set; }
__device__ __forceinline__ uint32_t tm_dq(uint32_t nsets, uint32_t set, uint32_t i) {
  return (nsets == 2u ? 384u + 64u * set : 320u) + 32u * i;
}
// Pair mode keeps the window-summed dBias^T of the CTA's head in tensor memory for the whole
// kernel: lanes = keys of unit A | unit B, 32 query columns per chunk, in the columns that the
// second dQ accumulator of a set would use (windows of at most 64 tokens have one query tile).
__device__ __forceinline__ uint32_t tm_db(uint32_t chunk) { return 416u + 64u * chunk; }
constexpr uint32_t kQdoStageBytes = 4u * kBoxBytes;   // [Q tile | dO tile]
constexpr uint32_t kDsTileBytes = 32768u;
constexpr int kNumQdoStages = 3;

enum BwdBar : int {
  kbKvFull = 0, kbKvReady = 4, kbKvFree = 8,          // up to four K/V stages
  kbQdoFull = 12, kbQdoReady = 15, kbQdoFree = 18,
  kbStFull = 21, kbPtFull = 25,       // index + 2 * warpgroup + chunk
  kbBmFull = 29, kbBmFree = 33,       // index + 2 * warpgroup + stage
  kbDsFree = 37,
  kbDkvFull = 39, kbDkvFree = 41, kbDqFull = 43, kbDqFree = 45,   // one per accumulator set
  kBwdNumBars = 47
};

// Epilogues may run one tile late (two accumulator sets) when the window has at most two query
// tiles and the K/V stage a late epilogue still reads cannot be the one the next-but-one job
// needs: jobs of a single tile need three stages for that, longer jobs two.
__device__ __forceinline__ uint32_t bwd_num_sets(const BwdParams& p, int kb, int mt) {
  if (mt > 2) return 1u;
  if (kb * mt >= 2) return p.n_kv_stages >= 2 ? 2u : 1u;
  return p.n_kv_stages >= 3 ? 2u : 1u;
}

struct BwdGeom {
  int N, H, pair, KB, MT, h, slot, nslots, count, njobs;
};

// kPair is a template parameter of the kernel: each launch runs code specialised for its mode, so
// the instruction cache holds none of the other mode's branches between the hot instructions.
template <bool kPair>
__device__ __forceinline__ BwdGeom bwd_geom(const BwdParams& p) {
  BwdGeom g;
  g.N = p.N;
  g.H = p.H;
  g.pair = kPair ? 1 : 0;
  g.KB = g.pair ? 1 : (p.N + kTileRows - 1) / kTileRows;
  g.MT = g.KB;
  g.h = static_cast<int>(blockIdx.x) % p.H;
  g.slot = static_cast<int>(blockIdx.x) / p.H;
  g.nslots = p.nslots;
  g.count = g.slot < p.BW ? (p.BW - g.slot + g.nslots - 1) / g.nslots : 0;
  g.njobs = g.pair ? (g.count + 1) / 2 : g.count;
  return g;
}

// Window (row of BW) of member m of job t; BW (out of range: TMA then delivers zeros) if absent.
__device__ __forceinline__ int bwd_bw(const BwdParams& p, const BwdGeom& g, int t, int m) {
  const int idx = g.pair ? 2 * t + m : t;
  return idx < g.count ? g.slot + idx * g.nslots : p.BW;
}

struct TileIt {
  int t, j, i;   // job, key block, query tile
};
__device__ __forceinline__ bool tile_next(const BwdGeom& g, TileIt& it) {
  if (++it.i >= g.MT) {
    it.i = 0;
    if (++it.j >= g.KB) {
      it.j = 0;
      ++it.t;
    }
  }
  return it.t < g.njobs;
}
// Queries of step w of query tile i that exist (<= 0: the step is skipped by every role).
__device__ __forceinline__ int step_rows(const BwdGeom& g, int i, int w) {
  return g.pair ? kStepCols : g.N - kTileRows * i - kStepCols * w;
}

// Pair mode interleaves the queries of the two units in shared memory (and so in the columns of
// S^T / dP^T and the lanes of dQ): row r holds query 32 (r / 64) + r % 32 of unit (r / 32) % 2, so
// that the 64 rows of step w -- the share of warpgroup w -- are the queries [32 w, 32 w + 32) of
// unit A followed by the same queries of unit B.  Each warpgroup then depends only on its own
// step, as it does for larger windows.
__device__ __forceinline__ int pair_row_unit(uint32_t r) { return static_cast<int>((r >> 5) & 1u); }
__device__ __forceinline__ int pair_row_query(uint32_t r) { return static_cast<int>(32u * (r >> 6) + (r & 31u)); }

__device__ __forceinline__ void red_add(float* addr, float a) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ uint4 ldg_nc_v4(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

// ------------------------------------------------------------------------------------------------
// Eight queries of a chunk for one key (= one thread):
//   p = exp2(x log2e - lse2),  ds = p (dP - delta),  x = scale * cos + bias + mask.
// Produces the packed P^T / dS^T words and adds ds into this CTA's dBias^T partial.  Queries past
// the end of the window need no special case: their Q and dO rows were zero-filled by the TMA
// load and their lse2 is +inf, so p = 0 and ds = 0 exactly.
//
// The per-element work is written for eight queries and run in a rolled loop (not unrolled over
// the 32 queries of a chunk): these kernels are bound by instruction fetch, and the loop body has
// to stay resident in the instruction cache next to the other roles' code.
// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void bwd_group(bool has_bias, bool has_mask, const uint32_t (&sv)[8],
                                          const uint32_t (&dpv)[8], uint32_t bias_addr,
                                          uint32_t mask_addr, const float* lse2, const float* delta,
                                          float scale, bool key_ok, float* db_ptr, int db_pitch,
                                          bool db_store, uint32_t (&pw)[4], uint32_t (&dw)[4]) {
  uint32_t wb[4] = {0u, 0u, 0u, 0u}, wm[4] = {0u, 0u, 0u, 0u};
  if (has_bias) lds128(bias_addr, wb);
  if (has_mask) lds128(mask_addr, wm);
  const float4 la = *reinterpret_cast<const float4*>(lse2);
  const float4 lb = *reinterpret_cast<const float4*>(lse2 + 4);
  const float4 da = *reinterpret_cast<const float4*>(delta);
  const float4 db = *reinterpret_cast<const float4*>(delta + 4);
  const float l8[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
  const float d8[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
  float dsv[8];
#pragma unroll
  for (int e2 = 0; e2 < 4; ++e2) {
    const int e = 2 * e2;
    const float x0 = fmaf(__uint_as_float(sv[e]), scale, Elem<T>::lo(wb[e2])) + Elem<T>::lo(wm[e2]);
    const float x1 = fmaf(__uint_as_float(sv[e + 1]), scale, Elem<T>::hi(wb[e2])) + Elem<T>::hi(wm[e2]);
    const float p0 = ex2f(fmaf(x0, kLog2e, -l8[e]));
    const float p1 = ex2f(fmaf(x1, kLog2e, -l8[e + 1]));
    const float s0 = p0 * (__uint_as_float(dpv[e]) - d8[e]);
    const float s1 = p1 * (__uint_as_float(dpv[e + 1]) - d8[e + 1]);
    pw[e2] = key_ok ? Elem<T>::pack(p0, p1) : 0u;
    dw[e2] = key_ok ? Elem<T>::pack(s0, s1) : 0u;
    dsv[e] = s0;
    dsv[e + 1] = s1;
  }
  // The partial is laid out (query, key): the 32 keys of a warp are 128 contiguous bytes of one
  // query row, so every store / reduction below is one fully used line (a (key, query) layout
  // with 16-byte vectors per thread touched 32 lines per instruction).
  if (db_ptr != nullptr) {
    if (db_store) {
#pragma unroll
      for (int e = 0; e < 8; ++e) db_ptr[e * db_pitch] = dsv[e];
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) red_add(db_ptr + e * db_pitch, dsv[e]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// The two compute warpgroups
// ------------------------------------------------------------------------------------------------
template <typename T, bool kPair>
__device__ void bwd_compute_role(const BwdParams& p, uint8_t* smem_ptr, uint32_t smem_base,
                                 uint32_t bars, uint32_t tmem, const WaitCtx& ctx,
                                 float& dscale_acc) {
  const BwdGeom g = bwd_geom<kPair>(p);
  if (g.njobs == 0) return;
  const uint32_t tid = threadIdx.x;
  const uint32_t wg = tid >> 7, lt = tid & 127u;
  const uint32_t lane_base = ((lt >> 5) * 32u) << 16;
  const float scale = load_scale<T>(p.scale, p.scale_is_tensor, g.h);
  const bool any_table = p.has_bias || p.has_mask;
  auto bar = [&](int i) { return bars + 8u * i; };
  float* rk_arr = reinterpret_cast<float*>(smem_ptr + p.off_rk);
  float* rowstats = reinterpret_cast<float*>(smem_ptr + p.off_rowstats);
  const uint32_t NKV = p.n_kv_stages, NDS = p.n_ds_bufs, NBM = p.n_bm_stages;

  // Warpgroup 0 writes dV, warpgroup 1 writes dK.  dQ: warpgroup (i mod 2) writes query tile i, so
  // for jobs of a single tile (windows of at most 128 tokens) warpgroup 0 alone (its barrier is
  // initialised with the matching arrival count).
  const bool single_tile = (g.KB * g.MT == 1);
  const uint32_t nsets = bwd_num_sets(p, g.KB, g.MT);
  const uint32_t sets_mask = nsets - 1u, sets_shift = nsets - 1u;
  uint32_t jt = 0, kdkv = 0, kdq = 0;
  uint32_t nst = 0u;   // phase bit per 32-query chunk of my step
  Ring kv_ring(NKV), qdo_ring(kNumQdoStages), ds_ring(NDS), bm_ring(NBM);
  TraceCursor tr = (lt == 0) ? trace_begin(p.trace, wg == 0 ? 0 : 3) : TraceCursor{nullptr, 0};
  // ---- dK, dV of one key block (thread = key): warpgroup 0 writes dV, warpgroup 1 writes dK ----
  auto dkv_epilogue = [&](const TileIt& it, uint32_t kvs_e, uint32_t kd) -> bool {
    // dK, dV of key block it.j are complete
    const uint32_t set = kd & sets_mask, use = kd >> sets_shift;
    if (!mbar_wait(bar(kbDkvFull + set), use & 1u, ctx, 55)) return false;
    tc_fence_after();
    trace_ev(tr, 10);
    const int m = g.pair ? static_cast<int>(lt >> 6) : 0;
    const int bw = bwd_bw(p, g, it.t, m);
    const int jg = g.pair ? static_cast<int>(lt & 63u) : it.j * kTileRows + static_cast<int>(lt);
    const bool ok = bw < p.BW && jg < g.N;
    // (rolled loops over groups of eight columns: see bwd_group about code size)
    if (wg == 0) {
      uint16_t* dst = static_cast<uint16_t*>(p.dv) + bw * p.dv_sbw + g.h * p.dv_sh + jg * p.dv_sn;
      const uint32_t t_dv = tmem + lane_base + tm_dv(set);
#pragma unroll 1
      for (uint32_t gq = 0; gq < 4u; ++gq) {
        uint32_t r[8];
        tmem_ld8(t_dv + 8u * gq, r);
        tmem_wait_ld();
        if (ok) {
          uint4 v;
          v.x = Elem<T>::pack(__uint_as_float(r[0]), __uint_as_float(r[1]));
          v.y = Elem<T>::pack(__uint_as_float(r[2]), __uint_as_float(r[3]));
          v.z = Elem<T>::pack(__uint_as_float(r[4]), __uint_as_float(r[5]));
          v.w = Elem<T>::pack(__uint_as_float(r[6]), __uint_as_float(r[7]));
          *reinterpret_cast<uint4*>(dst + 8u * gq) = v;
        }
      }
      tc_fence_before();
      mbar_arrive(bar(kbDkvFree + set));
    }
    if (wg == 1) {
      // dk = scale * (dK' - k^ (k^ . dK')) / |k|: one pass for the dot product, one for the output
      const uint32_t krow = g.pair ? lt : static_cast<uint32_t>(it.j) * kTileRows + lt;
      const uint32_t k_row = smem_base + p.off_kv + kvs_e * p.kv_stage_bytes + krow * 64u;
      const uint32_t k_sw = (krow >> 1) & 3u;
      const uint32_t t_dk = tmem + lane_base + tm_dk(set);
      float dot = 0.f;
#pragma unroll 1
      for (uint32_t gq = 0; gq < 4u; ++gq) {
        uint32_t r[8], w[4];
        tmem_ld8(t_dk + 8u * gq, r);
        lds128(k_row + ((gq ^ k_sw) << 4), w);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          dot = fmaf(Elem<T>::lo(w[i]), __uint_as_float(r[2 * i]), dot);
          dot = fmaf(Elem<T>::hi(w[i]), __uint_as_float(r[2 * i + 1]), dot);
        }
      }
      const float f = scale * rk_arr[kvs_e * p.rows_kv + krow];
      uint16_t* dst = static_cast<uint16_t*>(p.dk) + bw * p.dk_sbw + g.h * p.dk_sh + jg * p.dk_sn;
#pragma unroll 1
      for (uint32_t gq = 0; gq < 4u; ++gq) {
        uint32_t r[8], w[4];
        tmem_ld8(t_dk + 8u * gq, r);
        lds128(k_row + ((gq ^ k_sw) << 4), w);
        tmem_wait_ld();
        if (ok) {
          float o8[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            o8[2 * i] = f * (__uint_as_float(r[2 * i]) - Elem<T>::lo(w[i]) * dot);
            o8[2 * i + 1] = f * (__uint_as_float(r[2 * i + 1]) - Elem<T>::hi(w[i]) * dot);
          }
          uint4 v;
          v.x = Elem<T>::pack(o8[0], o8[1]);
          v.y = Elem<T>::pack(o8[2], o8[3]);
          v.z = Elem<T>::pack(o8[4], o8[5]);
          v.w = Elem<T>::pack(o8[6], o8[7]);
          *reinterpret_cast<uint4*>(dst + 8u * gq) = v;
        }
      }
      tc_fence_before();
      mbar_arrive(bar(kbDkvFree + set));
    }
    if (it.j == g.KB - 1) mbar_arrive(bar(kbKvFree + kvs_e));   // K^ in shared memory no longer needed
    trace_ev(tr, 11);
    return true;
  };
  // ---- dQ of a job (thread = query): warpgroup (i mod 2) writes query tile i ----
  // dq = scale * (dQ' - q^ (q^ . dQ')) / |q| from the raw q row: with q^ = q / |q| the dot product
  // is (q . dQ') / |q|, so one pass gives |q| and the dot product, a second the output.  The raw
  // row is fetched with four loads in flight before anything is waited for; every lane runs both
  // passes (the tensor-memory loads are warp-wide), only the global accesses are predicated.
  auto dq_epilogue = [&](int t_e, uint32_t kq) -> bool {
    if (single_tile && wg == 1) return true;
    const int mq = g.pair ? pair_row_unit(lt) : 0;
    const int bwq = bwd_bw(p, g, t_e, mq);
    uint4 qraw[4];
    auto load_q = [&](int i) -> bool {
      const int ig = g.pair ? pair_row_query(lt) : i * kTileRows + static_cast<int>(lt);
      const bool okq = bwq < p.BW && ig < g.N;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) qraw[ch] = make_uint4(0u, 0u, 0u, 0u);
      if (okq) {
        const uint16_t* qrow = static_cast<const uint16_t*>(p.q) + bwq * p.q_sbw + g.h * p.q_sh + ig * p.q_sn;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) qraw[ch] = ldg_nc_v4(qrow + ch * 8);
      }
      return okq;
    };
    bool okq = load_q(static_cast<int>(wg));
    // dQ of every query tile of the job is complete
    const uint32_t set = kq & sets_mask, use = kq >> sets_shift;
    if (!mbar_wait(bar(kbDqFull + set), use & 1u, ctx, 56)) return false;
    tc_fence_after();
    trace_ev(tr, 12);
#pragma unroll 1
    for (int i = static_cast<int>(wg); i < g.MT; i += 2) {
      const int ig = g.pair ? pair_row_query(lt) : i * kTileRows + static_cast<int>(lt);
      const uint32_t t_dq = tmem + lane_base + tm_dq(nsets, set, static_cast<uint32_t>(i));
      float ss = 0.f, qd = 0.f;
#pragma unroll
      for (int gq = 0; gq < 4; ++gq) {
        uint32_t r[8];
        tmem_ld8(t_dq + 8u * gq, r);
        tmem_wait_ld();
        const uint32_t w[4] = {qraw[gq].x, qraw[gq].y, qraw[gq].z, qraw[gq].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float a = Elem<T>::lo(w[e]), b = Elem<T>::hi(w[e]);
          ss = fmaf(a, a, ss);
          ss = fmaf(b, b, ss);
          qd = fmaf(a, __uint_as_float(r[2 * e]), qd);
          qd = fmaf(b, __uint_as_float(r[2 * e + 1]), qd);
        }
      }
      const float rn = rsqrtf(fmaxf(ss, 1e-24f));
      const float dot = qd * rn;
      if (okq) dscale_acc += dot;
      const float f = scale * rn, cq = rn * dot;
      uint16_t* dst = static_cast<uint16_t*>(p.dq) + bwq * p.dq_sbw + g.h * p.dq_sh + ig * p.dq_sn;
#pragma unroll
      for (int gq = 0; gq < 4; ++gq) {
        uint32_t r[8];
        tmem_ld8(t_dq + 8u * gq, r);
        tmem_wait_ld();
        const uint32_t w[4] = {qraw[gq].x, qraw[gq].y, qraw[gq].z, qraw[gq].w};
        float o8[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o8[2 * e] = f * (__uint_as_float(r[2 * e]) - Elem<T>::lo(w[e]) * cq);
          o8[2 * e + 1] = f * (__uint_as_float(r[2 * e + 1]) - Elem<T>::hi(w[e]) * cq);
        }
        uint4 o;
        o.x = Elem<T>::pack(o8[0], o8[1]);
        o.y = Elem<T>::pack(o8[2], o8[3]);
        o.z = Elem<T>::pack(o8[4], o8[5]);
        o.w = Elem<T>::pack(o8[6], o8[7]);
        if (okq) *reinterpret_cast<uint4*>(dst + 8 * gq) = o;
      }
      if (i + 2 < g.MT) okq = load_q(i + 2);
    }
    tc_fence_before();
    mbar_arrive(bar(kbDqFree + set));
    trace_ev(tr, 13);
    return true;
  };
  bool pend_dkv = false, pend_dq = false;
  TileIt pd_it{0, 0, 0};
  uint32_t pd_kvs = 0, pd_k = 0, pq_k = 0;
  int pq_t = 0;

  if (g.pair && p.db_partial != nullptr) {
    // the dBias^T sums in tensor memory start from zero (warpgroup w owns the columns of step w;
    // the first product that adds to them is issued after this warpgroup's first P^T barrier)
    uint32_t z[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) z[i] = 0u;
    tmem_st16(tmem + lane_base + tm_db(wg), z);
    tmem_st16(tmem + lane_base + tm_db(wg) + 16u, z);
    tmem_wait_st();
    tc_fence_before();
  }
  TileIt cur{0, 0, 0};
  while (true) {
    TileIt nxt = cur;
    const bool has_next = tile_next(g, nxt);
    trace_ev(tr, 1);
    Ring kv_next = kv_ring, qdo_next = qdo_ring;
    kv_next.advance();
    qdo_next.advance();
    // what the preparing warpgroup wrote for this tile and job (row statistics, 1 / |k|) is
    // visible once its barrier for the tile has been seen (it completed long ago; the job's K was
    // normalised by the same threads before they arrived here)
    if (!mbar_wait(bar(kbQdoReady + qdo_ring.stage), qdo_ring.phase, ctx, 51)) return;
    trace_ev(tr, 2);
    // ------------------------------ my share of the current tile ------------------------------
    // Warpgroup w takes step w (64 queries) of the tile.  Windows of more than 64 tokens: in two
    // chunks of 32 queries.  Pair mode: the step holds 32 queries of unit A and 32 of unit B, and
    // only the diagonal blocks (keys and queries of the same unit) carry work, so a thread takes
    // the one chunk of its key's unit and fills its part of the other chunk with zeros.
    const uint32_t um = lt >> 6;                       // pair mode: unit of my key
    const uint32_t step = wg;
    const int nr = step_rows(g, cur.i, static_cast<int>(step));
    const uint32_t kvs = kv_ring.stage;
    if (nr > 0) {
      bool key_ok;
      int jg;
      if (g.pair) {
        key_ok = bwd_bw(p, g, cur.t, static_cast<int>(um)) < p.BW && static_cast<int>(lt & 63u) < g.N;
        jg = static_cast<int>(lt & 63u);
      } else {
        jg = cur.j * kTileRows + static_cast<int>(lt);
        key_ok = jg < g.N;
      }
      const uint32_t dsb = ds_ring.stage;
      if (!mbar_wait(bar(kbDsFree + dsb), ds_ring.phase ^ 1u, ctx, 53)) return;
      trace_ev(tr, 4);
      const uint32_t ds_tile = smem_base + p.off_ds + dsb * kDsTileBytes;
      const uint32_t ds_slab = ds_tile + step * 16384u;
      const uint32_t qs = qdo_ring.stage;
      const float* lse2 = rowstats + qs * 256u + step * 64u;
      const float* delta = rowstats + qs * 256u + 128u + step * 64u;
      const long long db_buf = g.pair ? 2ll * blockIdx.x + um : static_cast<long long>(blockIdx.x);
      const int ig0 = g.pair ? 0 : cur.i * kTileRows + static_cast<int>(wg) * kStepCols;
      float* db_row = (p.db_partial != nullptr && key_ok && !g.pair)   // pair mode: summed by the tensor core
                          ? p.db_partial + db_buf * p.db_buf_stride + static_cast<long long>(ig0) * p.db_pitch + jg
                          : nullptr;
      const bool db_store = (jt == 0);
      const uint32_t tm_st = tmem + lane_base + step * 128u + kTmST;
      const uint32_t tm_dpt = tmem + lane_base + step * 128u + kTmDPT;
      const int c_first = g.pair ? static_cast<int>(um) : 0, c_last = g.pair ? static_cast<int>(um) : 1;

#pragma unroll 1
      for (int c = c_first; c <= c_last; ++c) {
        const int rows_left = nr - kChunkCols * c;
        if (rows_left > 0) {
          // scores of this chunk (the tensor core is meanwhile working on the other chunks)
          // (pair mode: one barrier per step, both chunks are produced and consumed together)
          const int bc = g.pair ? 0 : c;
          if (!mbar_wait(bar(kbStFull + 2 * step + bc), (nst >> bc) & 1u, ctx, 52)) return;
          tc_fence_after();
          trace_ev(tr, 3);
          if (g.pair) {
            // the other unit's queries must not see my key: zeros in the other chunk of the step
            // (issued now, so that the stores drain while my chunk is being computed)
            const uint32_t oc = static_cast<uint32_t>(c) ^ 1u;
            uint32_t z[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) z[i] = 0u;
            tmem_st16(tm_st + 32u * oc, z);
            tmem_st16(tm_dpt + 32u * oc, z);
            const uint32_t z4[4] = {0u, 0u, 0u, 0u};
#pragma unroll
            for (int qd = 0; qd < 4; ++qd)
              sts128(ds_slab + sw128_offset(lt, 4u * oc + qd), z4);
          }
          uint32_t bias_tile = 0, mask_tile = 0;
          const uint32_t st = bm_ring.stage;
          if (any_table) {
            bias_tile = smem_base + p.off_bm + (wg * NBM + st) * (2u * kTableTileBytes);
            mask_tile = bias_tile + kTableTileBytes;
            if (!mbar_wait(bar(kbBmFull + 2 * wg + st), bm_ring.phase, ctx, 54)) return;
          }
          trace_ev(tr, 6);
          // pair mode: one bias box serves both units (same head), the mask has a box per unit
          const uint32_t bias_row = g.pair ? (lt & 63u) : lt;
          const uint32_t bias_base = bias_tile + bias_row * 64u, bias_sw = (bias_row >> 1) & 3u;
          const uint32_t mask_base = mask_tile + lt * 64u, mask_sw = (lt >> 1) & 3u;
          const uint32_t ds_base = ds_slab + lt * 128u, ds_sw = lt & 7u;
          const uint32_t t_s = tm_st + 32u * c, t_d = tm_dpt + 32u * c;
          const float* lse2_c = lse2 + 32 * c;
          const float* delta_c = delta + 32 * c;
          float* dbp = db_row != nullptr ? db_row + kChunkCols * c * p.db_pitch : nullptr;
          // four groups of eight queries; the scores of the next group are fetched from tensor
          // memory while the current one is computed (one copy of the group's code: the register
          // moves that rotate the buffers are cheaper than a second copy in the instruction cache)
          uint32_t sa[8], da[8], sb[8], db8[8];
          tmem_ld8(t_s, sa);
          tmem_ld8(t_d, da);
          tmem_wait_ld();
#pragma unroll 1
          for (uint32_t gq = 0; gq < 4u; ++gq) {
            uint32_t pw[4], dw[4];
            if (gq + 1u < 4u) {
              tmem_ld8(t_s + 8u * (gq + 1u), sb);
              tmem_ld8(t_d + 8u * (gq + 1u), db8);
            }
            bwd_group<T>(p.has_bias, p.has_mask, sa, da, bias_base + ((gq ^ bias_sw) << 4),
                         mask_base + ((gq ^ mask_sw) << 4), lse2_c + 8u * gq, delta_c + 8u * gq, scale,
                         key_ok, dbp != nullptr ? dbp + 8u * gq * p.db_pitch : nullptr, p.db_pitch, db_store, pw, dw);
            // P^T and dS^T go back over the first 16 columns of this chunk's own S^T / dP^T columns
            tmem_st4(t_s + 4u * gq, pw);
            tmem_st4(t_d + 4u * gq, dw);
            sts128(ds_base + (((4u * c + gq) ^ ds_sw) << 4), dw);
            tmem_wait_ld();   // the next group's registers may be read from here on
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              sa[i] = sb[i];
              da[i] = db8[i];
            }
          }
          trace_ev(tr, 7);
          if (any_table) {
            // (behind the wait for the stores of the values computed from the table words: by then
            // the shared-memory loads of every one of them have certainly completed)
            tmem_wait_st();
            mbar_arrive(bar(kbBmFree + 2 * wg + st));
            bm_ring.advance();
          }
        } else {
          continue;   // no query of this chunk exists: nobody issues or reads anything for it
        }
        tmem_wait_st();
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(bar(kbPtFull + 2 * step + (g.pair ? 0 : c)));
        nst ^= 1u << (g.pair ? 0 : c);
        trace_ev(tr, 8);
      }
      trace_ev(tr, 9);
    }

    // ------------------------------ epilogues ------------------------------
    // With two accumulator sets they run one tile late: by then the products they read have
    // long been finished, and the tensor core is not left waiting for this warpgroup either.
    // Pass 0 runs what the previous tile deferred, pass 1 this tile's own epilogues when they
    // cannot be deferred (one accumulator set, or no further tile); one loop, so that the code
    // of the epilogues exists once.
    const bool last_q = cur.i == g.MT - 1, last_k = last_q && cur.j == g.KB - 1;
    const bool defer = nsets == 2u && has_next;
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
      const bool run_dkv = pass == 0 ? pend_dkv : (last_q && !defer);
      const bool run_dq = pass == 0 ? pend_dq : (last_k && !defer);
      if (run_dkv) {
        if (!dkv_epilogue(pass == 0 ? pd_it : cur, pass == 0 ? pd_kvs : kvs, pass == 0 ? pd_k : kdkv)) return;
      }
      if (run_dq) {
        if (!dq_epilogue(pass == 0 ? pq_t : cur.t, pass == 0 ? pq_k : kdq)) return;
      }
    }
    pend_dkv = last_q && defer;
    pend_dq = last_k && defer;
    if (pend_dkv) { pd_it = cur; pd_kvs = kvs; pd_k = kdkv; }
    if (pend_dq) { pq_t = cur.t; pq_k = kdq; }
    if (last_q) ++kdkv;
    if (last_k) ++kdq;

    if (!has_next) break;
    if (nxt.t != cur.t) {
      ++jt;
      kv_ring = kv_next;
    }
    qdo_ring = qdo_next;
    ds_ring.advance();
    cur = nxt;
  }

  // Pair mode: the dBias^T sums of this CTA leave tensor memory once, here.  Every product that
  // fed them was issued before the commits the last epilogues waited for.  Warpgroup w writes
  // the queries of chunk w; the buffer of unit slot m holds the keys on lanes [64 m, 64 m + 64).
  if (g.pair && p.db_partial != nullptr) {
    tc_fence_after();
    const int jg = static_cast<int>(lt & 63u);
    float* dst = p.db_partial + (2ll * blockIdx.x + (lt >> 6)) * p.db_buf_stride +
                 static_cast<long long>(kChunkCols * wg) * p.db_pitch + jg;
    const bool row_ok = jg < g.N && static_cast<int>(kChunkCols * wg) < p.db_pitch;
    const uint32_t t_db = tmem + lane_base + tm_db(wg);
#pragma unroll 1
    for (uint32_t gq = 0; gq < 4u; ++gq) {
      uint32_t r[8];
      tmem_ld8(t_db + 8u * gq, r);
      tmem_wait_ld();
      if (row_ok) {
#pragma unroll
        for (int e = 0; e < 8; ++e) dst[(8u * gq + e) * p.db_pitch] = __uint_as_float(r[e]);
      }
    }
    tc_fence_before();
  }
}

// ------------------------------------------------------------------------------------------------
// The preparing warpgroup (thread = row): everything a tile needs before its scores can be
// computed, one tile ahead of the compute warpgroups and off their critical path.
//   per job:   K rows normalised in place, 1 / |k| kept for the dK epilogue
//   per tile:  Q row normalised in place; delta = dO . O and lse * log2(e) of the row
// The O row comes straight from global memory, fetched one tile ahead into registers.
// ------------------------------------------------------------------------------------------------
template <typename T, bool kPair>
__device__ void bwd_prepare_role(const BwdParams& p, uint8_t* smem_ptr, uint32_t smem_base,
                                 uint32_t bars, const WaitCtx& ctx) {
  const BwdGeom g = bwd_geom<kPair>(p);
  if (g.njobs == 0) return;
  const uint32_t lt = threadIdx.x & 127u;
  auto bar = [&](int i) { return bars + 8u * i; };
  float* rk_arr = reinterpret_cast<float*>(smem_ptr + p.off_rk);
  float* rowstats = reinterpret_cast<float*>(smem_ptr + p.off_rowstats);

  TileIt it{0, 0, 0};
  Ring kv(p.n_kv_stages), qdo(kNumQdoStages);
  bool new_job = true;
#pragma unroll 1
  while (true) {
    // the O row and lse of my query: fetched first, used last (the normalisations hide most of the
    // latency; this warpgroup has slack, and one copy of the loads keeps its code small)
    const int m = g.pair ? pair_row_unit(lt) : 0;
    const int bw = bwd_bw(p, g, it.t, m);
    const int ig = g.pair ? pair_row_query(lt) : it.i * kTileRows + static_cast<int>(lt);
    const bool row_ok = bw < p.BW && ig < g.N;
    uint4 o_row[4];
    float lse = 0.f;
    if (row_ok) {
      const uint16_t* orow = static_cast<const uint16_t*>(p.o) + bw * p.o_sbw + g.h * p.o_sh + ig * p.o_sn;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) o_row[ch] = ldg_nc_v4(orow + ch * 8);
      lse = __ldg(p.lse + bw * p.lse_sbw + g.h * p.lse_sh + ig);
    }

    // K rows of a new job, then my Q row: the same normalisation code for both
    const uint32_t qs = qdo.stage;
    const uint32_t q_base = smem_base + p.off_qdo + qs * kQdoStageBytes;
#pragma unroll 1
    for (int what = new_job ? 0 : 1; what < 2; ++what) {
      const uint32_t kvs = kv.stage;
      const uint32_t base = what == 0 ? smem_base + p.off_kv + kvs * p.kv_stage_bytes : q_base;
      const uint32_t rows = what == 0 ? static_cast<uint32_t>(p.rows_kv) : static_cast<uint32_t>(kTileRows);
      if (!mbar_wait<true>(bar(what == 0 ? kbKvFull + kvs : kbQdoFull + qs), what == 0 ? kv.phase : qdo.phase, ctx, 80 + what))
        return;
#pragma unroll 1
      for (uint32_t rr = lt; rr < rows; rr += 128u) {
        const float rn = normalise_row<T>(base, rr);
        if (what == 0) rk_arr[kvs * p.rows_kv + rr] = rn;
      }
      fence_proxy_async_smem();
      if (what == 0) mbar_arrive(bar(kbKvReady + kvs));
    }
    {
      float l2 = INFINITY, dl = 0.f;
      if (row_ok) {
        float dlp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t wd[4];
          lds128(q_base + 2u * kBoxBytes + sw64_offset(lt, ch), wd);
          const uint32_t wo[4] = {o_row[ch].x, o_row[ch].y, o_row[ch].z, o_row[ch].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            dlp[ch] = fmaf(Elem<T>::lo(wd[i]), Elem<T>::lo(wo[i]), dlp[ch]);
            dlp[ch] = fmaf(Elem<T>::hi(wd[i]), Elem<T>::hi(wo[i]), dlp[ch]);
          }
        }
        dl = (dlp[0] + dlp[1]) + (dlp[2] + dlp[3]);
        l2 = (lse == -INFINITY) ? INFINITY : lse * kLog2e;
      }
      rowstats[qs * 256u + lt] = l2;
      rowstats[qs * 256u + 128u + lt] = dl;
      mbar_arrive(bar(kbQdoReady + qs));
    }
    const int t_before = it.t;
    if (!tile_next(g, it)) break;
    new_job = it.t != t_before;
    if (new_job) kv.advance();
    qdo.advance();
  }
}

// ------------------------------------------------------------------------------------------------
// MMA issuer (one thread)
// ------------------------------------------------------------------------------------------------
template <typename T, bool kPair>
__device__ void bwd_mma_role(const BwdParams& p, uint32_t smem_base, uint32_t bars, uint32_t tmem,
                             const WaitCtx& ctx) {
  const BwdGeom g = bwd_geom<kPair>(p);
  if (g.njobs == 0) return;
  constexpr uint32_t fmt = Elem<T>::kFmt;
  auto bar = [&](int i) { return bars + 8u * i; };
  const uint32_t NKV = p.n_kv_stages, NDS = p.n_ds_bufs;
  const uint32_t idesc_acc = make_idesc(fmt, 128, 32, 0, 1);   // A in TMEM, B MN-major
  const uint32_t idesc_dq = make_idesc(fmt, 128, 32, 1, 1);    // A and B MN-major
  // descriptor templates: only the start-address field changes from one MMA to the next
  const DescBase dk64 = make_desc_base(0, 16, 512, kSw64);      // K-major rows of 64 bytes
  const DescBase dm64 = make_desc_base(0, 512, 512, kSw64);     // MN-major rows of 64 bytes
  const DescBase dds = make_desc_base(0, 16384, 1024, kSw128);  // dS tile, MN-major, two slabs

  struct Bases {
    uint32_t k, v, q, dO;
  };
  auto stage_bases = [&](const Ring& kv, const Ring& qdo) {
    Bases b;
    b.k = smem_base + p.off_kv + kv.stage * p.kv_stage_bytes;
    b.v = b.k + static_cast<uint32_t>(p.rows_kv) * kRowBytes;
    b.q = smem_base + p.off_qdo + qdo.stage * kQdoStageBytes;
    b.dO = b.q + 2u * kBoxBytes;
    return b;
  };
  // S^T = K^ Q^^T and dP^T = V dO^T for the 64 queries of step w of a tile (two chunks; each chunk
  // that exists has its own barrier).  All 64 columns are always computed: query rows past the end
  // of the window are zeros in shared memory.
  const uint32_t idesc_s = make_idesc(fmt, 128, kStepCols, 0, 0);
  auto chunk_exists = [&](const TileIt& it, int w, int c) { return step_rows(g, it.i, w) - kChunkCols * c > 0; };
  auto issue_sdp = [&](const TileIt& it, int w, const Bases& b) {
    if (!chunk_exists(it, w, 0)) return;
    const uint32_t key_off = g.pair ? 0u : static_cast<uint32_t>(it.j) * (kTileRows * kRowBytes);
    const uint32_t row_off = static_cast<uint32_t>(w * kStepCols) * kRowBytes;
    const uint32_t st = tmem + w * 128u + kTmST, dpt = tmem + w * 128u + kTmDPT;
    // the two accumulation chains are interleaved: back-to-back MMAs into one accumulator wait
    // for each other
#pragma unroll
    for (uint32_t k = 0; k < 2u; ++k) {
      mma_ss(st, desc_at(dk64, b.k + key_off + 32u * k), desc_at(dk64, b.q + row_off + 32u * k), idesc_s, k);
      mma_ss(dpt, desc_at(dk64, b.v + key_off + 32u * k), desc_at(dk64, b.dO + row_off + 32u * k), idesc_s, k);
    }
    mma_commit(bar(kbStFull + 2 * w));
    if (chunk_exists(it, w, 1)) mma_commit(bar(kbStFull + 2 * w + 1));
  };

  uint32_t kdkv = 0, kdq = 0;
  const uint32_t nsets = bwd_num_sets(p, g.KB, g.MT);
  const uint32_t sets_mask = nsets - 1u, sets_shift = nsets - 1u;
  TraceCursor tr = trace_begin(p.trace, 1);
  uint32_t nst = 0u;   // phase bit per (2 * warpgroup + chunk)
  Ring kv_ring(NKV), qdo_ring(kNumQdoStages), ds_ring(NDS);
  TileIt cur{0, 0, 0};
  if (!mbar_wait(bar(kbKvReady + 0), 0u, ctx, 60)) return;
  if (!mbar_wait(bar(kbQdoReady + 0), 0u, ctx, 61)) return;
  tc_fence_after();
  {
    const Bases b0 = stage_bases(kv_ring, qdo_ring);
#pragma unroll 1
    for (int w = 0; w < 2; ++w) issue_sdp(cur, w, b0);
  }

  while (true) {
    TileIt nxt = cur;
    const bool has_next = tile_next(g, nxt);
    const bool cross = has_next && nxt.t != cur.t;
    Ring kv_next = kv_ring, qdo_next = qdo_ring;
    if (cross) kv_next.advance();
    qdo_next.advance();
    // Scores of the next tile are issued right behind this tile's dV / dK products, except across
    // a job boundary when K of the next job cannot be ready yet (single K/V stage).
    const bool look_now = has_next && !(cross && NKV < 2);
    const Bases b = stage_bases(kv_ring, qdo_ring);
    const Bases bn = stage_bases(kv_next, qdo_next);

    if (cur.i == 0) {
      // the previous key block's dK / dV must have been read out before they are overwritten
      if (!mbar_wait(bar(kbDkvFree + (kdkv & sets_mask)), ((kdkv >> sets_shift) & 1u) ^ 1u, ctx, 62)) return;
      if (cur.j == 0) {
        if (!mbar_wait(bar(kbDqFree + (kdq & sets_mask)), ((kdq >> sets_shift) & 1u) ^ 1u, ctx, 63)) return;
      }
    }
    // chunks in the order in which the two warpgroups finish them: (w0,c0) (w1,c0) (w0,c1) (w1,c1)
    // Pair mode: both chunks of a step come from the same warpgroup at the same time, so the step
    // is finished (and the next tile's scores of that warpgroup issued) before the other is looked at.
    bool looked = false;
#pragma unroll 1
    for (int idx = 0; idx < 4; ++idx) {
      {
        const int c = g.pair ? (idx & 1) : (idx >> 1), w = g.pair ? (idx >> 1) : (idx & 1);
        if (chunk_exists(cur, w, c)) {
          const int bi = 2 * w + c;
          if (!mbar_wait(bar(kbPtFull + bi), (nst >> bi) & 1u, ctx, 64)) return;
          nst ^= 1u << bi;
          tc_fence_after();
          trace_ev(tr, 30 + bi);
          const uint32_t row_off = static_cast<uint32_t>(w * kStepCols + c * kChunkCols) * kRowBytes;
          const uint32_t first = (cur.i > 0 || w > 0 || c > 0) ? 1u : 0u;
          const uint32_t a_p = tmem + w * 128u + kTmST + 32u * c, a_ds = tmem + w * 128u + kTmDPT + 32u * c;
#pragma unroll
          for (uint32_t k = 0; k < 2; ++k) {
            mma_ts(tmem + tm_dv(kdkv & sets_mask), a_p + k * 8u, desc_at(dm64, b.dO + row_off + k * 1024u),
                   idesc_acc, first | k);
            mma_ts(tmem + tm_dk(kdkv & sets_mask), a_ds + k * 8u, desc_at(dm64, b.q + row_off + k * 1024u),
                   idesc_acc, first | k);
          }
        }
        // the next tile's scores of step w go over this tile's P^T / dS^T of both chunks
        if (look_now && c == 1) {
          if (!looked) {
            if (cross) {
              if (!mbar_wait(bar(kbKvReady + kv_next.stage), kv_next.phase, ctx, 65)) return;
            }
            if (!mbar_wait(bar(kbQdoReady + qdo_next.stage), qdo_next.phase, ctx, 66)) return;
            tc_fence_after();
            looked = true;
          }
          issue_sdp(nxt, w, bn);
          trace_ev(tr, 34 + w);
        }
      }
    }
    // dQ^ of query tile cur.i += dS K^ (key block cur.j)
    {
      const uint32_t ds_base = smem_base + p.off_ds + ds_ring.stage * kDsTileBytes;
      const uint32_t kb = b.k + (g.pair ? 0u : static_cast<uint32_t>(cur.j) * (kTileRows * kRowBytes));
      const uint32_t dq_col = tmem + tm_dq(nsets, kdq & sets_mask, static_cast<uint32_t>(cur.i));
      const uint32_t first = cur.j > 0 ? 1u : 0u;
#pragma unroll 1
      for (uint32_t k = 0; k < 8; ++k)
        mma_ss(dq_col, desc_at(dds, ds_base + k * 2048u), desc_at(dm64, kb + k * 1024u), idesc_dq, first | k);
    }
    mma_commit(bar(kbDsFree + ds_ring.stage));
    mma_commit(bar(kbQdoFree + qdo_ring.stage));
    trace_ev(tr, 36);
    if (cur.i == g.MT - 1) {
      mma_commit(bar(kbDkvFull + (kdkv & sets_mask)));
      ++kdkv;
      if (cur.j == g.KB - 1) {
        mma_commit(bar(kbDqFull + (kdq & sets_mask)));
        ++kdq;
        mma_commit(bar(kbKvFree + kv_ring.stage));
      }
    }
    if (!has_next) break;
    if (!look_now) {
      if (!mbar_wait(bar(kbKvReady + kv_next.stage), kv_next.phase, ctx, 67)) return;
      if (!mbar_wait(bar(kbQdoReady + qdo_next.stage), qdo_next.phase, ctx, 68)) return;
      tc_fence_after();
#pragma unroll 1
      for (int w = 0; w < 2; ++w) issue_sdp(nxt, w, bn);
    }
    kv_ring = kv_next;
    qdo_ring = qdo_next;
    ds_ring.advance();
    cur = nxt;
  }
}

// ------------------------------------------------------------------------------------------------
// MMA issuer for pair mode (one thread).  Every tile is a job of its own (one key block, one query
// tile), every chunk exists, and the issuing thread is the busiest in the CTA: the whole tile is
// written out as straight-line code with as few waits and commits as the dependencies allow.
// Per step w one barrier announces the scores (kbStFull + 2 w) and one P^T / dS^T (kbPtFull + 2 w).
// ------------------------------------------------------------------------------------------------
template <typename T, bool kPair>
__device__ void bwd_mma_role_pair(const BwdParams& p, uint32_t smem_base, uint32_t bars, uint32_t tmem,
                                  const WaitCtx& ctx) {
  const BwdGeom g = bwd_geom<kPair>(p);
  if (g.njobs == 0) return;
  constexpr uint32_t fmt = Elem<T>::kFmt;
  auto bar = [&](int i) { return bars + 8u * i; };
  const uint32_t NKV = p.n_kv_stages, NDS = p.n_ds_bufs;
  const uint32_t idesc_acc = make_idesc(fmt, 128, 32, 0, 1);   // A in TMEM, B MN-major
  const uint32_t idesc_dq = make_idesc(fmt, 128, 32, 1, 1);    // A and B MN-major
  const uint32_t idesc_s = make_idesc(fmt, 128, kStepCols, 0, 0);
  const DescBase dk64 = make_desc_base(0, 16, 512, kSw64);      // K-major rows of 64 bytes
  const DescBase dm64 = make_desc_base(0, 512, 512, kSw64);     // MN-major rows of 64 bytes
  const DescBase dds = make_desc_base(0, 16384, 1024, kSw128);  // dS tile, MN-major, two slabs
  const uint32_t nsets = bwd_num_sets(p, 1, 1);
  const uint32_t sets_mask = nsets - 1u, sets_shift = nsets - 1u;
  const bool db_in_tmem = p.db_partial != nullptr;
  const uint32_t ident = smem_base + p.off_ident;
  const uint32_t kv_bytes = p.kv_stage_bytes, v_off = static_cast<uint32_t>(p.rows_kv) * kRowBytes;

  // S^T = K^ Q^^T and dP^T = V dO^T of step w (64 queries)
  auto issue_sdp = [&](uint32_t w, uint32_t k_base, uint32_t q_base) {
    const uint32_t row_off = w * (kStepCols * kRowBytes);
    const uint32_t st = tmem + w * 128u + kTmST, dpt = tmem + w * 128u + kTmDPT;
#pragma unroll
    for (uint32_t k = 0; k < 2u; ++k) {
      mma_ss(st, desc_at(dk64, k_base + 32u * k), desc_at(dk64, q_base + row_off + 32u * k), idesc_s, k);
      mma_ss(dpt, desc_at(dk64, k_base + v_off + 32u * k),
             desc_at(dk64, q_base + 2u * kBoxBytes + row_off + 32u * k), idesc_s, k);
    }
    mma_commit(bar(kbStFull + 2 * static_cast<int>(w)));
  };

  Ring kv_ring(NKV), qdo_ring(kNumQdoStages), ds_ring(NDS);
  uint32_t tile = 0, pt_phase = 0;
  if (!mbar_wait(bar(kbKvReady + 0), 0u, ctx, 60)) return;
  if (!mbar_wait(bar(kbQdoReady + 0), 0u, ctx, 61)) return;
  tc_fence_after();
#pragma unroll 1
  for (uint32_t w = 0; w < 2u; ++w) issue_sdp(w, smem_base + p.off_kv, smem_base + p.off_qdo);

#pragma unroll 1
  for (int t = 0; t < g.njobs; ++t, ++tile) {
    const bool has_next = t + 1 < g.njobs;
    Ring kv_next = kv_ring, qdo_next = qdo_ring;
    kv_next.advance();
    qdo_next.advance();
    const uint32_t set = tile & sets_mask, use = tile >> sets_shift;
    const uint32_t k_base = smem_base + p.off_kv + kv_ring.stage * kv_bytes;
    const uint32_t q_base = smem_base + p.off_qdo + qdo_ring.stage * kQdoStageBytes;
    const uint32_t kn_base = smem_base + p.off_kv + kv_next.stage * kv_bytes;
    const uint32_t qn_base = smem_base + p.off_qdo + qdo_next.stage * kQdoStageBytes;
    // the accumulators of this set have been read out
    if (!mbar_wait(bar(kbDkvFree + set), (use & 1u) ^ 1u, ctx, 62)) return;
    if (!mbar_wait(bar(kbDqFree + set), (use & 1u) ^ 1u, ctx, 63)) return;
#pragma unroll 1
    for (uint32_t w = 0; w < 2u; ++w) {
      if (!mbar_wait(bar(kbPtFull + 2 * static_cast<int>(w)), pt_phase, ctx, 64)) return;
      tc_fence_after();
#pragma unroll 1
      for (uint32_t c = 0; c < 2u; ++c) {
        const uint32_t row_off = (w * kStepCols + c * kChunkCols) * kRowBytes;
        const uint32_t a_p = tmem + w * 128u + kTmST + 32u * c, a_ds = tmem + w * 128u + kTmDPT + 32u * c;
#pragma unroll
        for (uint32_t k = 0; k < 2u; ++k) {
          const uint32_t acc = (w | c | k) ? 1u : 0u;
          mma_ts(tmem + tm_dv(set), a_p + k * 8u, desc_at(dm64, q_base + 2u * kBoxBytes + row_off + k * 1024u),
                 idesc_acc, acc);
          mma_ts(tmem + tm_dk(set), a_ds + k * 8u, desc_at(dm64, q_base + row_off + k * 1024u), idesc_acc, acc);
        }
      }
      // dBias^T += dS^T * I: the tensor core sums over the windows of this CTA.  Each step has its
      // own copy of the identity tile: with one shared copy the products of the step that came
      // second in a tile produced wrong sums on B200 (measured; the cause is not understood).
      if (db_in_tmem) {
#pragma unroll 1
        for (uint32_t ck = 0; ck < 4u; ++ck)   // chunk ck / 2, k-step ck % 2
          mma_ts(tmem + tm_db(w), tmem + w * 128u + kTmDPT + 32u * (ck >> 1) + (ck & 1u) * 8u,
                 desc_at(dm64, ident + 2048u * w + (ck & 1u) * 1024u), idesc_acc, 1u);
      }
      // the next tile's scores of step w go over this tile's P^T / dS^T
      if (has_next) {
        if (w == 0u) {
          if (!mbar_wait(bar(kbKvReady + kv_next.stage), kv_next.phase, ctx, 65)) return;
          if (!mbar_wait(bar(kbQdoReady + qdo_next.stage), qdo_next.phase, ctx, 66)) return;
          tc_fence_after();
        }
        issue_sdp(w, kn_base, qn_base);
      }
    }
    pt_phase ^= 1u;
    // dQ^ += dS K^
    {
      const uint32_t ds_base = smem_base + p.off_ds + ds_ring.stage * kDsTileBytes;
#pragma unroll 2
      for (uint32_t k = 0; k < 8u; ++k)
        mma_ss(tmem + tm_dq(nsets, set, 0u), desc_at(dds, ds_base + k * 2048u), desc_at(dm64, k_base + k * 1024u),
               idesc_dq, k);
    }
    mma_commit(bar(kbDsFree + ds_ring.stage));
    mma_commit(bar(kbQdoFree + qdo_ring.stage));
    mma_commit(bar(kbDkvFull + set));
    mma_commit(bar(kbDqFull + set));
    mma_commit(bar(kbKvFree + kv_ring.stage));
    kv_ring = kv_next;
    qdo_ring = qdo_next;
    ds_ring.advance();
  }
}

// ------------------------------------------------------------------------------------------------
// TMA producers: three warps (one thread each), one stream each, so that none of them ever waits
// for the consumers of another and each is a short loop of blocking waits:
//   warp 9   K/V of a job, then Q/dO of each of its tiles
//   warp 10  bias^T / mask^T chunks for warpgroup 0        warp 11  the same for warpgroup 1
// Every stream issues its loads in the order in which they are consumed.
// ------------------------------------------------------------------------------------------------
template <bool kPair>
__device__ void bwd_load_main(const BwdParams& p, uint32_t smem_base, uint32_t bars, const WaitCtx& ctx) {
  const BwdGeom g = bwd_geom<kPair>(p);
  if (g.njobs == 0) return;
  auto bar = [&](int i) { return bars + 8u * i; };
  TileIt it{0, 0, 0};
  Ring kv(p.n_kv_stages), qdo(kNumQdoStages);
  bool new_job = true;
#pragma unroll 1
  while (true) {
    if (new_job) {
      const uint32_t kvs = kv.stage;
      if (!mbar_wait<true>(bar(kbKvFree + kvs), kv.phase ^ 1u, ctx, 70)) return;
      const uint32_t k_base = smem_base + p.off_kv + kvs * p.kv_stage_bytes;
      const uint32_t v_base = k_base + static_cast<uint32_t>(p.rows_kv) * kRowBytes;
      const uint32_t full = bar(kbKvFull + kvs);
      mbar_arrive_expect_tx(full, 2u * static_cast<uint32_t>(p.rows_kv) * kRowBytes);
      const int nbox = p.rows_kv / kBoxRows;
#pragma unroll 1
      for (int b = 0; b < nbox; ++b) {
        const int bw = bwd_bw(p, g, it.t, g.pair ? b : 0);
        const int r0 = g.pair ? 0 : b * kBoxRows;
        tma_load_4d(k_base + b * kBoxBytes, &p.tm_k, full, 0, r0, g.h, bw);
        tma_load_4d(v_base + b * kBoxBytes, &p.tm_v, full, 0, r0, g.h, bw);
      }
    }
    {
      const uint32_t qs = qdo.stage;
      if (!mbar_wait<true>(bar(kbQdoFree + qs), qdo.phase ^ 1u, ctx, 71)) return;
      const uint32_t q_base = smem_base + p.off_qdo + qs * kQdoStageBytes;
      const uint32_t full = bar(kbQdoFull + qs);
      mbar_arrive_expect_tx(full, kQdoStageBytes);
      // two boxes of 64 rows; pair mode: four boxes of 32 rows, unit A and unit B alternating
      // (see pair_row_unit / pair_row_query)
      const int nb = g.pair ? 4 : 2;
      const uint32_t box_bytes = g.pair ? kBoxBytes / 2u : kBoxBytes;
#pragma unroll 1
      for (int b = 0; b < nb; ++b) {
        const int bw = bwd_bw(p, g, it.t, g.pair ? (b & 1) : 0);
        const int r0 = g.pair ? 32 * (b >> 1) : it.i * kTileRows + b * kBoxRows;
        tma_load_4d(q_base + b * box_bytes, &p.tm_q, full, 0, r0, g.h, bw);
        tma_load_4d(q_base + 2u * kBoxBytes + b * box_bytes, &p.tm_do, full, 0, r0, g.h, bw);
      }
      qdo.advance();
    }
    const int t_before = it.t;
    if (!tile_next(g, it)) return;
    new_job = it.t != t_before;
    if (new_job) kv.advance();
  }
}

// Tables of warpgroup w.  Pair mode: the warpgroup works on chunk w of both units, one table stage
// per tile.  Otherwise: the existing chunks of step w of every tile, in order.
template <bool kPair>
__device__ void bwd_load_tables(const BwdParams& p, uint32_t smem_base, uint32_t bars, const WaitCtx& ctx, int w) {
  const BwdGeom g = bwd_geom<kPair>(p);
  if (g.njobs == 0 || !(p.has_bias || p.has_mask)) return;
  auto bar = [&](int i) { return bars + 8u * i; };
  const uint32_t NBM = p.n_bm_stages;
  // two boxes of 64 keys per table; in pair mode the units share the bias box (same head) and
  // have a mask box each
  const int n_bias = p.has_bias ? (g.pair ? 1 : 2) : 0;
  const uint32_t tx_bytes = static_cast<uint32_t>(n_bias + (p.has_mask ? 2 : 0)) * kBoxBytes;
  TileIt it{0, 0, 0};
  Ring bm(NBM);
#pragma unroll 1
  do {
    const int nchunks = g.pair ? 1 : min(2, (step_rows(g, it.i, w) + kChunkCols - 1) / kChunkCols);
#pragma unroll 1
    for (int c = 0; c < nchunks; ++c) {
      const uint32_t st = bm.stage;
      if (!mbar_wait<true>(bar(kbBmFree + 2 * w + st), bm.phase ^ 1u, ctx, 72)) return;
      const uint32_t base = smem_base + p.off_bm + (w * NBM + st) * (2u * kTableTileBytes);
      const uint32_t full = bar(kbBmFull + 2 * w + st);
      mbar_arrive_expect_tx(full, tx_bytes);
      const int c0 = g.pair ? w * kChunkCols : it.i * kTileRows + w * kStepCols + c * kChunkCols;
#pragma unroll 1
      for (int hb = 0; hb < 2; ++hb) {
        const int r0 = g.pair ? 0 : it.j * kTileRows + hb * kBoxRows;
        if (hb < n_bias) tma_load_3d(base + hb * kBoxBytes, &p.tm_biasT, full, c0, r0, g.h);
        if (p.has_mask) {
          const int bw = bwd_bw(p, g, it.t, g.pair ? hb : 0);
          tma_load_3d(base + kTableTileBytes + hb * kBoxBytes, &p.tm_maskT, full, c0, r0,
                      bw < p.BW ? bw % p.nW : 0);
        }
      }
      bm.advance();
    }
  } while (tile_next(g, it));
}

// ------------------------------------------------------------------------------------------------
template <typename T, bool kPair>
__global__ void __launch_bounds__(kBwdThreads, 1) bwd_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t tid = threadIdx.x;
  const uint32_t warp = tid >> 5;
  const uint32_t lane = tid & 31u;
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t bars = smem_base + p.off_ctrl;
  uint32_t* ctrl_words = reinterpret_cast<uint32_t*>(smem_raw + p.off_ctrl + 8u * kBwdNumBars);
  uint32_t& tmem_slot = ctrl_words[0];
  float* warp_sums = reinterpret_cast<float*>(&ctrl_words[4]);
  if ((smem_base & 1023u) != 0u) {
    if (tid == 0 && p.status != nullptr) atomicCAS(&p.status->code, 0u, (99u << 8) | 2u);
    return;
  }

  if (tid == 0) {
    ctrl_words[1] = 0u;
    for (int i = 0; i < kBwdNumBars; ++i) {
      // jobs of a single tile: dQ is written by warpgroup 0 alone
      const bool single = kPair || p.N <= kTileRows;
      uint32_t count = 1u;
      if (i >= kbKvReady && i < kbKvFree) count = 128u;   // the preparing warpgroup
      else if (i >= kbKvFree && i < kbQdoFull) count = 257u;
      else if (i >= kbQdoReady && i < kbQdoFree) count = 128u;
      else if (i >= kbPtFull && i < kbBmFull) count = 128u;   // four chunk barriers
      else if (i >= kbBmFree && i < kbDsFree) count = 128u;
      else if (i >= kbDkvFree && i < kbDqFull) count = 256u;
      else if (i >= kbDqFree && i < kBwdNumBars) count = single ? 128u : 256u;
      mbar_init(bars + 8u * i, count);
    }
    mbar_fence_init();
    tma_prefetch_desc(&p.tm_q);
    tma_prefetch_desc(&p.tm_k);
    tma_prefetch_desc(&p.tm_v);
    tma_prefetch_desc(&p.tm_do);
    if (p.has_bias) tma_prefetch_desc(&p.tm_biasT);
    if (p.has_mask) tma_prefetch_desc(&p.tm_maskT);
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(&tmem_slot), kBwdTmemCols);
    tmem_relinquish();
  }
  // 32 x 32 identity in the layout of a dO chunk (row = query, 64 bytes of columns, 16-byte pieces
  // XOR-swizzled with the row), two copies: B operand of the products that sum dS^T into dBias^T
  for (uint32_t wj = tid; wj < 1024u; wj += kBwdThreads) {
    const uint32_t wi = wj & 511u;
    const uint32_t row = wi >> 4, piece = (wi >> 2) & 3u, word = wi & 3u;   // word = two columns
    const uint32_t col = ((piece ^ ((row >> 1) & 3u)) << 3) + 2u * word;     // logical column of the low half
    const uint32_t one = Elem<T>::pack(1.f, 0.f) & 0xFFFFu;
    uint32_t v = 0u;
    if (col == row) v = one;
    if (col + 1u == row) v = one << 16;
    reinterpret_cast<uint32_t*>(smem_raw + p.off_ident)[wj] = v;
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  WaitCtx ctx{&ctrl_words[1], p.status, (p.trace.buf != nullptr && p.trace.cap >= 700) ? p.trace.buf + 2ll * p.trace.cap + 500 : nullptr};

#if FWA2_TRACE
  // per-CTA wall time, clock cycles and SM id in the producer's (otherwise unused) trace region
  unsigned long long t_start = 0;
  long long c_start = 0;
  if (tid == 0 && p.trace.buf != nullptr) {
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_start));
    c_start = clock64();
  }
#endif
  float dscale_acc = 0.f;
  // 512 threads start with 128 registers each; the compute warpgroups take what the others give up
  if (warp < 8) {
    reg_alloc<176>();
    bwd_compute_role<T, kPair>(p, smem_raw, smem_base, bars, tmem, ctx, dscale_acc);
  } else if (warp < 12) {
    reg_dealloc<80>();
    if (lane == 0) {
      if (warp == 8) {
        if constexpr (kPair) bwd_mma_role_pair<T, true>(p, smem_base, bars, tmem, ctx);
        else bwd_mma_role<T, false>(p, smem_base, bars, tmem, ctx);
      } else if (warp == 9) bwd_load_main<kPair>(p, smem_base, bars, ctx);
      else bwd_load_tables<kPair>(p, smem_base, bars, ctx, static_cast<int>(warp) - 10);
    }
  } else {
    reg_dealloc<80>();
    bwd_prepare_role<T, kPair>(p, smem_raw, smem_base, bars, ctx);
  }
  __syncwarp();
  // deterministic CTA-wide sum of the dLogitScale contributions
  if (warp < 8) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dscale_acc += __shfl_xor_sync(0xFFFFFFFFu, dscale_acc, off);
    if (lane == 0) warp_sums[warp] = dscale_acc;
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && p.dscale_partial != nullptr) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += warp_sums[w];
    p.dscale_partial[blockIdx.x] =
        s * load_scale<T>(p.scale, p.scale_is_tensor, static_cast<int>(blockIdx.x) % p.H);
  }
#if FWA2_TRACE
  if (tid == 0 && p.trace.buf != nullptr && 3 * blockIdx.x + 2 < p.trace.cap) {
    unsigned long long t_end;
    uint32_t smid;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_end));
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    p.trace.buf[2ll * p.trace.cap + 3 * blockIdx.x] = t_start;
    p.trace.buf[2ll * p.trace.cap + 3 * blockIdx.x + 1] = t_end;
    p.trace.buf[2ll * p.trace.cap + 3 * blockIdx.x + 2] =
        (smid + 1000) | (static_cast<unsigned long long>(clock64() - c_start) << 16);
  }
#endif
  if (tid == 0) report_abort(ctrl_words[1], p.status);
  if (ctrl_words[1]) {
    __nanosleep(20000);
    __syncthreads();
  }
  if (warp == 8) tmem_dealloc(tmem, kBwdTmemCols);
}

template __global__ void bwd_kernel<__nv_bfloat16, false>(const __grid_constant__ BwdParams);
template __global__ void bwd_kernel<__nv_bfloat16, true>(const __grid_constant__ BwdParams);
template __global__ void bwd_kernel<__half, false>(const __grid_constant__ BwdParams);
template __global__ void bwd_kernel<__half, true>(const __grid_constant__ BwdParams);

cudaError_t launch_bwd(const BwdParams& p, int dtype_is_bf16, int grid, cudaStream_t stream) {
  auto go = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(p.smem_bytes));
    if (e != cudaSuccess) return e;
    kern<<<grid, kBwdThreads, p.smem_bytes, stream>>>(p);
    return cudaGetLastError();
  };
  if (p.pair_mode) return dtype_is_bf16 ? go(bwd_kernel<__nv_bfloat16, true>) : go(bwd_kernel<__half, true>);
  return dtype_is_bf16 ? go(bwd_kernel<__nv_bfloat16, false>) : go(bwd_kernel<__half, false>);
}

}  // namespace fwa2
