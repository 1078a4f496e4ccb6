// Forward kernel: fused L2-normalisation of Q and K, cosine scores on the tcgen05 tensor cores
// (accumulators in tensor memory), per-head clamped logit scale, relative-position bias,
// shifted-window mask, online softmax, P*V and the log-sum-exp, in one pass.
//
// One persistent CTA handles a sequence of jobs (one unit, or two units of <= 64 tokens).  Roles:
//   warps 0-3  softmax: thread t owns query row t of the current 128-row tile
//   warp  4    issues every tcgen05.mma (one thread)
//   warp  5    TMA producer (one thread): K, V, Q tiles and the bias / mask table chunks
// Replaces flash_win_attn_v2/kernels/attn_kernel_forward.py:21-258 (`_fwd_kernel`).
#ifndef FWA2_FWD_ROLLED_STEP
#define FWA2_FWD_ROLLED_STEP 0
#endif
#ifndef FWA2_FWD_NORMALISE_ROLLED
#define FWA2_FWD_NORMALISE_ROLLED 0
#endif
#ifndef FWA2_FWD_WAIT_INLINE
#define FWA2_FWD_WAIT_INLINE 1
#endif
#define FWA2_NORMALISE_ROLLED FWA2_FWD_NORMALISE_ROLLED
#define FWA2_WAIT_INLINE FWA2_FWD_WAIT_INLINE
#include "fwa2_common.cuh"

namespace fwa2 {

constexpr int kFwdThreads = 192;
constexpr uint32_t kFwdTmemCols = 256;
constexpr uint32_t kTmemS = 0;      // scores: two 64-column step buffers (one 128-column tile in pair mode)
constexpr uint32_t kTmemPV = 128;   // 32 columns: P*V of one step
constexpr uint32_t kTmemP = 160;    // packed P: 32 columns per step (64 in pair mode)

enum FwdBar : int {
  kBarKvFull = 0, kBarKvReady = 2, kBarKvFree = 4,
  kBarQFull = 6, kBarQReady = 8, kBarQFree = 10,
  kBarSFull = 12, kBarSFree = 14,
  kBarBmFull = 16, kBarBmFree = 20,
  kBarPFull = 24, kBarPvDone = 25,
  kFwdNumBars = 26
};

struct FwdShape {
  int N, H, U, pair, MT, KS, rows_kv;
};

// kPair is a template parameter of the kernel: a launch runs code specialised for its mode and the
// instruction cache holds none of the other mode's branches.
template <bool kPair>
__device__ __forceinline__ FwdShape fwd_shape(const FwdParams& p) {
  FwdShape s;
  s.N = p.N;
  s.H = p.H;
  s.U = p.BW * p.H;
  s.pair = kPair ? 1 : 0;
  s.MT = s.pair ? 1 : (p.N + kTileRows - 1) / kTileRows;
  s.KS = s.pair ? 1 : (p.N + kStepCols - 1) / kStepCols;
  s.rows_kv = s.pair ? 128 : ((p.N + 63) / 64) * 64;
  return s;
}

// (window, head, mask plane) of the one or two units of a job; recomputed when the job changes.
// Out of line: four integer divisions by run-time values, needed at four places of the producer.
struct JobUnits { int bw0, bw1, h0, h1, mw0, mw1; };
static __device__ __noinline__ JobUnits job_units(int job, bool pair, int H, int nW) {
  JobUnits u;
  const int u0 = pair ? 2 * job : job, u1 = pair ? 2 * job + 1 : job;
  u.bw0 = u0 / H; u.h0 = u0 - u.bw0 * H; u.mw0 = nW > 0 ? u.bw0 % nW : 0;
  u.bw1 = u1 / H; u.h1 = u1 - u.bw1 * H; u.mw1 = nW > 0 ? u.bw1 % nW : 0;
  return u;
}

// ------------------------------------------------------------------------------------------------
// Softmax warps
// ------------------------------------------------------------------------------------------------
template <typename T, bool kPTmem, bool kPair>
__device__ void fwd_softmax_role(const FwdParams& p, uint32_t smem_base, uint32_t bars,
                                 uint32_t tmem, const WaitCtx& ctx, const float* scale_tab) {
  const FwdShape sh = fwd_shape<kPair>(p);
  const uint32_t tid = threadIdx.x;          // 0..127 = row of the tile
  const uint32_t hf = tid >> 6;
  const uint32_t lane_base = ((tid >> 5) * 32u) << 16;
  const bool any_table = p.has_bias || p.has_mask;
  const uint32_t rt_zero = static_cast<uint32_t>(p.N) >> 30;   // 0, but not to the compiler
  auto bar = [&](int i) { return bars + 8u * i; };

  if (sh.pair) {
    // The half of P that belongs to the other unit of the pair stays zero for the whole kernel.
    if constexpr (kPTmem) {
      uint32_t z[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) z[i] = 0u;
      tmem_st16(tmem + lane_base + kTmemP + (hf ^ 1u) * 32u, z);
      tmem_st16(tmem + lane_base + kTmemP + (hf ^ 1u) * 32u + 16u, z);
      tmem_wait_st();
    } else {
      const uint32_t z[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        sts128(smem_base + p.off_p + (hf ^ 1u) * 16384u + sw128_offset(tid, ch), z);
    }
  }

  uint32_t tt = 0, pvc = 0;
  Ring kv_ring(p.n_kv_stages), s_ring(sh.pair ? 1u : 2u), bm_ring(p.n_bm_stages);
  TraceCursor tr = (tid == 0) ? trace_begin(p.trace, 0) : TraceCursor{nullptr, 0};
  // ---- K rows of a job (what = 0) and my Q row of a tile (what = 1), normalised in place.  One
  // loop for both, so that the normalisation code exists once per call site. ----
  auto prepare = [&](bool with_kv, const Ring& r, uint32_t ttn) -> bool {
#pragma unroll 1
    for (int what = with_kv ? 0 : 1; what < 2; ++what) {
      const uint32_t kvs = r.stage, qs = ttn & 1u;
      const uint32_t base = what == 0 ? smem_base + p.off_kv + kvs * p.kv_stage_bytes
                                      : smem_base + p.off_q + qs * (2u * kBoxBytes);
      const uint32_t rows = what == 0 ? static_cast<uint32_t>(sh.rows_kv) : static_cast<uint32_t>(kTileRows);
      if (!mbar_wait(bar(what == 0 ? kBarKvFull + kvs : kBarQFull + qs), what == 0 ? r.phase : ((ttn >> 1) & 1u),
                     ctx, 10 + what))
        return false;
      trace_ev(tr, 1 + 2 * what);
#pragma unroll 1
      for (uint32_t rr = tid; rr < rows; rr += 128u) normalise_row<T>(base, rr);
      fence_proxy_async_smem();
      mbar_arrive(bar(what == 0 ? kBarKvReady + kvs : kBarQReady + qs));
      trace_ev(tr, 2 + 2 * what);
    }
    return true;
  };
  // The prologue of the NEXT tile runs before the epilogue of the current one, so that the MMA
  // warp can already produce the next scores while this tile's output is written.
  bool kv_ahead = false, q_ahead = false;

  for (int job = blockIdx.x; job < p.n_jobs; job += gridDim.x, kv_ring.advance()) {
    const int unit = sh.pair ? 2 * job + static_cast<int>(hf) : job;
    const bool unit_ok = unit < sh.U;
    const int bw = unit / sh.H, h = unit - bw * sh.H;
    const float scale = scale_tab[h];

    // (ahead: already done at the end of the previous tile)
    const bool need_kv = !kv_ahead;
    kv_ahead = false;

    for (int mt = 0; mt < sh.MT; ++mt, ++tt) {
      if (!q_ahead) {
        if (!prepare(need_kv && mt == 0, kv_ring, tt)) return;
      }
      q_ahead = false;

      const int row = sh.pair ? static_cast<int>(tid & 63u) : mt * kTileRows + static_cast<int>(tid);
      const bool row_ok = unit_ok && row < sh.N;

      float m_run = -INFINITY, l_run = 0.f, alpha_pend = 0.f;
      float acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0.f;

#if FWA2_FWD_ROLLED_STEP
      for (int s = 0; s < sh.KS; ++s, s_ring.advance()) {
        const int ncols = sh.pair ? sh.N : min(kStepCols, sh.N - s * kStepCols);
        const int nch = ncols > kChunkCols ? 2 : 1;
        const uint32_t sb = s_ring.stage;
        if (!mbar_wait(bar(kBarSFull + sb), s_ring.phase, ctx, 12)) return;
        tc_fence_after();
        trace_ev(tr, 10);
        const uint32_t t_s = tmem + lane_base + kTmemS + (sh.pair ? hf * 64u : sb * 64u);

        // Both passes over the 64 scores of the row run as rolled loops over groups of eight
        // columns (this kernel is bound by instruction fetch: the loop bodies have to stay in the
        // instruction cache), two groups per trip so that the tensor-memory load of one group
        // overlaps the arithmetic of the other.
        // ---- pass 1: x = scale * cos + bias + mask, written back over the scores; row maximum ----
        float mxp[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        {
          const uint32_t row_off = tid * 64u, row_sw = (tid >> 1) & 3u;
          uint32_t bm_base = 0;
          auto group1 = [&](uint32_t g8, uint32_t (&r)[8]) {
            // g8: group index 0..7; r: its eight scores, replaced by x
            const int col0 = static_cast<int>(g8) * 8;
            const bool live = any_table && static_cast<int>(g8 >> 2) < nch;
            uint32_t wb[4] = {0u, 0u, 0u, 0u}, wm[4] = {0u, 0u, 0u, 0u};
            if (live) {
              const uint32_t off = row_off + (((g8 & 3u) ^ row_sw) << 4);
              if (p.has_bias) lds128(bm_base + off, wb);
              if (p.has_mask) lds128(bm_base + kTableTileBytes + off, wm);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float x0 = fmaf(__uint_as_float(r[2 * i]), scale, Elem<T>::lo(wb[i])) + Elem<T>::lo(wm[i]);
              float x1 = fmaf(__uint_as_float(r[2 * i + 1]), scale, Elem<T>::hi(wb[i])) + Elem<T>::hi(wm[i]);
              if (col0 + 8 > ncols) {   // columns past the end of the window
                if (col0 + 2 * i >= ncols) x0 = -INFINITY;
                if (col0 + 2 * i + 1 >= ncols) x1 = -INFINITY;
              }
              mxp[i] = fmaxf(mxp[i], fmaxf(x0, x1));
              r[2 * i] = __float_as_uint(x0);
              r[2 * i + 1] = __float_as_uint(x1);
            }
          };
          uint32_t ra[8], rb[8];
          tmem_ld8(t_s, ra);
#pragma unroll 1
          for (uint32_t g8 = 0; g8 < 8u; g8 += 2u) {
            if ((g8 & 3u) == 0u && any_table && static_cast<int>(g8 >> 2) < nch) {
              const uint32_t st = bm_ring.stage;
              bm_base = smem_base + p.off_bm + st * (2u * kTableTileBytes);
              if (!mbar_wait(bar(kBarBmFull + st), bm_ring.phase, ctx, 13)) return;
            }
            tmem_wait_ld();
            tmem_ld8(t_s + 8u * (g8 + 1u), rb);
            group1(g8, ra);
            tmem_st8(t_s + 8u * g8, ra);
            tmem_wait_ld();
            if (g8 + 2u < 8u) tmem_ld8(t_s + 8u * (g8 + 2u), ra);
            group1(g8 + 1u, rb);
            tmem_st8(t_s + 8u * (g8 + 1u), rb);
            if ((g8 & 3u) == 2u && any_table && static_cast<int>(g8 >> 2) < nch) {
              mbar_arrive(bar(kBarBmFree + bm_ring.stage));
              bm_ring.advance();
            }
          }
        }
        trace_ev(tr, 12);
        // ---- online softmax ----
        const float mx = fmaxf(fmaxf(mxp[0], mxp[1]), fmaxf(mxp[2], mxp[3]));
        const float m_new = fmaxf(m_run, mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = ex2f((m_run - m_use) * kLog2e);
        const float ml2 = m_use * kLog2e;
        trace_ev(tr, 13);
        // ---- fold the previous step's P*V into the running output (this also makes sure that the
        // tensor core has finished reading the previous P before pass 2 overwrites it) ----
        if (s > 0) {
          if (!mbar_wait(bar(kBarPvDone), pvc & 1u, ctx, 14)) return;
          ++pvc;
          tc_fence_after();
          uint32_t r[32];
          tmem_ld32(tmem + lane_base + kTmemPV, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = fmaf(acc[i], alpha_pend, __uint_as_float(r[i]));
        }
        alpha_pend = alpha;
        trace_ev(tr, 14);

        tmem_wait_st();
        // ---- pass 2: p = exp(x - max), row sum, P handed to the tensor core in 16-bit pairs ----
        float sp[4] = {0.f, 0.f, 0.f, 0.f};
        {
          const uint32_t t_p = tmem + lane_base + kTmemP + (sh.pair ? hf * 32u : 0u);
          const uint32_t p_row = smem_base + p.off_p + (sh.pair ? hf * 16384u : 0u) + tid * 128u, p_sw = tid & 7u;
          auto group2 = [&](uint32_t g8, const uint32_t (&r)[8]) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float p0 = ex2f(fmaf(__uint_as_float(r[2 * i]), kLog2e, -ml2));
              const float p1 = ex2f(fmaf(__uint_as_float(r[2 * i + 1]), kLog2e, -ml2));
              sp[i] += p0 + p1;
              w[i] = Elem<T>::pack(p0, p1);
            }
            if constexpr (kPTmem) tmem_st4(t_p + 4u * g8, w);
            else sts128(p_row + ((g8 ^ p_sw) << 4), w);
          };
          uint32_t ra[8], rb[8];
          tmem_ld8(t_s, ra);
#pragma unroll 1
          for (uint32_t g8 = 0; g8 < 8u; g8 += 2u) {
            tmem_wait_ld();
            tmem_ld8(t_s + 8u * (g8 + 1u), rb);
            group2(g8, ra);
            tmem_wait_ld();
            if (g8 + 2u < 8u) tmem_ld8(t_s + 8u * (g8 + 2u), ra);
            group2(g8 + 1u, rb);
          }
        }
        // the scores are no longer needed: the tensor core may overwrite them
        tc_fence_before();
        mbar_arrive(bar(kBarSFree + sb));
        trace_ev(tr, 11);
        const float sum = (sp[0] + sp[1]) + (sp[2] + sp[3]);
        l_run = fmaf(l_run, alpha, sum);
        m_run = m_new;

        // ---- hand P to the tensor core ----
        if constexpr (kPTmem) {
          tmem_wait_st();
          tc_fence_before();
        } else {
          fence_proxy_async_smem();
          tc_fence_before();
        }
        mbar_arrive(bar(kBarPFull));
        trace_ev(tr, 15);
      }

#else
      for (int s = 0; s < sh.KS; ++s, s_ring.advance()) {
        const int ncols = sh.pair ? sh.N : min(kStepCols, sh.N - s * kStepCols);
        // ---- scores of this step out of tensor memory ----
        const uint32_t sb = s_ring.stage;
        if (!mbar_wait(bar(kBarSFull + sb), s_ring.phase, ctx, 12)) return;
        tc_fence_after();
        trace_ev(tr, 10);
        float x[64];
        {
          const uint32_t col = kTmemS + (sh.pair ? hf * 64u : sb * 64u);
          uint32_t r0[32], r1[32];
          tmem_ld32(tmem + lane_base + col, r0);
          tmem_ld32(tmem + lane_base + col + 32u, r1);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            x[i] = __uint_as_float(r0[i]);
            x[32 + i] = __uint_as_float(r1[i]);
          }
        }
        tc_fence_before();
        mbar_arrive(bar(kBarSFree + sb));
        trace_ev(tr, 11);

        // ---- x = scale * cos + bias + mask ----
        if (any_table) {
          const int nch = ncols > kChunkCols ? 2 : 1;
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            if (c2 < nch) {
              const uint32_t st = bm_ring.stage;
              const uint32_t bm_base = smem_base + p.off_bm + st * (2u * kTableTileBytes);
              if (!mbar_wait(bar(kBarBmFull + st), bm_ring.phase, ctx, 13)) return;
              uint32_t loaded = 0u;
#pragma unroll
              for (int ch = 0; ch < 4; ++ch) {
                uint32_t wb[4] = {0u, 0u, 0u, 0u}, wm[4] = {0u, 0u, 0u, 0u};
                if (p.has_bias) lds128(bm_base + sw64_offset(tid, ch), wb);
                if (p.has_mask) lds128(bm_base + kTableTileBytes + sw64_offset(tid, ch), wm);
                loaded |= wb[0] | wm[0];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int j = c2 * 32 + ch * 8 + i * 2;
                  x[j] = fmaf(x[j], scale, Elem<T>::lo(wb[i])) + Elem<T>::lo(wm[i]);
                  x[j + 1] = fmaf(x[j + 1], scale, Elem<T>::hi(wb[i])) + Elem<T>::hi(wm[i]);
                }
              }
              mbar_arrive_after_loads(bar(kBarBmFree + st), loaded, rt_zero);
              bm_ring.advance();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) x[c2 * 32 + i] *= scale;
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) x[i] *= scale;
        }
        if (ncols < kStepCols) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (i >= ncols) x[i] = -INFINITY;
        }

        trace_ev(tr, 12);
        // ---- online softmax ----
        // eight independent chains instead of one 64-long dependent one
        float mxp[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mxp[i] = x[i];
#pragma unroll
        for (int i = 8; i < 64; ++i) mxp[i & 7] = fmaxf(mxp[i & 7], x[i]);
        const float mx = fmaxf(fmaxf(fmaxf(mxp[0], mxp[1]), fmaxf(mxp[2], mxp[3])),
                               fmaxf(fmaxf(mxp[4], mxp[5]), fmaxf(mxp[6], mxp[7])));
        const float m_new = fmaxf(m_run, mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = ex2f((m_run - m_use) * kLog2e);
        const float ml2 = m_use * kLog2e;
        float sp[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) sp[i] = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          x[i] = ex2f(fmaf(x[i], kLog2e, -ml2));
          sp[i & 7] += x[i];
        }
        const float sum = ((sp[0] + sp[1]) + (sp[2] + sp[3])) + ((sp[4] + sp[5]) + (sp[6] + sp[7]));
        l_run = fmaf(l_run, alpha, sum);
        m_run = m_new;

        trace_ev(tr, 13);
        // ---- fold the previous step's P*V into the running output ----
        if (s > 0) {
          if (!mbar_wait(bar(kBarPvDone), pvc & 1u, ctx, 14)) return;
          ++pvc;
          tc_fence_after();
          uint32_t r[32];
          tmem_ld32(tmem + lane_base + kTmemPV, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = fmaf(acc[i], alpha_pend, __uint_as_float(r[i]));
        }
        alpha_pend = alpha;
        trace_ev(tr, 14);

        // ---- hand P to the tensor core ----
        if constexpr (kPTmem) {
          uint32_t w[16];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              w[i] = Elem<T>::pack(x[half * 32 + 2 * i], x[half * 32 + 2 * i + 1]);
            tmem_st16(tmem + lane_base + kTmemP + (sh.pair ? hf * 32u : 0u) + half * 16u, w);
          }
          tmem_wait_st();
          tc_fence_before();
        } else {
          const uint32_t p_base = smem_base + p.off_p + (sh.pair ? hf * 16384u : 0u);
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) w[i] = Elem<T>::pack(x[ch * 8 + 2 * i], x[ch * 8 + 2 * i + 1]);
            sts128(p_base + sw128_offset(tid, ch), w);
          }
          fence_proxy_async_smem();
          tc_fence_before();
        }
        mbar_arrive(bar(kBarPFull));
        trace_ev(tr, 15);
      }

#endif
      // ---- prologue of the next tile (and job) ----
      {
        const bool next_tile = mt + 1 < sh.MT;
        const bool next_job = !next_tile && job + static_cast<int>(gridDim.x) < p.n_jobs && p.n_kv_stages >= 2;
        if (next_tile || next_job) {
          Ring nx = kv_ring;
          if (next_job) nx.advance();
          if (!prepare(next_job, nx, tt + 1)) return;
          q_ahead = true;
          kv_ahead = next_job;
        }
      }

      // ---- last P*V of the tile, then the epilogue ----
      if (!mbar_wait(bar(kBarPvDone), pvc & 1u, ctx, 15)) return;
      ++pvc;
      tc_fence_after();
      trace_ev(tr, 20);
      {
        uint32_t r[32];
        tmem_ld32(tmem + lane_base + kTmemPV, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = fmaf(acc[i], alpha_pend, __uint_as_float(r[i]));
      }
      tc_fence_before();
      if (row_ok) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint16_t* dst = static_cast<uint16_t*>(p.o) + bw * p.o_sbw + h * p.o_sh + row * p.o_sn;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint4 v;
          v.x = Elem<T>::pack(acc[ch * 8 + 0] * inv, acc[ch * 8 + 1] * inv);
          v.y = Elem<T>::pack(acc[ch * 8 + 2] * inv, acc[ch * 8 + 3] * inv);
          v.z = Elem<T>::pack(acc[ch * 8 + 4] * inv, acc[ch * 8 + 5] * inv);
          v.w = Elem<T>::pack(acc[ch * 8 + 6] * inv, acc[ch * 8 + 7] * inv);
          *reinterpret_cast<uint4*>(dst + ch * 8) = v;
        }
        const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
        p.lse[bw * p.lse_sbw + h * p.lse_sh + row] =
            l_run > 0.f ? m_use + __logf(l_run) : -INFINITY;
      }
      trace_ev(tr, 21);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// MMA issuer (one thread)
// ------------------------------------------------------------------------------------------------
template <typename T, bool kPTmem, bool kPair>
__device__ void fwd_mma_role(const FwdParams& p, uint32_t smem_base, uint32_t bars, uint32_t tmem,
                             const WaitCtx& ctx) {
  const FwdShape sh = fwd_shape<kPair>(p);
  constexpr uint32_t fmt = Elem<T>::kFmt;
  auto bar = [&](int i) { return bars + 8u * i; };
  const uint32_t idesc_pv = make_idesc(fmt, 128, 32, 0, 1);
  const uint32_t idesc_s_full = make_idesc(fmt, 128, sh.pair ? 128u : 64u, 0, 0);
  // the last step of a tile may cover fewer key columns
  const int last_cols = sh.pair ? 128 : min(kStepCols, ((sh.N - (sh.KS - 1) * kStepCols + 15) / 16) * 16);
  const uint32_t idesc_s_last = make_idesc(fmt, 128, static_cast<uint32_t>(last_cols), 0, 0);
  const uint32_t pv_ksteps = sh.pair ? 8u : 4u;
  uint32_t tt = 0, pc = 0;
  Ring kv_ring(p.n_kv_stages), s_ring(sh.pair ? 1u : 2u);
  TraceCursor tr = trace_begin(p.trace, 1);
  // descriptor templates: only the start-address field changes from one MMA to the next
  const DescBase d64 = make_desc_base(0, 16, 512, kSw64);       // K-major rows of 64 bytes
  const DescBase dv64 = make_desc_base(0, 512, 512, kSw64);     // MN-major rows of 64 bytes
  const DescBase dp128 = make_desc_base(smem_base + p.off_p, 16, 1024, kSw128);

  for (int job = blockIdx.x; job < p.n_jobs; job += gridDim.x, kv_ring.advance()) {
    const uint32_t kvs = kv_ring.stage;
    const uint32_t k_base = smem_base + p.off_kv + kvs * p.kv_stage_bytes;
    const uint32_t v_base = k_base + static_cast<uint32_t>(sh.rows_kv) * kRowBytes;
    if (!mbar_wait(bar(kBarKvReady + kvs), kv_ring.phase, ctx, 20)) return;
    trace_ev(tr, 30);

    for (int mt = 0; mt < sh.MT; ++mt, ++tt) {
      const uint32_t qs = tt & 1u;
      const uint32_t q_base = smem_base + p.off_q + qs * (2u * kBoxBytes);
      if (!mbar_wait(bar(kBarQReady + qs), (tt >> 1) & 1u, ctx, 21)) return;
      tc_fence_after();
      trace_ev(tr, 31);

      auto issue_scores = [&](int s) -> bool {
        const uint32_t sb = s_ring.stage;
        if (!mbar_wait(bar(kBarSFree + sb), s_ring.phase ^ 1u, ctx, 22)) return false;
        tc_fence_after();
        const uint32_t kb = sh.pair ? k_base : k_base + static_cast<uint32_t>(s) * (kStepCols * kRowBytes);
        const uint32_t dcol = tmem + kTmemS + (sh.pair ? 0u : sb * 64u);
        const uint32_t idesc = (s == sh.KS - 1) ? idesc_s_last : idesc_s_full;
        mma_ss(dcol, desc_at(d64, q_base), desc_at(d64, kb), idesc, 0u);
        mma_ss(dcol, desc_at(d64, q_base + 32u), desc_at(d64, kb + 32u), idesc, 1u);
        mma_commit(bar(kBarSFull + sb));
        s_ring.advance();
        trace_ev(tr, 32);
        return true;
      };

      if (!issue_scores(0)) return;
      for (int s = 0; s < sh.KS; ++s, ++pc) {
        if (s + 1 < sh.KS) {
          if (!issue_scores(s + 1)) return;
        }
        if (s + 1 == sh.KS) mma_commit(bar(kBarQFree + qs));
        if (!mbar_wait(bar(kBarPFull), pc & 1u, ctx, 23)) return;
        tc_fence_after();
        trace_ev(tr, 33);
        const uint32_t vb = sh.pair ? v_base : v_base + static_cast<uint32_t>(s) * (kStepCols * kRowBytes);
        if constexpr (kPTmem) {
#pragma unroll 1
          for (uint32_t k = 0; k < pv_ksteps; ++k)
            mma_ts(tmem + kTmemPV, tmem + kTmemP + k * 8u, desc_at(dv64, vb + k * 1024u), idesc_pv, k);
        } else {
#pragma unroll 1
          for (uint32_t k = 0; k < pv_ksteps; ++k)
            mma_ss(tmem + kTmemPV, desc_at(dp128, (k >> 2) * 16384u + (k & 3u) * 32u),
                   desc_at(dv64, vb + k * 1024u), idesc_pv, k);
        }
        mma_commit(bar(kBarPvDone));
        trace_ev(tr, 34);
      }
    }
    mma_commit(bar(kBarKvFree + kvs));
  }
}

// ------------------------------------------------------------------------------------------------
// TMA producer (one thread).  Two independent streams are interleaved without ever blocking on
// one of them: (a) K/V of a job and the Q tiles of its 128-row tiles, which run ahead by a whole
// job when two K/V stages fit, and (b) the bias / mask table chunks, which stay a few chunks
// ahead of the softmax warps.
// ------------------------------------------------------------------------------------------------
template <bool kPair>
__device__ void fwd_load_role(const FwdParams& p, uint32_t smem_base, uint32_t bars,
                              const WaitCtx& ctx) {
  const FwdShape sh = fwd_shape<kPair>(p);
  auto bar = [&](int i) { return bars + 8u * i; };
  const bool any_table = p.has_bias || p.has_mask;
  const uint32_t table_bytes =
      (p.has_bias ? kTableTileBytes : 0u) + (p.has_mask ? kTableTileBytes : 0u);

  // stream (a): item 0 of a job is K/V, items 1..MT are the Q tiles
  int a_job = blockIdx.x, a_item = 0;
  uint32_t a_tt = 0;
  Ring a_kv(p.n_kv_stages), b_ring(p.n_bm_stages);
  // stream (b)
  int b_job = blockIdx.x, b_mt = 0, b_s = 0, b_c2 = 0;
  bool a_done = a_job >= p.n_jobs;
  bool b_done = !any_table || b_job >= p.n_jobs;

  JobUnits a_u = job_units(a_job, kPair, sh.H, p.has_mask ? p.nW : 0);
  JobUnits b_u = job_units(b_job, kPair, sh.H, p.has_mask ? p.nW : 0);

  long long t0 = clock64();
  uint32_t idle = 0;
  TraceCursor tr = trace_begin(p.trace, 2);
#pragma unroll 1
  while (!a_done || !b_done) {
    bool progress = false;
    if (!a_done) {
      if (a_item == 0) {
        const uint32_t kvs = a_kv.stage;
        if (mbar_test_wait(bar(kBarKvFree + kvs), a_kv.phase ^ 1u)) {
          const uint32_t k_base = smem_base + p.off_kv + kvs * p.kv_stage_bytes;
          const uint32_t v_base = k_base + static_cast<uint32_t>(sh.rows_kv) * kRowBytes;
          const uint32_t full = bar(kBarKvFull + kvs);
          mbar_arrive_expect_tx(full, 2u * static_cast<uint32_t>(sh.rows_kv) * kRowBytes);
          const int nbox = sh.rows_kv / kBoxRows;
#pragma unroll 1
          for (int b = 0; b < nbox; ++b) {
            const int ui = sh.pair ? b : 0;
            const int r0 = sh.pair ? 0 : b * kBoxRows;
            tma_load_4d(k_base + b * kBoxBytes, &p.tm_k, full, 0, r0, ui ? a_u.h1 : a_u.h0, ui ? a_u.bw1 : a_u.bw0);
            tma_load_4d(v_base + b * kBoxBytes, &p.tm_v, full, 0, r0, ui ? a_u.h1 : a_u.h0, ui ? a_u.bw1 : a_u.bw0);
          }
          a_item = 1;
          progress = true;
          trace_ev(tr, 40);
        }
      } else {
        const uint32_t qs = a_tt & 1u;
        if (mbar_test_wait(bar(kBarQFree + qs), ((a_tt >> 1) & 1u) ^ 1u)) {
          const int mt = a_item - 1;
          const uint32_t q_base = smem_base + p.off_q + qs * (2u * kBoxBytes);
          const uint32_t qfull = bar(kBarQFull + qs);
          mbar_arrive_expect_tx(qfull, 2u * kBoxBytes);
#pragma unroll 1
          for (int b = 0; b < 2; ++b) {
            const int ui = sh.pair ? b : 0;
            const int r0 = sh.pair ? 0 : mt * kTileRows + b * kBoxRows;
            tma_load_4d(q_base + b * kBoxBytes, &p.tm_q, qfull, 0, r0, ui ? a_u.h1 : a_u.h0, ui ? a_u.bw1 : a_u.bw0);
          }
          ++a_tt;
          trace_ev(tr, 41);
          if (++a_item > sh.MT) {
            a_item = 0;
            a_kv.advance();
            a_job += gridDim.x;
            a_done = a_job >= p.n_jobs;
            a_u = job_units(a_job, kPair, sh.H, p.has_mask ? p.nW : 0);
          }
          progress = true;
        }
      }
    }
    if (!b_done) {
      const uint32_t st = b_ring.stage;
      if (mbar_test_wait(bar(kBarBmFree + st), b_ring.phase ^ 1u)) {
        const uint32_t base = smem_base + p.off_bm + st * (2u * kTableTileBytes);
        const uint32_t full = bar(kBarBmFull + st);
        mbar_arrive_expect_tx(full, table_bytes);
#pragma unroll 1
        for (int b = 0; b < 2; ++b) {
          const int ui = sh.pair ? b : 0;
          const int r0 = sh.pair ? 0 : b_mt * kTileRows + b * kBoxRows;
          const int c0 = sh.pair ? b_c2 * kChunkCols : b_s * kStepCols + b_c2 * kChunkCols;
          if (p.has_bias) tma_load_3d(base + b * kBoxBytes, &p.tm_bias, full, c0, r0, ui ? b_u.h1 : b_u.h0);
          if (p.has_mask)
            tma_load_3d(base + kTableTileBytes + b * kBoxBytes, &p.tm_mask, full, c0, r0, ui ? b_u.mw1 : b_u.mw0);
        }
        b_ring.advance();
        trace_ev(tr, 42);
        // advance (chunk, step, tile, job)
        const int ncols = sh.pair ? sh.N : min(kStepCols, sh.N - b_s * kStepCols);
        const int nch = ncols > kChunkCols ? 2 : 1;
        if (++b_c2 >= nch) {
          b_c2 = 0;
          if (++b_s >= sh.KS) {
            b_s = 0;
            if (++b_mt >= sh.MT) {
              b_mt = 0;
              b_job += gridDim.x;
              b_done = b_job >= p.n_jobs;
              b_u = job_units(b_job, kPair, sh.H, p.has_mask ? p.nW : 0);
            }
          }
        }
        progress = true;
      }
    }
    if (progress) {
      idle = 0;
    } else if ((++idle & 0x3Fu) != 0) {
      __nanosleep(20);
    } else {
      if (idle == 0x40u) t0 = clock64();
      if (*ctx.abort_flag) return;
      if (clock64() - t0 > kWaitLimitCycles) {
        *ctx.abort_flag = 1u;
        if (ctx.status != nullptr) {
          if (atomicCAS(&ctx.status->code, 0u, (30u << 8) | kStatusTimeout) == 0u) {
            ctx.status->block = blockIdx.x;
            ctx.status->detail = (static_cast<uint32_t>(a_item) << 16) | (b_ring.stage & 0xFFFFu);
          }
        }
        return;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
template <typename T, bool kPTmem, bool kPair>
__global__ void __launch_bounds__(kFwdThreads, 2) fwd_kernel(const __grid_constant__ FwdParams p) {
  // No static shared memory: the dynamic window then starts 1024-byte aligned, which the
  // swizzled tiles need; checked below.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t tid = threadIdx.x;
  const uint32_t warp = tid >> 5;
  const uint32_t lane = tid & 31u;
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t bars = smem_base + p.off_ctrl;
  uint32_t* ctrl_words = reinterpret_cast<uint32_t*>(smem_raw + p.off_ctrl + 8u * kFwdNumBars);
  uint32_t& tmem_slot = ctrl_words[0];
  volatile uint32_t& abort_flag = *reinterpret_cast<volatile uint32_t*>(&ctrl_words[1]);
  if ((smem_base & 1023u) != 0u) {
    if (tid == 0 && p.status != nullptr) atomicCAS(&p.status->code, 0u, (99u << 8) | 2u);
    return;
  }

  if (tid == 0) {
    abort_flag = 0u;
    for (int i = 0; i < kFwdNumBars; ++i) {
      uint32_t count = 1u;
      if ((i >= kBarKvReady && i < kBarKvFree) || (i >= kBarQReady && i < kBarQFree) ||
          (i >= kBarSFree && i < kBarBmFull) || (i >= kBarBmFree && i < kBarPFull) || i == kBarPFull)
        count = 128u;
      mbar_init(bars + 8u * i, count);
    }
    mbar_fence_init();
    tma_prefetch_desc(&p.tm_q);
    tma_prefetch_desc(&p.tm_k);
    tma_prefetch_desc(&p.tm_v);
    if (p.has_bias) tma_prefetch_desc(&p.tm_bias);
    if (p.has_mask) tma_prefetch_desc(&p.tm_mask);
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&tmem_slot), kFwdTmemCols);
    tmem_relinquish();
  }
  // per-head score multipliers, looked up from shared memory in the per-job path
  float* scale_tab = reinterpret_cast<float*>(smem_raw + p.off_ctrl + 256u);
  for (int hh = static_cast<int>(tid); hh < p.H; hh += kFwdThreads)
    scale_tab[hh] = load_scale<T>(p.scale, p.scale_is_tensor, hh);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  WaitCtx ctx{&ctrl_words[1], p.status, (p.trace.buf != nullptr && p.trace.cap >= 700) ? p.trace.buf + 2ll * p.trace.cap + 500 : nullptr};

  if (warp < 4) {
    fwd_softmax_role<T, kPTmem, kPair>(p, smem_base, bars, tmem, ctx, scale_tab);
  } else if (lane == 0) {
    if (warp == 4) fwd_mma_role<T, kPTmem, kPair>(p, smem_base, bars, tmem, ctx);
    else fwd_load_role<kPair>(p, smem_base, bars, ctx);
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (tid == 0) report_abort(ctrl_words[1], p.status);
  if (abort_flag) {
    // A wait ran out somewhere: give copies that may still be in flight time to land before the
    // shared memory is handed back.
    __nanosleep(20000);
    __syncthreads();
  }
  if (warp == 4) tmem_dealloc(tmem, kFwdTmemCols);
}

template __global__ void fwd_kernel<__nv_bfloat16, true, true>(const __grid_constant__ FwdParams);
template __global__ void fwd_kernel<__nv_bfloat16, true, false>(const __grid_constant__ FwdParams);
template __global__ void fwd_kernel<__nv_bfloat16, false, true>(const __grid_constant__ FwdParams);
template __global__ void fwd_kernel<__nv_bfloat16, false, false>(const __grid_constant__ FwdParams);
template __global__ void fwd_kernel<__half, true, true>(const __grid_constant__ FwdParams);
template __global__ void fwd_kernel<__half, true, false>(const __grid_constant__ FwdParams);
template __global__ void fwd_kernel<__half, false, true>(const __grid_constant__ FwdParams);
template __global__ void fwd_kernel<__half, false, false>(const __grid_constant__ FwdParams);

cudaError_t launch_fwd(const FwdParams& p, int dtype_is_bf16, int p_in_tmem, int grid,
                       cudaStream_t stream) {
  auto go = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(p.smem_bytes));
    if (e != cudaSuccess) return e;
    kern<<<grid, kFwdThreads, p.smem_bytes, stream>>>(p);
    return cudaGetLastError();
  };
  auto by_mode = [&](auto pair_tag) -> cudaError_t {
    constexpr bool kPair = decltype(pair_tag)::value;
    if (dtype_is_bf16) {
      return p_in_tmem ? go(fwd_kernel<__nv_bfloat16, true, kPair>) : go(fwd_kernel<__nv_bfloat16, false, kPair>);
    }
    return p_in_tmem ? go(fwd_kernel<__half, true, kPair>) : go(fwd_kernel<__half, false, kPair>);
  };
  return p.pair_mode ? by_mode(std::true_type{}) : by_mode(std::false_type{});
}

}  // namespace fwa2
