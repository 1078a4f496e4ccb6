// Forward kernel for windows of 129 to 256 tokens: the two 128-row tiles of a unit are worked on
// at the same time by two softmax warpgroups that share the unit's K and V in shared memory.
//
// One persistent CTA (two per SM) handles a sequence of units.  Roles:
//   warps 0-3   softmax of tile 0: thread t owns query row t
//   warps 4-7   softmax of tile 1: thread t owns query row 128 + t
//   warp  8, 9  issue the tcgen05.mma of tile 0 / tile 1 (one thread each)
//   warp  10    TMA producer (one thread): K, Q, V and the bias / mask table chunks
// A step is 32 keys.  Per warpgroup, tensor memory holds one 32-column score buffer, the packed
// probabilities and the running output.  A step is a single pass: the 32 scores of the row are
// read into registers (which frees the score buffer for the next step's product at once), scaled,
// biased and masked two at a time (fma / add .f32x2), and exponentiated against a reference
// maximum that is only raised when the row maximum has outgrown it by a factor e^8; the running output
// stays in tensor memory and is rescaled there on those occasions only.
//
// The code is written to be SMALL: an SM runs straight-line code at full speed only out of its
// 32 KiB instruction cache, and here four softmax warpgroups, four issuers and two producers per
// SM execute their loops at the same time.  Hence the short step, one copy of every role (the two
// issuers run the same code; the job loop is rotated so that the normalisation and the epilogue
// appear once), compact waits, and kernel instantiations per table combination instead of
// run-time branches in the step.
// Replaces flash_win_attn_v2/kernels/attn_kernel_forward.py:21-258 (`_fwd_kernel`) for these sizes.
#define FWA2_NORMALISE_ROLLED 0
#define FWA2_WAIT_INLINE 1
#include "fwa2_common.cuh"

namespace fwa2 {

constexpr int kDuoThreads = 384;
constexpr int kDuoStep = 32;             // keys per step = columns of a table chunk
constexpr uint32_t kDuoTmemCols = 256;   // 128 per warpgroup (80 used)
constexpr uint32_t kDuoTmS = 0;          // 32 columns: scores of one step
constexpr uint32_t kDuoTmO = 32;         // 32 columns: running output
constexpr uint32_t kDuoTmP = 64;         // 16 columns: 32 probabilities, 16 bit, two per column
constexpr uint32_t kDuoTableStageBytes = 2u * kTableTileBytes;
// The reference maximum of a row is raised when the row maximum exceeds it by more than this
// (natural-log units; e^8 < 2^12, far inside the range of fp16 probabilities and fp32 sums).
constexpr float kDuoRaise = 8.0f;

// Register budgets after setmaxnreg; the CTA is launched with 384 x 80.
constexpr uint32_t kDuoRegSoftmax = 96, kDuoRegOther = 48;
static_assert(256u * kDuoRegSoftmax + 128u * kDuoRegOther <= 384u * 80u, "register pool of the CTA");

enum DuoBar : int {
  dbKFull = 0, dbKReady = 1, dbKFree = 2,
  dbQFull = 3, dbQReady = 4 /* +wg */, dbQFree = 6,
  dbVFull = 7 /* +stage */, dbVFree = 9 /* +stage */,
  dbSFull = 11 /* +wg */, dbSFree = 13 /* +wg */,
  dbPFull = 15 /* +wg */, dbPvDone = 17 /* +wg */,
  dbTFull = 19 /* +stage */, dbTFree = 23 /* +stage */,
  kDuoNumBars = 27
};

// Position in the ring of table chunks.  The chunks are queued in the order (step, tile); a
// softmax warpgroup therefore moves two entries at a time and the producer one.
struct TableRing {
  uint32_t stage, phase, n_stages;   // 3 or 4 stages
  __device__ __forceinline__ void advance(uint32_t n) {
    stage += n;
    if (stage >= n_stages) {
      stage -= n_stages;
      phase ^= 1u;
    }
  }
};

#if FWA2_TRACE
#define DPROF_BEGIN() long long dprof_t = clock64()
#define DPROF_SEG(idx)                                                                              \
  do {                                                                                              \
    const long long dprof_n = clock64();                                                            \
    if (ctx.wait_acc != nullptr && blockIdx.x == 0 && threadIdx.x == 0)                             \
      atomicAdd(ctx.wait_acc + 150 + (idx), static_cast<unsigned long long>(dprof_n - dprof_t));    \
    dprof_t = dprof_n;                                                                              \
  } while (0)
#else
#define DPROF_BEGIN() do {} while (0)
#define DPROF_SEG(idx) do {} while (0)
#endif

// Bounded wait, written to be small (it is inlined at every site).  try_wait parks the thread until
// the phase completes or its time hint runs out, so the loop body runs rarely; the clock and the
// abort word are looked at every 256 trips.  Returns false once the wait was abandoned; the CTA's
// abort word then holds (site << 8 | kind).
__device__ __forceinline__ bool dwait(uint32_t bar, uint32_t parity, const WaitCtx& ctx, uint32_t site) {
#if FWA2_TRACE
  return mbar_wait(bar, parity, ctx, site);
#else
  uint32_t spins = 0, t0 = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xFFu) == 0u) {
      const uint32_t now = static_cast<uint32_t>(clock());
      if (spins == 0x100u) t0 = now;
      if (*ctx.abort_flag != 0u || now - t0 > static_cast<uint32_t>(kWaitLimitCycles)) {
        if (*ctx.abort_flag == 0u) *ctx.abort_flag = (site << 8) | kStatusTimeout;
        return false;
      }
    }
  }
  return true;
#endif
}

// The same for a whole warp that goes on to a warp-collective instruction (tcgen05.ld / st /
// wait are .sync.aligned): lanes may leave the polling loop on different trips, and nothing else
// brings them back together before the collective.
__device__ __forceinline__ bool dwait_warp(uint32_t bar, uint32_t parity, const WaitCtx& ctx, uint32_t site) {
  const bool ok = dwait(bar, parity, ctx, site);
#ifndef DUO_NO_WARPSYNC
  __syncwarp();
#endif
  return ok;
}

__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* m, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

// ------------------------------------------------------------------------------------------------
// Softmax warpgroups
// ------------------------------------------------------------------------------------------------
template <typename T, bool kBias, bool kMask, bool kComb>
__device__ __forceinline__ void duo_softmax_role(const FwdParams& p, uint32_t smem_base, uint32_t bars,
                                                 uint32_t tmem, const WaitCtx& ctx, const float* scale_tab) {
  constexpr bool kTable = kBias || kMask;
  const uint32_t tid = threadIdx.x;            // 0..255: K row to normalise, Q row of the unit
  const uint32_t wg = tid >> 7, t = tid & 127u;
  const uint32_t tm = tmem + ((((tid >> 5) & 3u) * 32u) << 16) + wg * 128u;
  const int N = p.N, H = p.H;
  const int KS = (N + kDuoStep - 1) / kDuoStep;
  const uint32_t rows_kv = static_cast<uint32_t>((N + 63) / 64) * 64u;
  const uint32_t bar_s_full = bars + 8u * (dbSFull + wg), bar_s_free = bars + 8u * (dbSFree + wg);
  const uint32_t bar_p_full = bars + 8u * (dbPFull + wg), bar_pv = bars + 8u * (dbPvDone + wg);
  // where thread t finds its row of a table chunk: rows of 64 bytes (64-byte swizzle) per 16-bit
  // table, rows of 128 bytes (128-byte swizzle) in the combined fp32 table
  const uint32_t row_off = kComb ? t * 128u : t * 64u, row_sw = kComb ? (t & 7u) : ((t >> 1) & 3u);
  const float2 log2e2 = make_float2(kLog2e, kLog2e);

  TableRing ring{wg, 0u, static_cast<uint32_t>(p.n_bm_stages)};
  uint32_t jc = 0, sc = 0;       // units and steps done by this thread
  // The loop is rotated so that every piece of code exists once: a trip normalises K and Q of its
  // unit, THEN finishes the previous unit (whose last P*V has been running meanwhile), then runs
  // the steps of its unit.
  int job = blockIdx.x, prev_bw = 0, prev_h = 0;
  bool have_prev = false;
  float m_ref = 0.f, l_run = 0.f;
  DPROF_BEGIN();

#pragma unroll 1
  while (true) {
    const bool have_job = job < p.n_jobs;
    if (have_job) {
      // ---- K row `tid` and Q row `tid` of this unit, normalised in place ----
#pragma unroll 1
      for (uint32_t what = 0; what < 2u; ++what) {
        if (!dwait_warp(bars + 8u * (what == 0u ? dbKFull : dbQFull), jc & 1u, ctx, 10u + what)) return;
        if (what == 1u || tid < rows_kv) normalise_row<T>(smem_base + (what == 0u ? p.off_kv : p.off_q), tid);
        fence_proxy_async_smem();
        mbar_arrive(bars + 8u * (what == 0u ? static_cast<uint32_t>(dbKReady) : dbQReady + wg));
      }
    }
    DPROF_SEG(6);
    if (have_prev) {
      // ---- epilogue of the previous unit ----
      if (!dwait_warp(bar_pv, (sc - 1u) & 1u, ctx, 16)) return;
      tc_fence_after();
      uint32_t o[32];
      tmem_ld32(tm + kDuoTmO, o);
      tmem_wait_ld();
      tc_fence_before();
      const int row = static_cast<int>(tid);
      if (row < N) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint16_t* dst = static_cast<uint16_t*>(p.o) + prev_bw * p.o_sbw + prev_h * p.o_sh + row * p.o_sn;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint4 v;
          v.x = Elem<T>::pack(__uint_as_float(o[ch * 8 + 0]) * inv, __uint_as_float(o[ch * 8 + 1]) * inv);
          v.y = Elem<T>::pack(__uint_as_float(o[ch * 8 + 2]) * inv, __uint_as_float(o[ch * 8 + 3]) * inv);
          v.z = Elem<T>::pack(__uint_as_float(o[ch * 8 + 4]) * inv, __uint_as_float(o[ch * 8 + 5]) * inv);
          v.w = Elem<T>::pack(__uint_as_float(o[ch * 8 + 6]) * inv, __uint_as_float(o[ch * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(dst + ch * 8) = v;
        }
        p.lse[prev_bw * p.lse_sbw + prev_h * p.lse_sh + row] = l_run > 0.f ? m_ref + __logf(l_run) : -INFINITY;
      }
    }
    DPROF_SEG(7);
    if (!have_job) break;
    int bw, h;
    if constexpr (kComb) {
      const int plane = job / p.n_img, wt = plane / H;
      h = plane - wt * H;
      bw = (job - plane * p.n_img) * p.nW + wt;
    } else {
      bw = job / H;
      h = job - bw * H;
    }
    const float scale = scale_tab[h];
    const float2 scale2 = make_float2(scale, scale);
    m_ref = 0.f;
    l_run = 0.f;

#pragma unroll 1
    for (int s = 0; s < KS; ++s, ++sc) {
      DPROF_SEG(0);
      if (!dwait_warp(bar_s_full, sc & 1u, ctx, 12)) return;
      tc_fence_after();
      DPROF_SEG(1);
      uint32_t r[32];
      tmem_ld32(tm + kDuoTmS, r);
      // (the table words are fetched while the tensor-memory load is in flight)
      uint32_t wb[4][4], wm[4][4];   // 16-bit tables: 8 columns per 16 bytes
      uint32_t wc[8][4];             // combined fp32 table: 4 columns per 16 bytes
      if constexpr (kTable) {
        const uint32_t base = smem_base + p.off_bm + ring.stage * kDuoTableStageBytes + row_off;
        if (!dwait_warp(bars + 8u * (dbTFull + ring.stage), ring.phase, ctx, 13)) return;
        if constexpr (kComb) {
#pragma unroll
          for (uint32_t ch = 0; ch < 8u; ++ch) lds128(base + ((ch ^ row_sw) << 4), wc[ch]);
        } else {
#pragma unroll
          for (uint32_t ch = 0; ch < 4u; ++ch) {
            const uint32_t off = base + ((ch ^ row_sw) << 4);
            if constexpr (kBias) lds128(off, wb[ch]);
            if constexpr (kMask) lds128(off + kTableTileBytes, wm[ch]);
          }
        }
      }
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar_s_free);   // the next step's product may overwrite the scores
      DPROF_SEG(2);

      // ---- x = scale * cos + bias + mask ----
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        float2 x2 = make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1]));
        if constexpr (kComb) {
          x2 = __ffma2_rn(x2, scale2, make_float2(__uint_as_float(wc[e >> 2][e & 3]),
                                                  __uint_as_float(wc[e >> 2][(e & 3) + 1])));
        } else if constexpr (kBias) {
          const uint32_t wv = wb[e >> 3][(e >> 1) & 3];
          x2 = __ffma2_rn(x2, scale2, make_float2(Elem<T>::lo(wv), Elem<T>::hi(wv)));
        } else {
          x2 = __fmul2_rn(x2, scale2);
        }
        if constexpr (kMask && !kComb) {
          const uint32_t wv = wm[e >> 3][(e >> 1) & 3];
          x2 = __fadd2_rn(x2, make_float2(Elem<T>::lo(wv), Elem<T>::hi(wv)));
        }
        r[e] = __float_as_uint(x2.x);
        r[e + 1] = __float_as_uint(x2.y);
      }
      {
        const int ncols = N - s * kDuoStep;
        if (ncols < kDuoStep) {   // keys past the end of the window
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (e >= ncols) r[e] = __float_as_uint(-INFINITY);
        }
      }
      DPROF_SEG(3);
      // ---- row maximum; the reference is raised only when the maximum has outgrown it ----
      float mxp[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 32; e += 2)
        mxp[(e >> 1) & 3] = max3f(mxp[(e >> 1) & 3], __uint_as_float(r[e]), __uint_as_float(r[e + 1]));
      const float mx = fmaxf(fmaxf(mxp[0], mxp[1]), fmaxf(mxp[2], mxp[3]));
      float alpha = 1.f;
      if (l_run == 0.f || mx > m_ref + kDuoRaise) {
        const float m_new = (mx == -INFINITY) ? 0.f : mx;
        if (l_run != 0.f) alpha = ex2f((m_ref - m_new) * kLog2e);
        m_ref = m_new;
        l_run *= alpha;
      }
      // ---- p = exp(x - reference), row sum ----
      uint32_t w[16];
      {
        const float nml2 = -m_ref * kLog2e;
        const float2 n2 = make_float2(nml2, nml2);
        float2 sum = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 y = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), log2e2, n2);
          const float2 pp = make_float2(ex2f(y.x), ex2f(y.y));
          sum = __fadd2_rn(sum, pp);
          w[i] = Elem<T>::pack(pp.x, pp.y);
        }
        l_run += sum.x + sum.y;
      }
      DPROF_SEG(4);

      // ---- the previous step's P*V is done: P may be overwritten, the output rescaled ----
      if (s > 0) {
        if (!dwait_warp(bar_pv, (sc - 1u) & 1u, ctx, 15)) return;
        tc_fence_after();
        if (__any_sync(0xFFFFFFFFu, alpha != 1.f)) {
          uint32_t o[32];
          tmem_ld32(tm + kDuoTmO, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st16(tm + kDuoTmO, reinterpret_cast<const uint32_t(&)[16]>(o[0]));
          tmem_st16(tm + kDuoTmO + 16u, reinterpret_cast<const uint32_t(&)[16]>(o[16]));
        }
      }
      tmem_st16(tm + kDuoTmP, w);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p_full);
      // The table stage is handed back only here.  Nothing but the arithmetic ties the table words
      // to program order, and arithmetic may be scheduled after a barrier arrival that does not
      // depend on it: an arrival placed right after the loads has let the producer overwrite the
      // stage while a warp's loads were still outstanding.  Behind the wait for the store of P,
      // which was computed from every one of those words, the loads are certainly complete.
      if constexpr (kTable) {
        mbar_arrive(bars + 8u * (dbTFree + ring.stage));
        ring.advance(2u);
      }
      DPROF_SEG(5);
    }

    prev_bw = bw;
    prev_h = h;
    have_prev = true;
    job += gridDim.x;
    ++jc;
  }
}

// ------------------------------------------------------------------------------------------------
// MMA issuer of one tile (one thread); both issuers run this one copy of the code.
// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void duo_mma_role(const FwdParams& p, uint32_t smem_base, uint32_t bars,
                                             uint32_t tmem, const WaitCtx& ctx, uint32_t wg) {
  constexpr uint32_t fmt = Elem<T>::kFmt;
  const int N = p.N;
  const int KS = (N + kDuoStep - 1) / kDuoStep;
  const uint32_t rows_kv = static_cast<uint32_t>((N + 63) / 64) * 64u;
  const uint32_t idesc_pv = make_idesc(fmt, 128, 32, 0, 1);
  const uint32_t idesc_s_full = make_idesc(fmt, 128, static_cast<uint32_t>(kDuoStep), 0, 0);
  const int last_cols = ((N - (KS - 1) * kDuoStep + 15) / 16) * 16;
  const uint32_t idesc_s_last = make_idesc(fmt, 128, static_cast<uint32_t>(last_cols), 0, 0);
  const DescBase d64 = make_desc_base(0, 16, 512, kSw64);      // K-major rows of 64 bytes
  const DescBase dv64 = make_desc_base(0, 512, 512, kSw64);    // MN-major rows of 64 bytes
  const uint32_t tm = tmem + wg * 128u;
  const uint32_t k_base = smem_base + p.off_kv;
  const uint32_t q_base = smem_base + p.off_q + wg * (2u * kBoxBytes);
  const uint32_t v_stage_bytes = rows_kv * kRowBytes;
  const uint32_t bar_s_full = bars + 8u * (dbSFull + wg), bar_s_free = bars + 8u * (dbSFree + wg);
  const uint32_t bar_p_full = bars + 8u * (dbPFull + wg), bar_pv = bars + 8u * (dbPvDone + wg);
  uint32_t jc = 0, sc = 0, pc = 0;
  Ring v_ring(static_cast<uint32_t>(p.n_kv_stages));

#pragma unroll 1
  for (int job = blockIdx.x; job < p.n_jobs; job += gridDim.x, ++jc, v_ring.advance()) {
    if (!dwait(bars + 8u * dbKReady, jc & 1u, ctx, 20)) return;
    if (!dwait(bars + 8u * (dbQReady + wg), jc & 1u, ctx, 21)) return;
    tc_fence_after();
    const uint32_t v_base = smem_base + p.off_p + v_ring.stage * v_stage_bytes;

    // trip `it` issues the scores of step `it` and then the P*V of step `it - 1`
#pragma unroll 1
    for (int it = 0; it <= KS; ++it) {
      if (it < KS) {
        // the softmax threads have taken the previous scores out of tensor memory
        if (!dwait(bar_s_free, (sc & 1u) ^ 1u, ctx, 22)) return;
        tc_fence_after();
        const uint32_t kb = k_base + static_cast<uint32_t>(it) * (kDuoStep * kRowBytes);
        const uint32_t idesc = (it == KS - 1) ? idesc_s_last : idesc_s_full;
        mma_ss(tm + kDuoTmS, desc_at(d64, q_base), desc_at(d64, kb), idesc, 0u);
        mma_ss(tm + kDuoTmS, desc_at(d64, q_base + 32u), desc_at(d64, kb + 32u), idesc, 1u);
        mma_commit(bar_s_full);
        ++sc;
        if (it == KS - 1) {   // every product that reads Q and K of this unit has been issued
          mma_commit(bars + 8u * dbQFree);
          mma_commit(bars + 8u * dbKFree);
        }
      }
      if (it > 0) {
        if (!dwait(bar_p_full, pc & 1u, ctx, 23)) return;
        if (it == 1) {
          if (!dwait(bars + 8u * (dbVFull + v_ring.stage), v_ring.phase, ctx, 24)) return;
        }
        tc_fence_after();
        const uint32_t vb = v_base + static_cast<uint32_t>(it - 1) * (kDuoStep * kRowBytes);
        mma_ts(tm + kDuoTmO, tm + kDuoTmP, desc_at(dv64, vb), idesc_pv, it > 1 ? 1u : 0u);
        mma_ts(tm + kDuoTmO, tm + kDuoTmP + 8u, desc_at(dv64, vb + 1024u), idesc_pv, 1u);
        mma_commit(bar_pv);
        ++pc;
      }
    }
    mma_commit(bars + 8u * (dbVFree + v_ring.stage));
  }
}

// ------------------------------------------------------------------------------------------------
// TMA producer (one thread).  Two queues are served without ever blocking on one of them:
// (a) V, K and Q of the units, (b) the table chunks.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void duo_load_role(const FwdParams& p, uint32_t smem_base, uint32_t bars,
                                              const WaitCtx& ctx) {
  const int N = p.N, H = p.H;
  const int KS = (N + kDuoStep - 1) / kDuoStep;
  const int nbox = (N + 63) / 64;                        // 64-row boxes of K and of V
  const uint32_t kv_bytes = static_cast<uint32_t>(nbox) * kBoxBytes;
  const bool any_table = p.has_bias || p.has_mask;
  const uint32_t table_bytes = (p.has_bias ? kTableTileBytes : 0u) + (p.has_mask ? kTableTileBytes : 0u);

  // queue (a): item 0 = K, 1 = Q, 2 = V -- the order in which their buffers come free
  int a_job = blockIdx.x, a_item = 0;
  uint32_t a_jc = 0;
  Ring a_v(static_cast<uint32_t>(p.n_kv_stages));
  // queue (b): entry e of a unit = (step e >> 1, tile e & 1)
  int b_job = blockIdx.x, b_e = 0;
  TableRing b_ring{0u, 0u, static_cast<uint32_t>(p.n_bm_stages)};
  bool a_done = a_job >= p.n_jobs, b_done = !any_table || b_job >= p.n_jobs;
  // unit of a job: (window, head); in combined-table order also the table plane
  auto unit_of = [&](int job, int& bw, int& h, int& plane) {
    if (p.comb) {
      plane = job / p.n_img;
      const int wt = plane / H;
      h = plane - wt * H;
      bw = (job - plane * p.n_img) * p.nW + wt;
    } else {
      bw = job / H;
      h = job - bw * H;
      plane = p.has_mask ? bw % p.nW : 0;   // the mask's window type
    }
  };
  int a_bw = 0, a_h = 0, a_plane = 0, b_bw = 0, b_h = 0, b_mw = 0;
  if (!a_done) unit_of(a_job, a_bw, a_h, a_plane);
  if (!b_done) unit_of(b_job, b_bw, b_h, b_mw);

  uint32_t idle = 0, t0 = 0;
#pragma unroll 1
  while (!a_done || !b_done) {
    bool progress = false;
    if (!a_done) {
      // what the item waits for, where it goes, which barrier it completes
      const uint32_t free_bar = bars + 8u * (a_item == 2 ? dbVFree + a_v.stage : (a_item == 0 ? dbKFree : dbQFree));
      const uint32_t free_par = (a_item == 2 ? a_v.phase : (a_jc & 1u)) ^ 1u;
      if (mbar_test_wait(free_bar, free_par)) {
        const uint32_t full = bars + 8u * (a_item == 2 ? dbVFull + a_v.stage : (a_item == 0 ? dbKFull : dbQFull));
        const uint32_t dst = smem_base + (a_item == 2 ? p.off_p + a_v.stage * kv_bytes : (a_item == 0 ? p.off_kv : p.off_q));
        const CUtensorMap* tm = a_item == 2 ? &p.tm_v : (a_item == 0 ? &p.tm_k : &p.tm_q);
        const int boxes = a_item == 1 ? 4 : nbox;
        mbar_arrive_expect_tx(full, static_cast<uint32_t>(boxes) * kBoxBytes);
#pragma unroll 1
        for (int b = 0; b < boxes; ++b) tma_load_4d(dst + b * kBoxBytes, tm, full, 0, b * kBoxRows, a_h, a_bw);
        if (a_item == 2) a_v.advance();
        if (++a_item == 3) {
          a_item = 0;
          ++a_jc;
          a_job += gridDim.x;
          a_done = a_job >= p.n_jobs;
          if (!a_done) {
            unit_of(a_job, a_bw, a_h, a_plane);
            // K, Q and V of the unit after this one: into L2 now, so that the loads that have to
            // wait for this unit's last products find them there
#pragma unroll 1
            for (int b = 0; b < nbox; ++b) {
              tma_prefetch_4d(&p.tm_k, 0, b * kBoxRows, a_h, a_bw);
              tma_prefetch_4d(&p.tm_q, 0, b * kBoxRows, a_h, a_bw);
              tma_prefetch_4d(&p.tm_v, 0, b * kBoxRows, a_h, a_bw);
            }
          }
        }
        progress = true;
      }
    }
    if (!b_done) {
      const uint32_t st = b_ring.stage;
      if (mbar_test_wait(bars + 8u * (dbTFree + st), b_ring.phase ^ 1u)) {
        const uint32_t base = smem_base + p.off_bm + st * kDuoTableStageBytes;
        const uint32_t full = bars + 8u * (dbTFull + st);
        const int c0 = (b_e >> 1) * kDuoStep;
        const int r0 = (b_e & 1) * kTileRows;
        mbar_arrive_expect_tx(full, table_bytes);
        if (p.comb) {
          tma_load_3d(base, &p.tm_bias, full, c0, r0, b_mw);   // one box of 128 rows x 32 fp32
        } else {
#pragma unroll 1
          for (int b = 0; b < 2; ++b) {
            if (p.has_bias) tma_load_3d(base + b * kBoxBytes, &p.tm_bias, full, c0, r0 + b * kBoxRows, b_h);
            if (p.has_mask)
              tma_load_3d(base + kTableTileBytes + b * kBoxBytes, &p.tm_mask, full, c0, r0 + b * kBoxRows, b_mw);
          }
        }
        b_ring.advance(1u);
        if (++b_e >= 2 * KS) {
          b_e = 0;
          b_job += gridDim.x;
          b_done = b_job >= p.n_jobs;
          if (!b_done) unit_of(b_job, b_bw, b_h, b_mw);
        }
        progress = true;
      }
    }
    if (progress) {
      idle = 0;
    } else if ((++idle & 0x3Fu) != 0u) {
      __nanosleep(20);
    } else {
      const uint32_t now = static_cast<uint32_t>(clock());
      if (idle == 0x40u) t0 = now;
      if (*ctx.abort_flag != 0u) return;
      if (now - t0 > static_cast<uint32_t>(kWaitLimitCycles)) {
        *ctx.abort_flag = (30u << 8) | kStatusTimeout;
        return;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
template <typename T, bool kBias, bool kMask, bool kComb>
__global__ void __launch_bounds__(kDuoThreads, 2) fwd_duo_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t tid = threadIdx.x;
  const uint32_t warp = tid >> 5;
  const uint32_t lane = tid & 31u;
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t bars = smem_base + p.off_ctrl;
  uint32_t* ctrl_words = reinterpret_cast<uint32_t*>(smem_raw + p.off_ctrl + 8u * kDuoNumBars);
  uint32_t& tmem_slot = ctrl_words[0];
  volatile uint32_t& abort_flag = *reinterpret_cast<volatile uint32_t*>(&ctrl_words[1]);
  if ((smem_base & 1023u) != 0u) {
    if (tid == 0 && p.status != nullptr) atomicCAS(&p.status->code, 0u, (99u << 8) | 2u);
    return;
  }

  if (tid == 0) {
    abort_flag = 0u;
    for (int i = 0; i < kDuoNumBars; ++i) {
      uint32_t count = 1u;                                   // TMA (expect_tx) or one commit
      if (i == dbKReady) count = 256u;
      else if (i == dbKFree || i == dbQFree || (i >= dbVFree && i < dbSFull)) count = 2u;   // both issuers
      else if ((i >= dbQReady && i < dbQFree) || (i >= dbSFree && i < dbPvDone) || i >= dbTFree) count = 128u;
      mbar_init(bars + 8u * i, count);
    }
    mbar_fence_init();
    tma_prefetch_desc(&p.tm_q);
    tma_prefetch_desc(&p.tm_k);
    tma_prefetch_desc(&p.tm_v);
    if (kBias) tma_prefetch_desc(&p.tm_bias);
    if (kMask && !kComb) tma_prefetch_desc(&p.tm_mask);
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(&tmem_slot), kDuoTmemCols);
    tmem_relinquish();
  }
  float* scale_tab = reinterpret_cast<float*>(smem_raw + p.off_ctrl + 256u);
  for (int hh = static_cast<int>(tid); hh < p.H; hh += kDuoThreads)
    scale_tab[hh] = load_scale<T>(p.scale, p.scale_is_tensor, hh);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  WaitCtx ctx{&ctrl_words[1], p.status,
              (p.trace.buf != nullptr && p.trace.cap >= 700) ? p.trace.buf + 2ll * p.trace.cap + 500 : nullptr};

  if (warp < 8) {
    reg_alloc<kDuoRegSoftmax>();
    duo_softmax_role<T, kBias, kMask, kComb>(p, smem_base, bars, tmem, ctx, scale_tab);
  } else {
    reg_dealloc<kDuoRegOther>();
    if (lane == 0) {
      if (warp <= 9) duo_mma_role<T>(p, smem_base, bars, tmem, ctx, warp - 8u);
      else if (warp == 10) duo_load_role(p, smem_base, bars, ctx);
    }
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0) report_abort(ctrl_words[1], p.status);
  if (abort_flag) {
    // A wait ran out somewhere: give copies that may still be in flight time to land before the
    // shared memory is handed back.
    __nanosleep(20000);
    __syncthreads();
  }
  if (warp == 8) tmem_dealloc(tmem, kDuoTmemCols);
}

// ------------------------------------------------------------------------------------------------
// out[(wt * H + h)][i][j] = float(bias[h][i][j]) + float(mask[wt][i][j]), fp32, rows of `pitch`
// floats (columns from N on are written as zero).  One thread per 8 columns, 32 threads per row,
// 8 rows per CTA.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) combine_tables_kernel(const uint16_t* __restrict__ bias, long long bias_pitch,
                                                             const uint16_t* __restrict__ mask, long long mask_pitch,
                                                             float* __restrict__ out, int N, int H, int pitch) {
  const int plane = blockIdx.y, wt = plane / H, h = plane - wt * H;
  const int row = blockIdx.x * 8 + static_cast<int>(threadIdx.x >> 5);
  const int col = static_cast<int>(threadIdx.x & 31u) * 8;
  if (row >= N || col >= pitch) return;
  float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
  if (col < N) {   // the tables' rows are padded to multiples of 8 elements: the 16 bytes exist
    const uint4 b = *reinterpret_cast<const uint4*>(bias + (static_cast<long long>(h) * N + row) * bias_pitch + col);
    const uint4 m = *reinterpret_cast<const uint4*>(mask + (static_cast<long long>(wt) * N + row) * mask_pitch + col);
    lo = make_float4(Elem<T>::lo(b.x) + Elem<T>::lo(m.x), Elem<T>::hi(b.x) + Elem<T>::hi(m.x),
                     Elem<T>::lo(b.y) + Elem<T>::lo(m.y), Elem<T>::hi(b.y) + Elem<T>::hi(m.y));
    hi = make_float4(Elem<T>::lo(b.z) + Elem<T>::lo(m.z), Elem<T>::hi(b.z) + Elem<T>::hi(m.z),
                     Elem<T>::lo(b.w) + Elem<T>::lo(m.w), Elem<T>::hi(b.w) + Elem<T>::hi(m.w));
    if (col + 8 > N) {   // the tail of the last group of a row
      float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (col + i >= N) v[i] = 0.f;
      lo = make_float4(v[0], v[1], v[2], v[3]);
      hi = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
  float* dst = out + (static_cast<long long>(plane) * N + row) * pitch + col;
  *reinterpret_cast<float4*>(dst) = lo;
  *reinterpret_cast<float4*>(dst + 4) = hi;
}

cudaError_t launch_combine_tables(const void* bias, long long bias_pitch, const void* mask, long long mask_pitch,
                                  float* out, int n, int heads, int n_windows, int pitch, int dtype_is_bf16,
                                  cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>((n + 7) / 8), static_cast<unsigned>(n_windows * heads));
  const uint16_t* b = static_cast<const uint16_t*>(bias);
  const uint16_t* m = static_cast<const uint16_t*>(mask);
  if (dtype_is_bf16)
    combine_tables_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(b, bias_pitch, m, mask_pitch, out, n, heads, pitch);
  else
    combine_tables_kernel<__half><<<grid, 256, 0, stream>>>(b, bias_pitch, m, mask_pitch, out, n, heads, pitch);
  return cudaGetLastError();
}

cudaError_t launch_fwd_duo(const FwdParams& p, int dtype_is_bf16, int grid, cudaStream_t stream) {
  auto go = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(p.smem_bytes));
    if (e != cudaSuccess) return e;
    kern<<<grid, kDuoThreads, p.smem_bytes, stream>>>(p);
    return cudaGetLastError();
  };
  auto by_tables = [&](auto type_tag) -> cudaError_t {
    using T = decltype(type_tag);
    if (p.comb) return go(fwd_duo_kernel<T, true, true, true>);
    if (p.has_bias)
      return p.has_mask ? go(fwd_duo_kernel<T, true, true, false>) : go(fwd_duo_kernel<T, true, false, false>);
    return p.has_mask ? go(fwd_duo_kernel<T, false, true, false>) : go(fwd_duo_kernel<T, false, false, false>);
  };
  return dtype_is_bf16 ? by_tables(__nv_bfloat16{}) : by_tables(__half{});
}

}  // namespace fwa2
