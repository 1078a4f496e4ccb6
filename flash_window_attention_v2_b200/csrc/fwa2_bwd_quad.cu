// Backward kernel for windows of 65 to 256 tokens.
//
// The N x N score matrix of a (window, head) unit is cut into 128 x 128 tiles: key block a, query
// tile b.  A thread-block cluster of four CTAs (one CTA for windows of at most 128 tokens) works
// on one unit at a time, CTA rank 2 a + b on tile (a, b), and every cluster keeps to one head.
// What that buys:
//   * the window-summed dBias tile of the CTA never leaves tensor memory: the tensor core adds
//     every window's dS^T into it (dB^T += dS^T I) and it is written out once, at the end;
//   * the CTA's tile of the bias table is loaded once and stays in shared memory;
//   * every job of a CTA is the same short pipeline (two 64-query steps, five products).
// What it costs: dV and dK of a key block are sums over the two query tiles, dQ of a query tile
// over the two key blocks.  Each of those sums has exactly two terms, held by two CTAs of the
// cluster; the two CTAs split the 128 rows between them, push the 64 rows they do not keep into
// the other's shared memory (st.shared::cluster), and finish the rows they keep.  A sum of two
// floats does not depend on the order, so the result is bitwise reproducible.
//
// As in the other backward kernel everything is computed transposed (keys on the tensor-memory
// lanes): S^T = K^ Q^^T, dP^T = V dO^T, P^T and dS^T written back over them as packed 16-bit
// pairs and used as tensor-memory A operands of dV += P^T dO, dK^ += dS^T Q^, dB^T += dS^T I; dS
// also goes through shared memory for dQ^ += dS K^.
//
// Roles (640 threads): warps 0-3 / 4-7 compute warpgroups (step 0 / 1 of the tile, thread = key),
// warps 8-11 epilogue warpgroup (exchange and epilogues of dV and dK, one job behind), warps 12-15
// preparing warpgroup (normalises K and Q rows in place, delta, lse, up to two jobs ahead; in its
// idle time the exchange and epilogue of dQ), warp 16 issues every tcgen05.mma, warp 17 is the TMA
// producer.
// Replaces flash_win_attn_v2/kernels/attn_kernel_backward.py:6-51 and :84-564 for these sizes.
#define FWA2_NORMALISE_ROLLED 1
#define FWA2_WAIT_INLINE 1
#include "fwa2_common.cuh"

#include <cuda_runtime.h>

#include <type_traits>

namespace fwa2 {

constexpr int kQuadThreads = 640;
constexpr uint32_t kQuadTmemCols = 512;
// Tensor-memory columns.  Step w: S^T at 128 w, dP^T at 128 w + 64 (64 queries each).
constexpr uint32_t kQTmS = 0, kQTmDP = 64;
constexpr uint32_t kQTmDV = 256, kQTmDK = 288, kQTmDQ = 320;
constexpr uint32_t kQTmDB = 384;            // dB^T of the tile: 128 query columns (chunk c at 32 c)
constexpr uint32_t kQStageBytes = 32768u;   // [K | V | Q | dO], 128 rows x 64 bytes each
constexpr uint32_t kQTableBytes = 32768u;   // four chunks of (128 keys x 32 queries)
constexpr uint32_t kQRecvPart = 64u * 128u; // 64 rows x 32 fp32 of one pushed accumulator

enum QuadBar : int {
  qbFull = 0, qbReady = 3, qbFree = 6,        // per stage (up to three)
  qbMaskFull = 9, qbMaskFree = 11,            // per mask stage (two)
  qbBiasFull = 13,
  qbSFull = 14, qbPReady = 16,                // per step
  qbAccFull = 18, qbAccFree = 19,
  qbRecvFull = 20, qbRecvFree = 23,           // per pushed accumulator: 0 dV, 1 dK, 2 dQ
  qbDsFree = 26, qbAccFreeQ = 27,
  kQuadNumBars = 28
};

struct QuadGeom {
  int h, slot, count;
  uint32_t rank, a, b;
};
__device__ __forceinline__ QuadGeom quad_geom(const QuadParams& p, uint32_t rank) {
  QuadGeom g;
  const int cid = static_cast<int>(blockIdx.x) / p.cluster;
  g.h = cid % p.H;
  g.slot = cid / p.H;
  g.count = g.slot < p.BW ? (p.BW - g.slot + p.nslots - 1) / p.nslots : 0;
  g.rank = rank;
  g.a = rank >> 1;
  g.b = rank & 1u;
  return g;
}

// Bounded wait, written to be small: it is inlined at sixteen sites of a kernel whose roles must
// share a 32 KiB instruction cache.  kCluster: the phase is completed by a peer CTA (acquire at
// cluster scope).  Returns false once the wait was abandoned; the CTA's abort word then holds
// (site << 8 | kind).  The clock and the abort word are looked at every 4096 polls.
template <bool kCluster = false>
__device__ __forceinline__ bool qwait(uint32_t bar, uint32_t parity, const WaitCtx& ctx, uint32_t site) {
#if FWA2_TRACE
  return kCluster ? mbar_wait_cluster(bar, parity, ctx, site) : mbar_wait(bar, parity, ctx, site);
#else
  uint32_t spins = 0, t0 = 0;
  while (!(kCluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity))) {
    if ((++spins & 0xFFFu) == 0u) {
      const uint32_t now = static_cast<uint32_t>(clock());
      if (spins == 0x1000u) t0 = now;
      if (*ctx.abort_flag != 0u || now - t0 > static_cast<uint32_t>(kWaitLimitCycles)) {
        if (*ctx.abort_flag == 0u) *ctx.abort_flag = (site << 8) | kStatusTimeout;
        return false;
      }
    }
  }
  return true;
#endif
}

#if FWA2_TRACE
#define QPROF_BEGIN() long long qprof_t = clock64()
#define QPROF_SEG(idx)                                                                              \
  do {                                                                                              \
    const long long qprof_n = clock64();                                                            \
    if (p.prof != nullptr && blockIdx.x == 0 && (threadIdx.x & 31u) == 0u && ((threadIdx.x >> 5) & 3u) == 0u) \
      atomicAdd(p.prof + 200 + (idx), static_cast<unsigned long long>(qprof_n - qprof_t));        \
    qprof_t = qprof_n;                                                                              \
  } while (0)
#else
#define QPROF_BEGIN() do {} while (0)
#define QPROF_SEG(idx) do {} while (0)
#endif

__device__ __forceinline__ uint4 quad_ldg_v4(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

// ------------------------------------------------------------------------------------------------
// Eight queries of one key (= one thread):
//   x = scale * cos + bias + mask,  p = exp2(x log2e - lse2),  ds = p (dP - delta).
// Keys and queries past the end of the window need no special case.  Their rows of K, V, Q and dO
// were zero-filled by the TMA loads and the tables read as zero there, so every value stays
// finite; a query past the end has lse2 = +inf, hence p = ds = 0; a key past the end only feeds
// rows of dK / dV / dB that are never stored, and its row of K^ is zero in the dQ product.
// ------------------------------------------------------------------------------------------------
// Sixteen queries at a time, two per instruction where the hardware has paired fp32 forms
// (fma / add / mul .f32x2).  nl2 = -lse * log2(e) and nd = -delta come from shared memory with
// their signs already flipped, so that both subtractions are additions.
template <typename T>
__device__ __forceinline__ void quad_half(const uint32_t (&sv)[16], const uint32_t (&dpv)[16],
                                          const uint32_t* wb /* 8 words */, bool has_mask, uint32_t mask_addr0,
                                          uint32_t mask_addr1, const float* nl2, const float* nd, float scale,
                                          uint32_t (&pw)[8], uint32_t (&dw)[8]) {
  uint32_t wm[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
  if (has_mask) {
    lds128(mask_addr0, reinterpret_cast<uint32_t(&)[4]>(wm[0]));
    lds128(mask_addr1, reinterpret_cast<uint32_t(&)[4]>(wm[4]));
  }
  const float2 scale2 = make_float2(scale, scale), log2e2 = make_float2(kLog2e, kLog2e);
#pragma unroll
  for (int g4 = 0; g4 < 4; ++g4) {
    const float4 l4 = *reinterpret_cast<const float4*>(nl2 + 4 * g4);
    const float4 d4 = *reinterpret_cast<const float4*>(nd + 4 * g4);
#pragma unroll
    for (int hp = 0; hp < 2; ++hp) {
      const int e2 = 2 * g4 + hp, e = 2 * e2;
      const float2 s2 = make_float2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1]));
      const float2 b2 = make_float2(Elem<T>::lo(wb[e2]), Elem<T>::hi(wb[e2]));
      const float2 m2 = make_float2(Elem<T>::lo(wm[e2]), Elem<T>::hi(wm[e2]));
      const float2 l2 = hp == 0 ? make_float2(l4.x, l4.y) : make_float2(l4.z, l4.w);
      const float2 n2 = hp == 0 ? make_float2(d4.x, d4.y) : make_float2(d4.z, d4.w);
      float2 x2 = __ffma2_rn(s2, scale2, b2);
      if (has_mask) x2 = __fadd2_rn(x2, m2);
      const float2 y2 = __ffma2_rn(x2, log2e2, l2);
      const float2 p2 = make_float2(ex2f(y2.x), ex2f(y2.y));
      const float2 t2 = __fadd2_rn(make_float2(__uint_as_float(dpv[e]), __uint_as_float(dpv[e + 1])), n2);
      const float2 ds2 = __fmul2_rn(p2, t2);
      pw[e2] = Elem<T>::pack(p2.x, p2.y);
      dw[e2] = Elem<T>::pack(ds2.x, ds2.y);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// The two compute warpgroups: step w (64 queries) of every job's tile, back to back
// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ void quad_compute_role(const QuadParams& p, uint8_t* smem_ptr, uint32_t smem_base,
                                  uint32_t bars, uint32_t tmem, const WaitCtx& ctx, uint32_t rank) {
  const QuadGeom g = quad_geom(p, rank);
  if (g.count == 0) return;
  const uint32_t tid = threadIdx.x;
  const uint32_t wg = tid >> 7, lt = tid & 127u;
  const uint32_t lane_base = ((lt >> 5) * 32u) << 16;
  const float scale = load_scale<T>(p.scale, p.scale_is_tensor, g.h);
  auto bar = [&](int i) { return bars + 8u * i; };
  const float* rowstats = reinterpret_cast<const float*>(smem_ptr + p.off_rowstats);
  const uint32_t NS = p.n_stages, NM = p.n_mask_stages;
  const uint32_t ds_base = smem_base + p.off_ds + wg * 16384u + lt * 128u, ds_sw = lt & 7u;
  const uint32_t tab_row = lt * 64u, tab_sw = (lt >> 1) & 3u;
  const uint32_t tm_s = tmem + lane_base + wg * 128u + kQTmS;
  const uint32_t tm_d = tmem + lane_base + wg * 128u + kQTmDP;

  // This thread meets the same 64 bias entries in every job (its key, the 64 queries of its step,
  // the cluster's head): they live in registers for the whole kernel, as 32 packed pairs, read
  // once from the transposed table.
  uint32_t wb[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) wb[i] = 0u;
  if (p.has_bias) {
    const int key = static_cast<int>(g.a * kTileRows + lt);
    const int q0 = static_cast<int>(g.b * kTileRows + wg * kStepCols);
    if (key < p.N) {
      const uint16_t* src = static_cast<const uint16_t*>(p.bias_t) +
                            (static_cast<long long>(g.h) * p.N + key) * p.table_pitch + q0;
#pragma unroll
      for (int pc = 0; pc < 8; ++pc) {
        if (q0 + 8 * pc < p.table_pitch) {
          const uint4 v = quad_ldg_v4(src + 8 * pc);
          wb[4 * pc] = v.x; wb[4 * pc + 1] = v.y; wb[4 * pc + 2] = v.z; wb[4 * pc + 3] = v.w;
        }
      }
    }
  }

  if (p.db_partial != nullptr) {
    // the dB^T sums of my step's 64 query columns start from zero (the first product that adds to
    // them is issued after this warpgroup's first P^T barrier)
    uint32_t z[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) z[i] = 0u;
#pragma unroll
    for (uint32_t c = 0; c < 4u; ++c) tmem_st16(tmem + lane_base + kQTmDB + 64u * wg + 16u * c, z);
    tmem_wait_st();
    tc_fence_before();
  }

  Ring st(NS), mk(NM);
#pragma unroll 1
  for (int n = 0; n < g.count; ++n) {
    const uint32_t par = static_cast<uint32_t>(n) & 1u;
    if (!qwait(bar(qbReady + st.stage), st.phase, ctx, 51)) return;     // row statistics
    if (p.has_mask) {
      if (!qwait(bar(qbMaskFull + mk.stage), mk.phase, ctx, 54)) return;
    }
    if (!qwait(bar(qbSFull + wg), par, ctx, 52)) return;
    tc_fence_after();
    QPROF_BEGIN();
    {
      const float* nl2 = rowstats + st.stage * 256u + wg * 64u;
      const float* nd = rowstats + st.stage * 256u + 128u + wg * 64u;
      const uint32_t mask_row = smem_base + p.off_mask + mk.stage * kQTableBytes + tab_row;
      // Two trips of 32 queries (one table chunk each), each of two pieces of sixteen.  Both
      // loops are rolled to keep the code small (all roles of the kernel have to fit the
      // instruction cache together): the code of a piece exists once, and its eight bias words
      // are picked out of the 32 the thread holds with selects.
#pragma unroll 1
      for (uint32_t c = 0; c < 2u; ++c) {
        uint32_t wsel[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) wsel[i] = c == 0u ? wb[i] : wb[16 + i];
        const uint32_t mchunk = mask_row + (2u * wg + c) * static_cast<uint32_t>(kTableTileBytes);
#pragma unroll 1
        for (uint32_t hh = 0; hh < 2u; ++hh) {
          uint32_t sv[16], dv[16], pw[8], dw[8], w8[8];
          tmem_ld16(tm_s + 32u * c + 16u * hh, sv);
          tmem_ld16(tm_d + 32u * c + 16u * hh, dv);
#pragma unroll
          for (int i = 0; i < 8; ++i) w8[i] = hh == 0u ? wsel[i] : wsel[8 + i];
          tmem_wait_ld();
          quad_half<T>(sv, dv, w8, p.has_mask != 0, mchunk + (((2u * hh) ^ tab_sw) << 4),
                       mchunk + (((2u * hh + 1u) ^ tab_sw) << 4), nl2 + 32u * c + 16u * hh, nd + 32u * c + 16u * hh,
                       scale, pw, dw);
          // P^T and dS^T go back over the first 16 columns of this chunk's own S^T / dP^T
          // columns (columns whose scores were read in an earlier piece or in this one)
          tmem_st8(tm_s + 32u * c + 8u * hh, pw);
          tmem_st8(tm_d + 32u * c + 8u * hh, dw);
        }
      }
    }
    QPROF_SEG(10);
    tmem_wait_st();
    // (the mask stage is handed back behind the wait for the stores of the values computed from
    // its words: by then the shared-memory loads of every one of them have certainly completed)
    if (p.has_mask) {
      mbar_arrive(bar(qbMaskFree + mk.stage));
      mk.advance();
    }
    QPROF_SEG(11);
    // dS also goes to shared memory (A operand of dQ^ += dS K^), but only now: the product that
    // read the previous job's copy was issued while this step was being computed, so it is
    // normally done and this wait costs nothing.  The packed words are read back from tensor
    // memory rather than kept in 32 more registers.
    if (n > 0) {
      if (!qwait(bar(qbDsFree), par ^ 1u, ctx, 53)) return;
    }
#pragma unroll
    for (uint32_t c = 0; c < 2u; ++c) {
      uint32_t dsw[16];
      tmem_ld16(tm_d + 32u * c, dsw);
      tmem_wait_ld();
#pragma unroll
      for (uint32_t gq = 0; gq < 4u; ++gq) {
        const uint32_t w4[4] = {dsw[4 * gq], dsw[4 * gq + 1], dsw[4 * gq + 2], dsw[4 * gq + 3]};
        sts128(ds_base + (((4u * c + gq) ^ ds_sw) << 4), w4);
      }
    }
    tc_fence_before();
    fence_proxy_async_smem();
    mbar_arrive(bar(qbPReady + wg));
    QPROF_SEG(12);
    st.advance();
  }

  // The dB^T sums of this CTA's tile leave tensor memory once, here, after the last product that
  // fed them (it precedes the last dQ product, whose completion the last barrier phase signals).
  // Warpgroup w writes the 64 query columns of its step; the partial buffer is laid out
  // (query, key) like the result.
  if (!qwait(bar(qbDsFree), (static_cast<uint32_t>(g.count) & 1u) ^ 1u, ctx, 56)) return;
  if (p.db_partial != nullptr) {
    tc_fence_after();
    const int key = static_cast<int>(g.a * kTileRows + lt);
    const int cid = static_cast<int>(blockIdx.x) / p.cluster;
    const int q0 = static_cast<int>(g.b * kTileRows + wg * kStepCols);
    float* dst = p.db_partial + static_cast<long long>(cid) * p.db_buf_stride + key;
    const bool key_ok = key < p.N;
    const uint32_t t_db = tmem + lane_base + kQTmDB + 64u * wg;
#pragma unroll 1
    for (uint32_t gq = 0; gq < 8u; ++gq) {
      uint32_t r[8];
      tmem_ld8(t_db + 8u * gq, r);
      tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int qi = q0 + static_cast<int>(8u * gq) + e;
        if (key_ok && qi < p.N) dst[static_cast<long long>(qi) * p.db_pitch] = __uint_as_float(r[e]);
      }
    }
    tc_fence_before();
  }
}

// ------------------------------------------------------------------------------------------------
// One row of one accumulator of one job (0 dV, 1 dK, 2 dQ), already in registers: either pushed
// to the partner CTA that finishes it, or finished here -- the partner's term added, the Jacobian
// of the L2 normalisation applied (dK^, dQ^), the row stored.
// Row r of an accumulator is tensor-memory lane r.  Of dV and dK (rows = keys of block a; the
// other term of the sum is held by CTA (a, 1 - b) = rank ^ 1) a CTA keeps the rows of half
// f = a ^ b and pushes the other half to that partner; of dQ (rows = queries of tile b; partner
// (1 - a, b) = rank ^ 2) it keeps half 1 - f.  A sum of two floats does not depend on the order,
// so the results are bitwise reproducible.
// ------------------------------------------------------------------------------------------------
struct QuadRowCtx {
  uint32_t bars, recv_base, rank, row64, row_sw, par;
  bool quad;
  float scale;
};
template <typename T>
__device__ __forceinline__ bool quad_row(const QuadRowCtx& c, const WaitCtx& ctx, uint32_t (&r)[32], uint32_t X,
                                         bool push, const uint4 (&raw)[4], bool ok, uint16_t* dst,
                                         float& dscale_acc) {
  const uint32_t partner = c.rank ^ (X == 2u ? 2u : 1u);
  const uint32_t full = c.bars + 8u * (qbRecvFull + X), free_ = c.bars + 8u * (qbRecvFree + X);
  const uint32_t slot = c.recv_base + X * kQRecvPart + c.row64 * 128u;
  if (push) {
    // the partner has read what I pushed for the previous job; each 16-byte piece credits the
    // partner's barrier when it has landed there
    // (a plain wait: the partner's arrival carries no data, it only says "read")
    if (!qwait(free_, c.par ^ 1u, ctx, 58)) return false;
    const uint32_t dst_row = cluster_map(slot, partner), dst_bar = cluster_map(full, partner);
#pragma unroll
    for (uint32_t ch = 0; ch < 8u; ++ch) st_async_cluster_v4(dst_row + ((ch ^ c.row_sw) << 4), &r[4 * ch], dst_bar);
    return true;
  }
  if (c.quad) {
    // The rows were delivered by st.async, which completes on this barrier with transaction
    // bytes like a TMA load: observing the phase makes them visible, so a plain wait is enough.
    // (An acquire at cluster scope would also wait for every global load this thread still has in
    // flight -- the raw row requested at the top of the job -- which cost thousands of cycles.)
    if (!qwait(full, c.par, ctx, 59)) return false;
#pragma unroll
    for (uint32_t ch = 0; ch < 8u; ++ch) {
      uint32_t w4[4];
      lds128(slot + ((ch ^ c.row_sw) << 4), w4);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        r[4 * ch + i] = __float_as_uint(__uint_as_float(r[4 * ch + i]) + __uint_as_float(w4[i]));
    }
    // (the additions above have consumed every loaded value: the buffer may be overwritten)
    mbar_arrive_cluster_relaxed(cluster_map(free_, partner));
  }
  // rows of dV are stored as they are; rows of dK^ / dQ^ go through the Jacobian:
  // dx = scale (dX' - x^ (x^ . dX')) / |x| from the raw row x
  float fmul = 1.f, cq = 0.f;
  if (X != 0u) {
    float ss = 0.f, qd = 0.f;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      const uint32_t w4[4] = {raw[ch].x, raw[ch].y, raw[ch].z, raw[ch].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x0 = Elem<T>::lo(w4[e]), x1 = Elem<T>::hi(w4[e]);
        ss = fmaf(x0, x0, ss);
        ss = fmaf(x1, x1, ss);
        qd = fmaf(x0, __uint_as_float(r[8 * ch + 2 * e]), qd);
        qd = fmaf(x1, __uint_as_float(r[8 * ch + 2 * e + 1]), qd);
      }
    }
    const float rn = rsqrtf(fmaxf(ss, 1e-24f));
    const float dot = qd * rn;
    if (X == 2u && ok) dscale_acc += dot;
    fmul = c.scale * rn;
    cq = rn * dot;
  }
  if (ok) {
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      const uint32_t w4[4] = {raw[ch].x, raw[ch].y, raw[ch].z, raw[ch].w};
      uint32_t o4[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v0 = __uint_as_float(r[8 * ch + 2 * e]), v1 = __uint_as_float(r[8 * ch + 2 * e + 1]);
        if (X != 0u) {
          v0 = fmul * (v0 - Elem<T>::lo(w4[e]) * cq);
          v1 = fmul * (v1 - Elem<T>::hi(w4[e]) * cq);
        }
        o4[e] = Elem<T>::pack(v0, v1);
      }
      *reinterpret_cast<uint4*>(dst + 8 * ch) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
    }
  }
  return true;
}

// ------------------------------------------------------------------------------------------------
// The preparing warpgroup (thread = row).  Ahead of the compute warpgroups: K row and Q row of a
// job normalised in place, delta = dO . O and lse * log2(e) of the query row.  Behind them, in
// the time it would otherwise wait for the next tiles to arrive: the dQ accumulator of the job
// that has just finished (pushed to the partner by a keeper of dV / dK, finished by the others).
// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ void quad_prepare_role(const QuadParams& p, uint8_t* smem_ptr, uint32_t smem_base,
                                  uint32_t bars, uint32_t tmem, const WaitCtx& ctx, uint32_t rank,
                                  float& dscale_acc) {
  const QuadGeom g = quad_geom(p, rank);
  if (g.count == 0) return;
  const uint32_t lt = threadIdx.x & 127u;
  const uint32_t lane_base = ((lt >> 5) * 32u) << 16;
  float* rowstats = reinterpret_cast<float*>(smem_ptr + p.off_rowstats);
  const int ig = static_cast<int>(g.b * kTileRows + lt);
  const bool row_ok = ig < p.N;
  const bool quad = p.cluster > 1;
  const bool keeper = quad ? ((lt >> 6) == (g.a ^ g.b)) : false;   // pushes its row of dQ
  QuadRowCtx rc;
  rc.bars = bars; rc.recv_base = smem_base + p.off_recv; rc.rank = rank; rc.row64 = lt & 63u; rc.row_sw = lt & 7u;
  rc.quad = quad; rc.scale = load_scale<T>(p.scale, p.scale_is_tensor, g.h);
  // The O row and lse of a job come straight from global memory (first touch: a trip to DRAM).
  // They are prefetched into L2 one job ahead (no registers held), so that the loads proper, issued
  // before the wait for the job's tiles, are short.
  auto row_ptr = [&](int n) {
    const int bw = g.slot + n * p.nslots;
    return static_cast<const uint16_t*>(p.o) + bw * p.o_sbw + g.h * p.o_sh + ig * p.o_sn;
  };
  auto lse_ptr = [&](int n) {
    const int bw = g.slot + n * p.nslots;
    return p.lse + bw * p.lse_sbw + g.h * p.lse_sh + ig;
  };
  auto prefetch = [&](int n) {
    if (row_ok && n < g.count) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(row_ptr(n)));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(lse_ptr(n)));
    }
  };
  // dQ of job n is handled right after the tiles of job n + lag have been prepared: that job's
  // tiles could only be requested once job n + lag - stages had released its stage, so for
  // lag = stages - 1 the accumulators of job n complete about when this thread gets there.
  const int lag = p.n_stages - 1;
  Ring st(p.n_stages);
  prefetch(0);
  prefetch(1);
#pragma unroll 1
  for (int i = 0; i < g.count + lag; ++i) {
    const int n = i - lag;       // the job whose dQ is handled in this trip (if >= 0)
    // the raw q row for the Jacobian of dQ: requested first, used last
    uint4 raw[4];
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) raw[ch] = make_uint4(0u, 0u, 0u, 0u);
    if (n >= 0 && !keeper && row_ok) {
      const int bw = g.slot + n * p.nslots;
      const uint16_t* qsrc = static_cast<const uint16_t*>(p.q) + bw * p.q_sbw + g.h * p.q_sh + ig * p.q_sn;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) raw[ch] = quad_ldg_v4(qsrc + ch * 8);
    }
    if (i < g.count) {
      prefetch(i + 2);
      uint4 o_row[4];
      float lse = 0.f;
      if (row_ok) {
        const uint16_t* orow = row_ptr(i);
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) o_row[ch] = quad_ldg_v4(orow + ch * 8);
        lse = __ldg(lse_ptr(i));
      }
      const uint32_t base = smem_base + p.off_stage + st.stage * kQStageBytes;
      if (!qwait(bars + 8u * (qbFull + st.stage), st.phase, ctx, 80)) return;
      normalise_row<T>(base, lt);              // K^
      normalise_row<T>(base + 16384u, lt);     // Q^
      float l2 = INFINITY, dl = 0.f;   // a row past the end of the window: p = exp2(-inf) = 0
      if (row_ok) {
        float dlp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t wd[4];
          lds128(base + 24576u + sw64_offset(lt, ch), wd);
          const uint32_t wo[4] = {o_row[ch].x, o_row[ch].y, o_row[ch].z, o_row[ch].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            dlp[ch] = fmaf(Elem<T>::lo(wd[k]), Elem<T>::lo(wo[k]), dlp[ch]);
            dlp[ch] = fmaf(Elem<T>::hi(wd[k]), Elem<T>::hi(wo[k]), dlp[ch]);
          }
        }
        dl = (dlp[0] + dlp[1]) + (dlp[2] + dlp[3]);
        l2 = (lse == -INFINITY) ? INFINITY : lse * kLog2e;
      }
      rowstats[st.stage * 256u + lt] = -l2;            // the compute warpgroups add, never subtract
      rowstats[st.stage * 256u + 128u + lt] = -dl;
      fence_proxy_async_smem();
      mbar_arrive(bars + 8u * (qbReady + st.stage));
      st.advance();
    }
    if (n >= 0) {
      const int bw = g.slot + n * p.nslots;
      rc.par = static_cast<uint32_t>(n) & 1u;
      // what the partner will push for this job: 64 rows x 128 bytes
      if (quad && !keeper && rc.row64 == 0u) mbar_arrive_expect_tx(bars + 8u * (qbRecvFull + 2), kQRecvPart);
      if (!qwait(bars + 8u * qbAccFull, rc.par, ctx, 81)) return;
      tc_fence_after();
      uint32_t r[32];
      tmem_ld32(tmem + lane_base + kQTmDQ, r);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bars + 8u * qbAccFreeQ);
      if (!quad_row<T>(rc, ctx, r, 2u, quad && keeper, raw, row_ok,
                       static_cast<uint16_t*>(p.dq) + bw * p.dq_sbw + g.h * p.dq_sh + ig * p.dq_sn, dscale_acc))
        return;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// The epilogue warpgroup (thread = row), behind the compute warpgroups: the dV and dK accumulators
// of every job (pushed to the partner or finished and stored, see quad_row).  Both are read out of
// tensor memory at once, so that the tensor core can start the next job's sums while the exchange
// and the epilogues run.
// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ void quad_epilogue_role(const QuadParams& p, uint32_t smem_base, uint32_t bars, uint32_t tmem,
                                   const WaitCtx& ctx, uint32_t rank) {
  const QuadGeom g = quad_geom(p, rank);
  if (g.count == 0) return;
  const uint32_t lt = threadIdx.x & 127u;
  const uint32_t lane_base = ((lt >> 5) * 32u) << 16;
  const bool quad = p.cluster > 1;
  const bool keeper = quad ? ((lt >> 6) == (g.a ^ g.b)) : true;   // finishes its rows of dV and dK
  const int krow = static_cast<int>(g.a * kTileRows + lt);
  const bool k_ok = krow < p.N;
  QuadRowCtx rc;
  rc.bars = bars; rc.recv_base = smem_base + p.off_recv; rc.rank = rank; rc.row64 = lt & 63u; rc.row_sw = lt & 7u;
  rc.quad = quad; rc.scale = load_scale<T>(p.scale, p.scale_is_tensor, g.h);
  float unused = 0.f;

#pragma unroll 1
  for (int n = 0; n < g.count; ++n) {
    const int bw = g.slot + n * p.nslots;
    rc.par = static_cast<uint32_t>(n) & 1u;
    // the raw k row for the Jacobian of dK: requested first, used last
    uint4 raw[4];
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) raw[ch] = make_uint4(0u, 0u, 0u, 0u);
    if (keeper && k_ok) {
      const uint16_t* src = static_cast<const uint16_t*>(p.k) + bw * p.k_sbw + g.h * p.k_sh + krow * p.k_sn;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) raw[ch] = quad_ldg_v4(src + ch * 8);
    }
    // what the partner will push for this job: 64 rows x 128 bytes per accumulator I finish
    if (quad && keeper && rc.row64 == 0u) {
      mbar_arrive_expect_tx(bars + 8u * (qbRecvFull + 0), kQRecvPart);
      mbar_arrive_expect_tx(bars + 8u * (qbRecvFull + 1), kQRecvPart);
    }
    if (!qwait(bars + 8u * qbAccFull, rc.par, ctx, 55)) return;
    tc_fence_after();
    QPROF_BEGIN();
    uint32_t r[32], hold[32];
    tmem_ld32(tmem + lane_base + kQTmDV, r);
    tmem_ld32(tmem + lane_base + kQTmDK, hold);
    tmem_wait_ld();
    tc_fence_before();
    mbar_arrive(bars + 8u * qbAccFree);
    QPROF_SEG(0);
    // one trip per accumulator, rolled: the pushing and the finishing code exist once
#pragma unroll 1
    for (uint32_t X = 0; X < 2u; ++X) {
      if (X == 1u) {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = hold[i];
      }
      uint16_t* dst = X == 0u ? static_cast<uint16_t*>(p.dv) + bw * p.dv_sbw + g.h * p.dv_sh + krow * p.dv_sn
                              : static_cast<uint16_t*>(p.dk) + bw * p.dk_sbw + g.h * p.dk_sh + krow * p.dk_sn;
      if (!quad_row<T>(rc, ctx, r, X, quad && !keeper, raw, k_ok, dst, unused)) return;
      QPROF_SEG(1 + X);
    }
  }
}

// The issuing thread (some forty to fifty-six products per job).  Descriptors are assembled from
// a template with one addition: tensor-memory addresses and descriptor offsets are cheap, and a
// descriptor costs one addition (the stage's base address, in 16-byte units, plus a constant).
struct Desc16 {
  uint32_t lo, hi;   // descriptor for shared-memory address 0; add (address >> 4) to lo
};
__device__ __forceinline__ Desc16 make_desc16(uint32_t lbo_bytes, uint32_t sbo_bytes, SmemSwizzle sw) {
  const DescBase b = make_desc_base(0, lbo_bytes, sbo_bytes, sw);
  return Desc16{b.lo, b.hi};
}
__device__ __forceinline__ uint64_t desc16_at(const Desc16& d, uint32_t base16, uint32_t const_bytes) {
  return (static_cast<uint64_t>(d.hi) << 32) | static_cast<uint64_t>(d.lo + base16 + (const_bytes >> 4));
}
// (inside a cluster the shared-memory address of a CTA other than rank 0 carries the rank above
// bit 24: only the offset inside the CTA's own window belongs in a descriptor)
__device__ __forceinline__ uint32_t smem16(uint32_t addr) { return (addr & 0x3FFFFu) >> 4; }

template <typename T>
__device__ void quad_mma_role(const QuadParams& p, uint32_t smem_base, uint32_t bars, uint32_t tmem,
                              const WaitCtx& ctx, uint32_t rank) {
  const QuadGeom g = quad_geom(p, rank);
  if (g.count == 0) return;
  constexpr uint32_t fmt = Elem<T>::kFmt;
  auto bar = [&](int i) { return bars + 8u * i; };
  constexpr uint32_t idesc_s = make_idesc(fmt, 128, kStepCols, 0, 0);
  constexpr uint32_t idesc_acc = make_idesc(fmt, 128, 32, 0, 1);   // A in TMEM, B MN-major
  constexpr uint32_t idesc_dq = make_idesc(fmt, 128, 32, 1, 1);    // A and B MN-major
  const Desc16 dk64 = make_desc16(16, 512, kSw64);      // K-major rows of 64 bytes
  const Desc16 dm64 = make_desc16(512, 512, kSw64);     // MN-major rows of 64 bytes
  const Desc16 dds = make_desc16(16384, 1024, kSw128);  // dS tile, MN-major, two slabs
  const bool with_db = p.db_partial != nullptr;
  const uint32_t ident16_c = smem16(smem_base + p.off_ident);
  const uint32_t ds16_c = smem16(smem_base + p.off_ds);
  constexpr uint32_t kK = 0u, kV = 8192u, kQ = 16384u, kDO = 24576u;   // byte offsets inside a stage

  // Everything is issued from rolled loops with one call site each: this role's code has to share
  // the instruction cache with four other roles, and the issuing thread has time to spare.
  Ring st(p.n_stages);            // the stage of job n + 1 (trip n = -1 issues the first job's scores)
  uint32_t s16 = 0u;              // the stage of job n, in 16-byte units
#pragma unroll 1
  for (int n = -1; n < g.count; ++n) {
    const uint32_t par = static_cast<uint32_t>(n) & 1u;
    const bool has_next = n + 1 < g.count;
    const uint32_t n16 = smem16(smem_base + p.off_stage + st.stage * kQStageBytes);
#pragma unroll 1
    for (uint32_t w = 0; w < 2u; ++w) {
      const uint32_t tw = tmem + w * 128u;
      if (n >= 0) {
        // the accumulators of the previous job have been read out
        if (w == 0u && n > 0) {
          if (!qwait(bar(qbAccFree), par ^ 1u, ctx, 62)) return;
        }
        if (!qwait(bar(qbPReady + static_cast<int>(w)), par, ctx, 64)) return;
        tc_fence_after();
        // dV += P^T dO, dK^ += dS^T Q^, dB^T += dS^T I for step w (each step has its own copy of
        // the identity tile)
#pragma unroll 1
        for (uint32_t ck = 0; ck < 4u; ++ck) {
          const uint32_t c = ck >> 1, k = ck & 1u;
          const uint32_t row_off = (w * kStepCols + c * kChunkCols) * kRowBytes + k * 1024u;
          const uint32_t a_p = tw + kQTmS + 32u * c + 8u * k, a_ds = tw + kQTmDP + 32u * c + 8u * k;
          const uint32_t acc = (w | ck) ? 1u : 0u;
          mma_ts(tmem + kQTmDV, a_p, desc16_at(dm64, s16, kDO + row_off), idesc_acc, acc);
          mma_ts(tmem + kQTmDK, a_ds, desc16_at(dm64, s16, kQ + row_off), idesc_acc, acc);
          if (with_db)
            mma_ts(tmem + kQTmDB + 64u * w + 32u * c, a_ds, desc16_at(dm64, ident16_c, 2048u * w + k * 1024u),
                   idesc_acc, 1u);
        }
      }
      // The next job's scores of step w go over this job's P^T / dS^T of the step (the tensor core
      // works in issue order), so that the warpgroup can go on while the rest is issued:
      // S^T = K^ Q^^T and dP^T = V dO^T for the 64 queries of the step.
      if (has_next) {
        if (w == 0u) {
          if (!qwait(bar(qbReady + st.stage), st.phase, ctx, 66)) return;
          tc_fence_after();
        }
        const uint32_t row_off = w * (kStepCols * kRowBytes);
#pragma unroll 1
        for (uint32_t k = 0; k < 2u; ++k) {
          mma_ss(tw + kQTmS, desc16_at(dk64, n16, kK + 32u * k), desc16_at(dk64, n16, kQ + row_off + 32u * k), idesc_s, k);
          mma_ss(tw + kQTmDP, desc16_at(dk64, n16, kV + 32u * k), desc16_at(dk64, n16, kDO + row_off + 32u * k), idesc_s,
                 k);
        }
        mma_commit(bar(qbSFull + static_cast<int>(w)));
      }
    }
    if (n >= 0) {
      // dQ^ = dS K^ over the 128 keys of the block (the previous job's dQ has been read out)
      if (n > 0) {
        if (!qwait(bar(qbAccFreeQ), par ^ 1u, ctx, 63)) return;
      }
#pragma unroll 1
      for (uint32_t k = 0; k < 8u; ++k)
        mma_ss(tmem + kQTmDQ, desc16_at(dds, ds16_c, k * 2048u), desc16_at(dm64, s16, kK + k * 1024u), idesc_dq, k);
      mma_commit(bar(qbAccFull));
      mma_commit(bar(qbDsFree));
      // the stage of job n: the one before `st`
      mma_commit(bar(qbFree + static_cast<int>(st.stage == 0u ? p.n_stages - 1 : st.stage - 1u)));
    }
    s16 = n16;
    if (has_next) st.advance();
  }
}

// ------------------------------------------------------------------------------------------------
// TMA producer (one thread): the bias tile once, then per job the four row tiles and the mask tile
// ------------------------------------------------------------------------------------------------
__device__ void quad_load_role(const QuadParams& p, uint32_t smem_base, uint32_t bars, const WaitCtx& ctx,
                               uint32_t rank) {
  const QuadGeom g = quad_geom(p, rank);
  if (g.count == 0) return;
  auto bar = [&](int i) { return bars + 8u * i; };
  const int k0 = static_cast<int>(g.a) * kTileRows, q0 = static_cast<int>(g.b) * kTileRows;
  auto load_table = [&](uint32_t dst, const CUtensorMap* map, uint32_t full, int plane) {
    mbar_arrive_expect_tx(full, kQTableBytes);
#pragma unroll 1
    for (int ci = 0; ci < 4; ++ci) {
#pragma unroll 1
      for (int hb = 0; hb < 2; ++hb)
        tma_load_3d(dst + ci * kTableTileBytes + hb * kBoxBytes, map, full, q0 + ci * kChunkCols,
                    k0 + hb * kBoxRows, plane);
    }
  };
  Ring st(p.n_stages), mk(p.n_mask_stages);
#pragma unroll 1
  for (int n = 0; n < g.count; ++n) {
    const int bw = g.slot + n * p.nslots;
    if (!qwait(bar(qbFree + st.stage), st.phase ^ 1u, ctx, 70)) return;
    const uint32_t base = smem_base + p.off_stage + st.stage * kQStageBytes;
    const uint32_t full = bar(qbFull + st.stage);
    mbar_arrive_expect_tx(full, kQStageBytes);
#pragma unroll 1
    for (int hb = 0; hb < 2; ++hb) {
      tma_load_4d(base + hb * kBoxBytes, &p.tm_k, full, 0, k0 + hb * kBoxRows, g.h, bw);
      tma_load_4d(base + 16384u + hb * kBoxBytes, &p.tm_q, full, 0, q0 + hb * kBoxRows, g.h, bw);
      tma_load_4d(base + 8192u + hb * kBoxBytes, &p.tm_v, full, 0, k0 + hb * kBoxRows, g.h, bw);
      tma_load_4d(base + 24576u + hb * kBoxBytes, &p.tm_do, full, 0, q0 + hb * kBoxRows, g.h, bw);
    }
    st.advance();
    if (p.has_mask) {
      if (!qwait(bar(qbMaskFree + mk.stage), mk.phase ^ 1u, ctx, 72)) return;
      load_table(smem_base + p.off_mask + mk.stage * kQTableBytes, &p.tm_maskT, bar(qbMaskFull + mk.stage),
                 bw % p.nW);
      mk.advance();
    }
  }
}

// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kQuadThreads, 1) bwd_quad_kernel(const __grid_constant__ QuadParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t tid = threadIdx.x;
  const uint32_t warp = tid >> 5;
  const uint32_t lane = tid & 31u;
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t bars = smem_base + p.off_ctrl;
  uint32_t* ctrl_words = reinterpret_cast<uint32_t*>(smem_raw + p.off_ctrl + 8u * kQuadNumBars);
  uint32_t& tmem_slot = ctrl_words[0];
  float* warp_sums = reinterpret_cast<float*>(&ctrl_words[4]);
  const bool clustered = p.cluster > 1;
  const uint32_t rank = clustered ? cluster_ctarank() : 0u;
  // (a misaligned dynamic shared-memory base would be the same in every CTA of the launch, so
  // leaving here cannot strand a partner in the cluster)
  if ((smem_base & 1023u) != 0u) {
    if (tid == 0 && p.status != nullptr) atomicCAS(&p.status->code, 0u, (99u << 8) | 2u);
    return;
  }

  if (tid == 0) {
    ctrl_words[1] = 0u;
    for (int i = 0; i < kQuadNumBars; ++i) {
      uint32_t count = 1u;
      if (i >= qbReady && i < qbFree) count = 128u;            // the preparing warpgroup
      else if (i >= qbMaskFree && i < qbBiasFull) count = 256u;
      else if (i >= qbPReady && i < qbAccFull) count = 128u;
      else if (i == qbAccFree || i == qbAccFreeQ) count = 128u; // the epilogue / preparing warpgroup
      else if (i >= qbRecvFull && i < qbRecvFree) count = 1u;  // one arrive.expect_tx; the data credits the rest
      else if (i >= qbRecvFree && i < qbDsFree) count = 64u;
      mbar_init(bars + 8u * i, count);
    }
    mbar_fence_init();
    tma_prefetch_desc(&p.tm_q);
    tma_prefetch_desc(&p.tm_k);
    tma_prefetch_desc(&p.tm_v);
    tma_prefetch_desc(&p.tm_do);
    if (p.has_mask) tma_prefetch_desc(&p.tm_maskT);
  }
  if (warp == 16) {
    tmem_alloc(smem_u32(&tmem_slot), kQuadTmemCols);
    tmem_relinquish();
  }
  // 32 x 32 identity in the layout of a dO chunk (row = query, 64 bytes of columns, 16-byte pieces
  // XOR-swizzled with the row), two copies: B operand of the products that sum dS^T into dB^T
  for (uint32_t wj = tid; wj < 1024u; wj += kQuadThreads) {
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
  // every CTA of the cluster has initialised its barriers before anyone arrives on a peer's
  if (clustered) cluster_sync_all();
  const uint32_t tmem = tmem_slot;
  WaitCtx ctx{&ctrl_words[1], p.status, p.prof};
#if FWA2_TRACE
  const long long prof_t0 = clock64();
  unsigned long long prof_g0 = 0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(prof_g0));
#endif

  float dscale_acc = 0.f;
  // 640 threads start with 96 registers each.  setmaxnreg only moves registers inside what the
  // CTA was given at launch (an increase beyond it would wait for ever), so the four budgets
  // below must not add up to more than 640 x 96.
  constexpr uint32_t kRegCompute = 96, kRegEpilogue = 128, kRegPrepare = 112, kRegIssue = 40;
  static_assert(2 * 128 * kRegCompute + 128 * (kRegEpilogue + kRegPrepare + kRegIssue) <= kQuadThreads * 96,
                "register budgets exceed the launch allocation");
  // (setmaxnreg.inc below what a thread already has, or .dec above it, is an illegal instruction)
  static_assert(kRegCompute >= 96 && kRegEpilogue >= 96 && kRegPrepare >= 96 && kRegIssue <= 96,
                "increase / decrease directions do not match the launch allocation of 96");
  if (warp < 8) {
    reg_alloc<kRegCompute>();
    quad_compute_role<T>(p, smem_raw, smem_base, bars, tmem, ctx, rank);
  } else if (warp < 12) {
    reg_alloc<kRegEpilogue>();
    quad_epilogue_role<T>(p, smem_base, bars, tmem, ctx, rank);
  } else if (warp < 16) {
    reg_alloc<kRegPrepare>();
    quad_prepare_role<T>(p, smem_raw, smem_base, bars, tmem, ctx, rank, dscale_acc);
  } else {
    reg_dealloc<kRegIssue>();
    if (lane == 0) {
      if (warp == 16) quad_mma_role<T>(p, smem_base, bars, tmem, ctx, rank);
      else if (warp == 17) quad_load_role(p, smem_base, bars, ctx, rank);
    }
  }
  __syncwarp();
  // deterministic CTA-wide sum of the dLogitScale contributions
  if (warp >= 12 && warp < 16) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dscale_acc += __shfl_xor_sync(0xFFFFFFFFu, dscale_acc, off);
    if (lane == 0) warp_sums[warp - 12] = dscale_acc;
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && p.dscale_partial != nullptr) {
    const int cid = static_cast<int>(blockIdx.x) / p.cluster;
    const int h = cid % p.H, slot = cid / p.H;
    float s = 0.f;
    for (int w = 0; w < 4; ++w) s += warp_sums[w];
    p.dscale_partial[(slot * p.cluster + static_cast<int>(rank)) * p.H + h] =
        s * load_scale<T>(p.scale, p.scale_is_tensor, h);
  }
#if FWA2_TRACE
  if (tid == 0 && blockIdx.x == 0 && p.prof != nullptr) {
    p.prof[0] = static_cast<unsigned long long>(clock64() - prof_t0);
    p.prof[1] = static_cast<unsigned long long>(quad_geom(p, rank).count);
  }
  if (tid == 0 && p.prof != nullptr && blockIdx.x < 160) {
    unsigned long long g1;
    uint32_t smid;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g1));
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    p.prof[256 + 3 * blockIdx.x] = prof_g0;
    p.prof[257 + 3 * blockIdx.x] = g1;
    p.prof[258 + 3 * blockIdx.x] = smid;
  }
#endif
  if (tid == 0) report_abort(ctrl_words[1], p.status);
  if (ctrl_words[1]) {
    __nanosleep(20000);
    __syncthreads();
  }
  // nobody leaves (and frees its shared memory) while a peer may still push rows or arrive here
  if (clustered) cluster_sync_all();
  if (warp == 16) tmem_dealloc(tmem, kQuadTmemCols);
}

template __global__ void bwd_quad_kernel<__nv_bfloat16>(const __grid_constant__ QuadParams);
template __global__ void bwd_quad_kernel<__half>(const __grid_constant__ QuadParams);

namespace {
template <typename K>
cudaError_t quad_config(K kern, const QuadParams& p, int grid, cudaStream_t stream, cudaLaunchConfig_t* cfg,
                        cudaLaunchAttribute* attr) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(p.smem_bytes));
  if (e != cudaSuccess) return e;
  cfg->gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg->blockDim = dim3(kQuadThreads, 1, 1);
  cfg->dynamicSmemBytes = p.smem_bytes;
  cfg->stream = stream;
  attr->id = cudaLaunchAttributeClusterDimension;
  attr->val.clusterDim.x = static_cast<unsigned>(p.cluster);
  attr->val.clusterDim.y = 1;
  attr->val.clusterDim.z = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
  return cudaSuccess;
}
}  // namespace

// How many clusters of `cluster` CTAs with `smem_bytes` of shared memory the current device can
// hold at once (0 on error).
int quad_max_active_clusters(int dtype_is_bf16, int cluster, uint32_t smem_bytes) {
  QuadParams p{};
  p.cluster = cluster;
  p.smem_bytes = smem_bytes;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr{};
  int n = 0;
  cudaError_t e;
  if (dtype_is_bf16) {
    e = quad_config(bwd_quad_kernel<__nv_bfloat16>, p, cluster, nullptr, &cfg, &attr);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&n, bwd_quad_kernel<__nv_bfloat16>, &cfg);
  } else {
    e = quad_config(bwd_quad_kernel<__half>, p, cluster, nullptr, &cfg, &attr);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&n, bwd_quad_kernel<__half>, &cfg);
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

cudaError_t launch_bwd_quad(const QuadParams& p, int dtype_is_bf16, int grid, cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr{};
  cudaError_t e;
  if (dtype_is_bf16) {
    e = quad_config(bwd_quad_kernel<__nv_bfloat16>, p, grid, stream, &cfg, &attr);
    if (e != cudaSuccess) return e;
    e = cudaLaunchKernelEx(&cfg, bwd_quad_kernel<__nv_bfloat16>, p);
  } else {
    e = quad_config(bwd_quad_kernel<__half>, p, grid, stream, &cfg, &attr);
    if (e != cudaSuccess) return e;
    e = cudaLaunchKernelEx(&cfg, bwd_quad_kernel<__half>, p);
  }
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

}  // namespace fwa2
