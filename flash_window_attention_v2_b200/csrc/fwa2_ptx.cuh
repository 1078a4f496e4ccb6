// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor, no
// multicast anywhere), tcgen05 (TMEM alloc, MMA, commit, ld/st) and the shared
// memory / instruction descriptors the 5th-generation tensor cores consume.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace fwa2 {

// ---------------------------------------------------------------------------------------------
// Error reporting from device code.  Every wait in the kernels is bounded; a wait that runs out
// records a code here (first writer wins) and raises a CTA-wide abort flag so that all roles
// fall through their loops and the kernel returns normally.
// ---------------------------------------------------------------------------------------------
struct DeviceStatus {
  unsigned int code;     // 0 = ok, otherwise (site << 8) | kind
  unsigned int block;    // blockIdx.x of the first reporter
  unsigned int detail;   // site-specific
  unsigned int pad;
};

enum : unsigned int { kStatusTimeout = 1 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrival that hands a shared-memory buffer back to an asynchronous producer (TMA) after this
// thread has read it with ld.shared.  A plain arrival may be issued while those loads are still
// outstanding: only the arithmetic on the loaded values is tied to them, and arithmetic may be
// scheduled after an arrival that does not depend on it -- the producer has then been seen to
// overwrite the buffer under a warp that had not got its data yet.  Here the barrier address is
// made to depend on the loaded words (`loaded`: an OR over one word of every load; `zero`: a value
// that is 0 at run time but unknown to the compiler), so the arrival cannot issue before they are
// all in registers.
__device__ __forceinline__ void mbar_arrive_after_loads(uint32_t bar, uint32_t loaded, uint32_t zero) {
  mbar_arrive(bar + (loaded & zero));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// The thread may stay suspended for up to kTryWaitHintNs while the phase is incomplete and is
// woken when it completes: a waiting warp then takes (almost) no issue slots from the warps that
// do the arithmetic on the same scheduler, and no latency is added.
#ifndef FWA2_TRY_WAIT_HINT_NS
#define FWA2_TRY_WAIT_HINT_NS 20000
#endif
constexpr uint32_t kTryWaitHintNs = FWA2_TRY_WAIT_HINT_NS;
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
#if FWA2_TRY_WAIT_HINT_NS > 0
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kTryWaitHintNs)
      : "memory");
#else
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
#endif
  return ok;
}

// Non-blocking test of a phase (try_wait may suspend the thread for a while; pollers that serve
// several queues must not).
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Shared-memory abort flag + global status word, handed to every bounded wait.
struct WaitCtx {
  volatile uint32_t* abort_flag;   // in shared memory
  DeviceStatus* status;            // in global memory (may be nullptr)
  unsigned long long* wait_acc;    // development builds (-DFWA2_TRACE=1): cycles waited per site, CTA 0
};

// About one second at ~1.9 GHz: far beyond any legitimate wait in these kernels.
constexpr long long kWaitLimitCycles = 2000000000ll;

// Bounded wait on an mbarrier phase.  Returns false if the wait was abandoned.  The polling loop
// is kept out of line: the kernels that use it are bound by instruction fetch, and the fast path
// (the phase has already completed) is what runs nearly every time.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                            DeviceStatus* status, uint32_t site) {
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3Fu) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *abort_flag = 1u;
        if (status != nullptr) {
          if (atomicCAS(&status->code, 0u, (site << 8) | kStatusTimeout) == 0u) {
            status->block = blockIdx.x;
            status->detail = parity;
          }
        }
        return false;
      }
    }
  }
}
#ifndef FWA2_WAIT_INLINE
#define FWA2_WAIT_INLINE 0
#endif
// kRelaxed: for roles that run ahead of their consumers (producers, preparing warps) -- the polling
// loop backs off with nanosleep, so that it does not take issue slots from the warps that do the
// arithmetic on the same scheduler.
template <bool kRelaxed = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                          uint32_t site) {
#if defined(FWA2_TRACE) && FWA2_TRACE
  // cycles spent waiting, per site, for one warp of each role of CTA 0 (second compute
  // warpgroup: site + 100)
  {
    const long long w0 = clock64();
    bool done = false;
    for (long long it = 0; it < (1ll << 26) && !done; ++it) done = mbar_try_wait(bar, parity);
    const uint32_t warp = threadIdx.x >> 5;
    if (ctx.wait_acc != nullptr && blockIdx.x == 0 && (threadIdx.x & 31u) == 0u &&
        (warp == 0u || warp == 4u || warp == 8u || warp == 12u || warp == 16u))
      atomicAdd(ctx.wait_acc + site + (warp == 4u ? 100u : 0u), static_cast<unsigned long long>(clock64() - w0));
    return done;
  }
#endif
  if (mbar_try_wait(bar, parity)) return true;
#if FWA2_WAIT_INLINE
  // Inline polling loop, kept short (it exists at every wait site of an instruction-cache-bound
  // kernel): on expiry only the CTA's abort word is set, to (site << 8 | kind); the kernel copies
  // it into the caller's status word at its end (report_abort()).
  // (32-bit clock: the limit is below 2^32 cycles and the clock is read every 256 polls)
  const uint32_t t0 = static_cast<uint32_t>(clock());
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (kRelaxed) __nanosleep(200);
    if ((++spins & 0xFFu) == 0) {
      if (*ctx.abort_flag) return false;
      if (static_cast<uint32_t>(clock()) - t0 > static_cast<uint32_t>(kWaitLimitCycles)) {
        *ctx.abort_flag = (site << 8) | kStatusTimeout;
        return false;
      }
    }
  }
#else
  return mbar_wait_slow(bar, parity, ctx.abort_flag, ctx.status, site);
#endif
}

// End of kernel, one thread: a wait that ran out left (site << 8 | kind) in the CTA's abort word;
// the first CTA to report wins the caller's status word.
__device__ __forceinline__ void report_abort(uint32_t abort_word, DeviceStatus* status) {
  if (abort_word != 0u && status != nullptr) {
    const uint32_t code = (abort_word >> 8) != 0u ? abort_word : ((99u << 8) | kStatusTimeout);
    if (atomicCAS(&status->code, 0u, code) == 0u) {
      status->block = blockIdx.x;
      status->detail = 0u;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Thread-block clusters: the rank of this CTA, a peer CTA's view of one of my shared-memory
// addresses, plain stores into a peer's shared memory, and mbarrier traffic with cluster scope
// (a peer's stores followed by its release-arrive are visible after an acquire-wait).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, const uint32_t* v) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(v[0]),
               "r"(v[1]), "r"(v[2]), "r"(v[3])
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// An arrival that orders nothing: for "I have finished READING your buffer" signals, issued after
// the instructions that consumed the loaded values (a release at cluster scope would also wait
// for every global store the thread still has in flight).
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// 16 bytes into a peer's shared memory; the peer's mbarrier (in the same CTA as the destination)
// is credited with 16 transaction bytes when the data has landed, so the sender needs no fence
// and no arrival of its own.
__device__ __forceinline__ void st_async_cluster_v4(uint32_t cluster_addr, const uint32_t* v,
                                                    uint32_t cluster_mbar) {
  asm volatile(
      "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
      ::"r"(cluster_addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(cluster_mbar)
      : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kTryWaitHintNs)
      : "memory");
  return ok;
}
// Bounded wait for a phase that a peer CTA of the cluster completes.  Same contract as
// mbar_wait(): false once the wait was abandoned (the CTA's abort word then names the site).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                                  uint32_t site) {
#if defined(FWA2_TRACE) && FWA2_TRACE
  {
    const long long w0 = clock64();
    bool done = false;
    for (long long it = 0; it < (1ll << 26) && !done; ++it) done = mbar_try_wait_cluster(bar, parity);
    const uint32_t warp = threadIdx.x >> 5;
    if (ctx.wait_acc != nullptr && blockIdx.x == 0 && (threadIdx.x & 31u) == 0u &&
        (warp == 0u || warp == 4u || warp == 8u || warp == 12u || warp == 16u))
      atomicAdd(ctx.wait_acc + site + (warp == 4u ? 100u : 0u), static_cast<unsigned long long>(clock64() - w0));
    return done;
  }
#endif
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint32_t t0 = static_cast<uint32_t>(clock());
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++spins & 0xFFu) == 0) {
      if (*ctx.abort_flag) return false;
      if (static_cast<uint32_t>(clock()) - t0 > static_cast<uint32_t>(kWaitLimitCycles)) {
        *ctx.abort_flag = (site << 8) | kStatusTimeout;
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Proxy fences
// ---------------------------------------------------------------------------------------------
// Make generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA (tiled tensor maps).  The innermost coordinate times the element size is always a
// multiple of 16 bytes at every call site in this library.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// Tensor memory (TMEM)
// ---------------------------------------------------------------------------------------------
// Warp-collective.  ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 columns of 32 bit: thread t of the warp gets lane (base_lane + t), registers
// r[0..31] get consecutive columns.  taddr = (lane << 16) | column.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 8 columns.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                 "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
// 32 lanes x 16 columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15])
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05.mma descriptors
// ---------------------------------------------------------------------------------------------
enum SmemSwizzle : uint64_t { kSwNone = 0, kSw128 = 2, kSw64 = 4, kSw32 = 6 };

// 64-bit shared-memory matrix descriptor (sm_100 format): start address, leading and stride
// byte offsets in 16-byte units, descriptor version 1, swizzle mode in bits 61..63.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, SmemSwizzle sw) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= static_cast<uint64_t>(sw) << 61;
  return d;
}

// 32-bit instruction descriptor for kind::f16 with fp32 accumulation.
// in_fmt: 0 = f16, 1 = bf16.  a_mn / b_mn: 1 when the operand is MN-major in shared memory.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t in_fmt, uint32_t m, uint32_t n,
                                                  uint32_t a_mn, uint32_t b_mn) {
  return (1u << 4) | (in_fmt << 7) | (in_fmt << 10) | (a_mn << 15) | (b_mn << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

// A descriptor whose start address can be advanced with one 32-bit add (the address field sits in
// the low word and never carries out of its 14 bits for addresses below 256 KiB).
struct DescBase {
  uint32_t lo, hi;
};
__device__ __forceinline__ DescBase make_desc_base(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, SmemSwizzle sw) {
  const uint64_t d = make_smem_desc(smem_addr, lbo_bytes, sbo_bytes, sw);
  return DescBase{static_cast<uint32_t>(d), static_cast<uint32_t>(d >> 32)};
}
// (Inside a thread-block cluster the shared-memory address of a CTA other than rank 0 carries the
// rank above bit 24; only the offset inside the CTA's own window belongs in the descriptor.)
__device__ __forceinline__ uint64_t desc_at(const DescBase& b, uint32_t byte_offset) {
  return (static_cast<uint64_t>(b.hi) << 32) | static_cast<uint64_t>(b.lo + ((byte_offset & 0x3FFFFu) >> 4));
}

// Position in a ring of `n` pipeline stages with the mbarrier phase bit that goes with it.
struct Ring {
  uint32_t stage, phase, n;
  __device__ __forceinline__ explicit Ring(uint32_t n_) : stage(0), phase(0), n(n_) {}
  __device__ __forceinline__ void advance() {
    if (++stage == n) {
      stage = 0;
      phase ^= 1u;
    }
  }
};

// Warpgroup-wide register reallocation (all four warps of a warpgroup execute the same one).
template <uint32_t kRegs>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <uint32_t kRegs>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// One lane of a fully converged warp (the same lane every time).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xFFFFFFFF;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// D[tmem] (+)= A[smem] * B[smem].  Issued by one thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem].  A holds 16-bit elements packed two per 32-bit column.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival once every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// Swizzled tile addressing used by threads (must match what TMA writes and the MMA reads).
// Tiles are stored as rows of 64 bytes (SW64) or 128 bytes (SW128); the 16-byte chunk index is
// XOR-ed with row bits.  Tile bases are 1024-byte aligned.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t sw64_offset(uint32_t row, uint32_t chunk) {
  return row * 64u + ((chunk ^ ((row >> 1) & 3u)) << 4);
}
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

__device__ __forceinline__ void lds128(uint32_t addr, uint32_t (&v)[4]) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "r"(addr));
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint32_t (&v)[4]) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3])
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// 16-bit element helpers, templated on the storage type (__nv_bfloat16 or __half).
// ---------------------------------------------------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<__nv_bfloat16> {
  static constexpr uint32_t kFmt = 1;
  __device__ static __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
  __device__ static __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
  __device__ static __forceinline__ uint32_t pack(float a, float b) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
  }
  __device__ static __forceinline__ float from_raw(uint16_t x) {
    return __uint_as_float(static_cast<uint32_t>(x) << 16);
  }
};
template <>
struct Elem<__half> {
  static constexpr uint32_t kFmt = 0;
  __device__ static __forceinline__ float lo(uint32_t w) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xFFFFu)));
  }
  __device__ static __forceinline__ float hi(uint32_t w) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
  }
  __device__ static __forceinline__ uint32_t pack(float a, float b) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
  }
  __device__ static __forceinline__ float from_raw(uint16_t x) {
    return __half2float(__ushort_as_half(x));
  }
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace fwa2
