// Device-side building blocks for the sm_100a attention kernels: mbarriers with
// bounded waits, TMA tile copies (never cluster-multicast), tcgen05 MMA / TMEM
// access and the shared-memory / instruction descriptors they consume.
//
// Every wait in this file gives up after a fixed number of clock cycles, records
// an error word and lets the kernel run to its normal end, so a protocol bug or a
// late peer can never leave an SM spinning.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pith {

// ---------------------------------------------------------------------------
// Error reporting: one 32-bit status word in global memory per launch.
// 0 = ok; otherwise (code << 24) | detail. First error wins.
// ---------------------------------------------------------------------------
enum : uint32_t {
  kErrWaitTimeout = 1u,   // an mbarrier wait ran out of cycles
  kErrTmemAlloc = 2u,     // TMEM allocation returned an unexpected base
  kErrSmemAlign = 4u,     // the dynamic shared-memory window does not start on a 1024-byte boundary (3 = peer wait)
};

struct AbortCtl {
  uint32_t* status;         // global status word (may be nullptr)
  volatile uint32_t* flag;  // shared-memory abort flag of this CTA
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void report_error(const AbortCtl& ctl, uint32_t code, uint32_t detail) {
  *ctl.flag = 1u;
  if (ctl.status != nullptr) atomicCAS(ctl.status, 0u, (code << 24) | (detail & 0xFFFFFFu));
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Cycle budget of one wait (~0.2 s at 2 GHz; a healthy wait lasts microseconds). Checked every 32 polls.
constexpr long long kWaitCycleLimit = 400000000ll;

// Waits for the phase with the given parity to complete. Returns false (after
// recording the error and raising the CTA's abort flag) when the budget runs out
// or another thread of the CTA has already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const AbortCtl& ctl, uint32_t tag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++polls & 31u) == 0u) {
      if (*ctl.flag != 0u) return false;
      if (clock64() - t0 > kWaitCycleLimit) {
        report_error(ctl, kErrWaitTimeout, tag);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Fences
// ---------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA (tiled, 4-D tensors [B][S][H][D] addressed as {d, h, s, b}); the destination
// is always this CTA's own shared memory.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// ---------------------------------------------------------------------------
// TMEM allocation (whole-warp, converged)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------------------
// CTA pairs (cluster of two CTAs driving one tcgen05 MMA with cta_group::2).
// Rank 0 of the pair issues the MMAs; both CTAs stage operands in their own shared
// memory and own half of the accumulator rows in their own TMEM.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// All threads of both CTAs: arrive, then wait (hardware cluster barrier; every thread reaches it because
// every other wait in the kernels is bounded).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrives on an mbarrier given by its shared::cluster address (own CTA or the peer).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load into this CTA's shared memory whose completion bytes are counted by an mbarrier that may live in
// the peer CTA (given by its shared::cluster address). One destination CTA only: no multicast.
__device__ __forceinline__ void tma_load_4d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// TMEM allocation over the pair: one converged warp of EACH CTA executes these with the same arguments.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem, 256 rows over the pair] (+)= A[smem of each CTA: its 128 rows] * B[smem of each CTA: its half of N]
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem of each CTA: its 128 rows] * B[smem of each CTA: its half of N]
__device__ __forceinline__ void umma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Once every MMA issued so far by this thread has completed, arrives on the mbarrier at this shared-memory offset
// in BOTH CTAs of the pair (a barrier signal, not a data copy).
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(both)
      : "memory");
}

// ---------------------------------------------------------------------------
// Descriptors
// ---------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle. Offsets are in bytes.
//  K-major operand  ([rows][64 bf16], 128 B per row): sbo = 1024 (8 rows), lbo unused.
//  MN-major operand ([k rows][64 bf16] blocks):       sbo = 1024 (8 k rows), lbo = bytes between 64-wide MN blocks.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4)                                   // D = f32
         | (1u << 7)                                 // A = bf16
         | (1u << 10)                                // B = bf16
         | (static_cast<uint32_t>(a_mn_major) << 15) // A major
         | (static_cast<uint32_t>(b_mn_major) << 16) // B major
         | (static_cast<uint32_t>(n >> 3) << 17)     // N / 8
         | (static_cast<uint32_t>(m >> 4) << 24);    // M / 16
}

// ---------------------------------------------------------------------------
// tcgen05.mma (single issuing thread), commit
// ---------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------
// TMEM <-> registers. Shape 32x32b: thread i of the warp owns lane (32 * (warp % 4) + i)
// and receives N consecutive 32-bit columns.
// ---------------------------------------------------------------------------
#define PITH_R8(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7])
#define PITH_W8(r, o) "r"(r[o + 0]), "r"(r[o + 1]), "r"(r[o + 2]), "r"(r[o + 3]), "r"(r[o + 4]), "r"(r[o + 5]), "r"(r[o + 6]), "r"(r[o + 7])

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : PITH_R8(r, 0), PITH_R8(r, 8), PITH_R8(r, 16), PITH_R8(r, 24)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : PITH_R8(r, 0), PITH_R8(r, 8)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};" ::PITH_W8(r, 0),
      PITH_W8(r, 8), PITH_W8(r, 16), PITH_W8(r, 24), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};" ::PITH_W8(r, 0),
      PITH_W8(r, 8), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------
// Launch order. The grid is (tiles, heads, batch) and CTAs are dispatched x-fastest; the kernels number their tiles
// heaviest first (causal), which balances one head but leaves the heavy tiles of the last heads for the end of the
// launch. This maps the linear CTA index to (tile, head) so that heads go in groups of G = 8 with the tile index
// outermost inside a group: the last group is short enough to be balanced by its own heavy-first order, and only G
// heads' streamed tensors are hot in L2 at a time (32 heads x 8192^2 causal: forward 0.485 -> 0.431 ms, dK/dV pass
// 0.861 -> 0.832 ms, dQ pass 0.622 -> 0.600 ms; groups of 4 measured the same).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void launch_order(int x, int tiles, bool causal, int& tile, int& head) {
  const int H = gridDim.y;
  const int G = (H % 8 == 0) ? 8 : (H % 4 == 0) ? 4 : (H % 2 == 0) ? 2 : 1;
  if (!causal || G == 1) {  // equal tiles: nothing to balance
    tile = x;
    head = blockIdx.y;
    return;
  }
  const int l = x + tiles * blockIdx.y;
  const int g = l / (G * tiles), r = l - g * (G * tiles);
  tile = r / G;
  head = g * G + (r - tile * G);
}

// ---------------------------------------------------------------------------
// Small helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed fp32 pairs (one 64-bit register = two floats): Blackwell issues fma/add/mul on both halves at once.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^x for a pair of floats on the FMA pipe instead of the MUFU: x = n + f with n = round(x), |f| <= 0.5, 2^f by a
// degree-3 polynomial (relative error below 8e-5, far inside the bf16 rounding the results get), n added to the
// exponent field. Inputs are clamped to >= -125 (the result stays a normal number, about 2e-38): callers that need an
// exact 0 for -inf (masked scores, rows without any visible key) must take the MUFU path for those. The backward passes
// route a quarter (dQ) or a third (dK/dV) of their exponentials through it: the MUFU's 16 results per clock otherwise
// bound the 16384 exponentials of a tile at 1024 cycles. The forward measured no gain and keeps the MUFU.
__device__ __forceinline__ void exp2_poly2(float x0, float x1, float& p0, float& p1) {
  const uint64_t x2 = f2_pack(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
  const uint64_t magic = f2_pack(12582912.f, 12582912.f), nmagic = f2_pack(-12582912.f, -12582912.f);  // 1.5 * 2^23
  const uint64_t xi = f2_add(x2, magic);  // low mantissa bits = round(x)
  const uint64_t fr = f2_fma(f2_add(xi, nmagic), f2_pack(-1.f, -1.f), x2);
  uint64_t p = f2_fma(f2_pack(0.05508868396282196f, 0.05508868396282196f), fr,
                      f2_pack(0.24260404706001282f, 0.24260404706001282f));
  p = f2_fma(p, fr, f2_pack(0.6932762265205383f, 0.6932762265205383f));
  p = f2_fma(p, fr, f2_pack(0.9999289512634277f, 0.9999289512634277f));
  float a0, a1, n0, n1;
  f2_unpack(p, a0, a1);
  f2_unpack(xi, n0, n1);
  p0 = __int_as_float(__float_as_int(a0) + (__float_as_int(n0) << 23));
  p1 = __int_as_float(__float_as_int(a1) + (__float_as_int(n1) << 23));
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Register budget hand-over between warpgroups (whole warpgroup, converged).
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
// Elects one lane of a converged warp (the same lane every time). The MMA-issuing warps run their whole loop
// converged and guard only the tcgen05 instructions with this predicate: descriptor arithmetic then stays
// warp-uniform, which measured 5 % faster backward passes than branching to a single lane around the loop.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
// Adds a byte offset to the start-address field of a shared-memory descriptor.
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) { return desc + (bytes >> 4); }

// Packs two floats into a bf16x2 word: lo -> bits [0,16), hi -> bits [16,32).
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// Byte offset of element (row, col) inside a [rows][64] bf16 tile stored with the 128-byte
// swizzle (tile base 1024-byte aligned): 16-byte chunk index XOR (row mod 8).
__device__ __forceinline__ uint32_t swz128_off(uint32_t row, uint32_t col) {
  return row * 128u + ((((col >> 3) ^ row) & 7u) << 4) + ((col & 7u) << 1);
}

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace pith
