// Attention backward for head dimension 128 (GQA / MHA) on sm_100a.
//
// A tcgen05 MMA with M = 128 and K = 16 costs 64 cycles at N = 128 and still 48 at N = 64 (measured), so
// every GEMM here is 128 x 128: a 128-row tile is resident for the whole CTA and 128-row tiles stream past it. TMEM then has room for exactly one pair of score tiles next to the
// accumulators, so instead of double-buffering the scores the four GEMMs of an iteration are
// interleaved with the next iteration's so that the tensor core always has a GEMM to run while the
// 256 compute threads are in the exponentials:
//
//   mode kDkDv (resident K_n, V_n; streamed Q_i, dO_i; lane = key, column = query)
//     MMA order   S^T(0) dP^T(0) | dV(0) S^T(1) dK(0) dP^T(1) | dV(1) S^T(2) dK(1) dP^T(2) | ...
//     compute     P^T(k) = exp2(S^T c - lse) after S^T(k)      -> bf16 into T1, feeds dV(k) = P^T dO_i
//                 (stored in two halves: dV(k) starts on the first while the second is in the exponentials)
//                 dS^T(k) = P^T (dP^T - delta) after dP^T(k)   -> bf16 into T2, feeds dK(k) = dS^T Q_i
//   mode kDq (resident Q_m, dO_m; streamed K_j, V_j; lane = query, column = key)
//     MMA order   S(0) dP(0) | S(1) dQ(0) dP(1) | S(2) dQ(1) dP(2) | ...
//     compute     P(k) after S(k) (kept in registers), dS(k) after dP(k) -> bf16 into T2, feeds dQ(k) = dS K_j
//
// lse is the log2-domain LSE of the complete softmax row, delta = rowsum(O dO). Results are scaled
// (dK, dQ by softmax_scale) and ADDED to fp32 accumulators with vector atomics.
//
// Warps (384 threads): 0 = TMA producer (+ per-query statistics of the streamed tile in kDkDv), 1 = MMA
// issuer, 4..11 = compute: thread (warp & 3, lane) owns TMEM lane = row of the resident tile, warps 4..7
// take score columns 0..63 and warps 8..11 columns 64..127.
// TMEM columns: T1 [0,128), T2 [128,256), accumulators [256,384) (dV or dQ) and [384,512) (dK).
// The packed bf16 operands overlay the first half of each thread's own 64 score columns:
// queries/keys 0..63 at columns [0,32), 64..127 at [64,96) of T1 (P^T) / T2 (dS).
#include <type_traits>

#include "attn_bwd_common.h"
#include "common.cuh"
#include "host_common.h"

namespace pith {
namespace bwd128 {

constexpr int kThreads = 384;
constexpr int kRegsLo = 72;
constexpr int kRegsHi = 208;
constexpr int kT = 128;             // tile edge (rows of both tiles, head dimension)
constexpr int kTile = kT * kT * 2;  // bytes of one bf16 tile
// Ring depths. X1 (Q_i / K_j) is read first by the score GEMM of an iteration and last by its final GEMM, so a stage is
// held for a whole iteration, and a two-deep ring leaves the next load (a TMA round trip of ~2000 cycles) no time before
// the next-but-one score GEMM wants it: three stages. X2 (dO_i / V_j) is released early: two stages, plus in mode kDq a
// third one in the resident dO tile's shared memory, which is free once the resident tiles have been copied into TMEM
// (a fourth K_j stage in the resident Q tile's memory measured slower). With two stages for Q_i the dK/dV pass took
// 1.08 ms on 32 heads x 8192^2 causal; with three, 0.87 ms.
constexpr int kNS1 = 3;
constexpr int kNS2 = 2;
constexpr int kMaxST = 3;

struct Smem {
  static constexpr int kR1Off = 0;
  static constexpr int kR2Off = kR1Off + kTile;
  static constexpr int kX1Off = kR2Off + kTile;
  static constexpr int kX2Off = kX1Off + kNS1 * kTile;
  static constexpr int kStatOff = kX2Off + kNS2 * kTile;  // [2][2][128] floats: a two-deep ring of its own
  static constexpr int kFlagOff = kStatOff + 2 * 2 * kT * 4;
  static constexpr int kBarOff = kFlagOff + 8;
  static constexpr int kNumBars = 1 + 4 * kMaxST + 7 + 4;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;
  static constexpr int kAlloc = kTotal;  // no slack: the kernel checks that the dynamic window starts 1024-aligned
};
static_assert(Smem::kAlloc <= 232448, "shared memory budget");

constexpr uint32_t kColT1 = 0, kColT2 = 128, kColAcc = 256, kColAcc2 = 384;
// Mode kDq leaves TMEM columns [384,512) unused: the resident Q and dO tiles are copied there once (packed bf16,
// 64 columns each) so that S and dP take their A operand from TMEM and only the streamed tile is read from shared
// memory; an MMA with both operands in shared memory re-reads 8 KB per K-step and competes with the TMA writes.
constexpr uint32_t kColR1 = 384, kColR2 = 448;

// D[128 x 128] = A[128 x 128] * B[128 x 128]^T, both K-major in shared memory (two [128][64] sub-tiles each).
__device__ __forceinline__ void gemm_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool leader) {
#pragma unroll
  for (int kk = 0; kk < kT / 16; ++kk) {
    const uint32_t off = (kk >> 2) * (kT * 128) + (kk & 3) * 32;
    if (leader) umma_ss(d_tmem, desc_advance(adesc, off), desc_advance(bdesc, off), idesc, kk > 0 ? 1u : 0u);
  }
}
// D[128 x 128] (+)= A[128 x 128] (packed bf16 in TMEM, halves at columns +0 and +64) * B (MN-major tile in shared memory)
// PART 0: all eight K-steps; 1: K-steps {0,1,4,5} (the first half of every thread's packed columns); 2: {2,3,6,7},
// always accumulating.
template <int PART = 0>
__device__ __forceinline__ void gemm_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, bool acc,
                                        bool leader) {
#pragma unroll
  for (int kk = 0; kk < kT / 16; ++kk) {
    if (PART == 1 && (kk & 2)) continue;
    if (PART == 2 && !(kk & 2)) continue;
    const uint32_t a = a_tmem + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8);
    if (leader) umma_ts(d_tmem, a, desc_advance(bdesc, kk * 2048), idesc, (PART == 2 || acc || kk > 0) ? 1u : 0u);
  }
}

// D[128 x 128] = A[128 x 128] (packed bf16 in TMEM, 64 consecutive columns) * B[128 x 128]^T (K-major in shared memory)
__device__ __forceinline__ void gemm_tk(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, bool leader) {
#pragma unroll
  for (int kk = 0; kk < kT / 16; ++kk) {
    const uint32_t off = (kk >> 2) * (kT * 128) + (kk & 3) * 32;
    if (leader) umma_ts(d_tmem, a_tmem + kk * 8, desc_advance(bdesc, off), idesc, kk > 0 ? 1u : 0u);
  }
}
// Row `row` of a [128][128] bf16 tile (two swizzled [128][64] sub-tiles in shared memory) -> 64 packed TMEM columns.
__device__ __forceinline__ void copy_row_to_tmem(const uint8_t* tile, int row, uint32_t taddr) {
#pragma unroll
  for (int sub = 0; sub < 2; ++sub) {
    uint32_t r[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 v = *reinterpret_cast<const uint4*>(tile + sub * (kT * 128) + row * 128 + ((c ^ (row & 7)) << 4));
      r[4 * c] = v.x; r[4 * c + 1] = v.y; r[4 * c + 2] = v.z; r[4 * c + 3] = v.w;
    }
    tmem_st32(taddr + sub * 32, r);
  }
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    attn_bwd128_kernel(const __grid_constant__ CUtensorMap tm_r1, const __grid_constant__ CUtensorMap tm_r2,
                       const __grid_constant__ CUtensorMap tm_x1, const __grid_constant__ CUtensorMap tm_x2,
                       const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sR1 = smem + Smem::kR1Off;
  uint8_t* sR2 = smem + Smem::kR2Off;
  uint8_t* sX1 = smem + Smem::kX1Off;
  uint8_t* sX2 = smem + Smem::kX2Off;
  float* sStat = reinterpret_cast<float*>(smem + Smem::kStatOff);
  volatile int* sFlag = reinterpret_cast<volatile int*>(smem + Smem::kFlagOff);  // [2], per statistics stage
  constexpr int NS1 = kNS1;
  constexpr int NS2 = (MODE == kDq) ? kNS2 + 1 : kNS2;
  auto x1_stage = [&](int st) { return sX1 + st * kTile; };
  auto x2_stage = [&](int st) { return st < kNS2 ? sX2 + st * kTile : sR2; };
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBarOff);
  uint64_t* res_full = bars;
  // The two streamed tiles have separate rings: X2 (dO_i / V_j) is last used earlier than X1 (Q_i / K_j), so
  // its next load can start earlier, and the GEMM that needs X1 does not wait for X2's bytes.
  uint64_t* x_full = bars + 1;          // X1 (+ statistics in kDkDv)
  uint64_t* x_empty = x_full + kMaxST;
  uint64_t* x2_full = x_empty + kMaxST;
  uint64_t* x2_empty = x2_full + kMaxST;
  uint64_t* t1_full = x2_empty + kMaxST;
  uint64_t* t2_full = t1_full + 1;
  uint64_t* p_full = t2_full + 1;   // kDkDv: P^T is in TMEM; kDq: T1 has been read
  uint64_t* ds_full = p_full + 1;   // dS is in TMEM
  uint64_t* acc_full = ds_full + 1;
  uint64_t* rt_full = acc_full + 1;  // kDq: resident tiles are in TMEM
  uint64_t* ph_full = rt_full + 1;   // kDkDv: the first half of every thread's P^T columns is in TMEM
  uint64_t* st_full = ph_full + 1;   // kDkDv: statistics of the streamed queries (two stages)
  uint64_t* st_empty = st_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Smem::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortCtl ctl{p.status, abort_flag};

  // kDkDv: one CTA walks the query tiles of `hpc` consecutive query heads of one GQA group (same K_n, V_n, same
  // accumulators): fewer prologues and fewer fp32 write-outs per unit of work. `head` is the first of them.
  const int hpc = (MODE == kDkDv) ? p.hpc : 1;
  int tile_i, head_i;
  launch_order(blockIdx.x, gridDim.x, p.causal != 0, tile_i, head_i);
  const int head = head_i * hpc;
  const int batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  int r0, it_begin, it_end;
  if constexpr (MODE == kDkDv) {
    r0 = tile_i * kT;  // first key; small r0 = most work, launched first
    it_begin = p.causal ? max(0, r0 - p.causal_off) / kT : 0;
    it_end = (p.Sq + kT - 1) / kT;
  } else {
    r0 = (gridDim.x - 1 - tile_i) * kT;  // first query; late queries first
    it_begin = 0;
    it_end = (p.Sk + kT - 1) / kT;
    if (p.causal) {
      const int last_key = min(r0 + kT - 1, p.Sq - 1) + p.causal_off;
      it_end = last_key < 0 ? 0 : min(it_end, last_key / kT + 1);
    }
  }
  const int n_tile = max(0, it_end - it_begin);  // streamed tiles per head
  const int n_div = max(n_tile, 1);
  int n_it = n_tile * hpc;

  if (threadIdx.x == 0) {
    // a launch that finds an error already recorded (by an earlier CTA or launch) does no work
    *abort_flag = (p.status != nullptr && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) ? 1u : 0u;
    mbar_init(res_full, 1);
    for (int i = 0; i < kMaxST; ++i) {
      mbar_init(&x_full[i], 1);
      mbar_init(&x_empty[i], 1);
      mbar_init(&x2_full[i], 1);
      mbar_init(&x2_empty[i], 1);
    }
    mbar_init(t1_full, 1);
    mbar_init(t2_full, 1);
    mbar_init(p_full, 256);
    mbar_init(ds_full, 256);
    mbar_init(acc_full, 1);
    mbar_init(rt_full, 256);
    mbar_init(ph_full, 256);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&st_full[i], 1);
      mbar_init(&st_empty[i], 256);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if ((smem_u32(smem) & 1023u) != 0u) {  // the swizzled tiles need a 1024-byte aligned window
    if (threadIdx.x == 0) report_error(ctl, kErrSmemAlign, smem_u32(smem));
    n_it = 0;
  }
  if (*abort_flag != 0u) n_it = 0;

  const int r1_head = (MODE == kDkDv) ? kv_head : head;  // head index of the resident tensors

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    setmaxnreg_dec<kRegsLo>();
    if (n_it > 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tm_r1);
        tma_prefetch_desc(&tm_r2);
        tma_prefetch_desc(&tm_x1);
        tma_prefetch_desc(&tm_x2);
        mbar_arrive_expect_tx(res_full, 2 * kTile);
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          tma_load_4d(sR1 + sub * (kT * 128), &tm_r1, res_full, sub * 64, r1_head, r0, batch);
          tma_load_4d(sR2 + sub * (kT * 128), &tm_r2, res_full, sub * 64, r1_head, r0, batch);
        }
      }
      // Statistics of the streamed queries (kDkDv): raw lse / delta of iteration k are loaded two iterations ahead
      // into registers (plain global loads take thousands of cycles next to the TMA traffic) and written to the
      // stage as -lse (-inf where the row does not exist or saw no key) and -delta.
      auto load_stats = [&](int k, float (&rl)[4], float (&rd)[4]) {
        if constexpr (MODE == kDkDv) {
          const int hs = k / n_div, x0 = (it_begin + k - hs * n_tile) * kT;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int m = x0 + j * 32 + lane;
            rl[j] = -INFINITY;
            rd[j] = 0.f;
            if (k < n_it && m < p.Sq) {
              rl[j] = p.lse[batch * p.ls[0] + (head + hs) * p.ls[1] + m];
              rd[j] = p.delta[batch * p.dls[0] + (head + hs) * p.dls[1] + m];
            }
          }
        }
      };
      auto step = [&](int k, float (&rl)[4], float (&rd)[4]) {
        const int s1 = k % NS1, s2 = k % NS2;
        const int hs = k / n_div, x0 = (it_begin + k - hs * n_tile) * kT;
        const int x_head = (MODE == kDkDv) ? head + hs : kv_head;  // head index of the streamed tensors
        if (lane == 0) {
          if (MODE == kDq && k == kNS2) mbar_wait(rt_full, 0, ctl, 0x1F0);  // the resident tiles' memory is free now
          mbar_wait(&x_empty[s1], ((k / NS1) & 1) ^ 1, ctl, 0x100 + s1);
          mbar_arrive_expect_tx(&x_full[s1], kTile);
#pragma unroll
          for (int sub = 0; sub < 2; ++sub)
            tma_load_4d(x1_stage(s1) + sub * (kT * 128), &tm_x1, &x_full[s1], sub * 64, x_head, x0, batch);
          mbar_wait(&x2_empty[s2], ((k / NS2) & 1) ^ 1, ctl, 0x180 + s2);
          mbar_arrive_expect_tx(&x2_full[s2], kTile);
#pragma unroll
          for (int sub = 0; sub < 2; ++sub)
            tma_load_4d(x2_stage(s2) + sub * (kT * 128), &tm_x2, &x2_full[s2], sub * 64, x_head, x0, batch);
        }
        if constexpr (MODE == kDkDv) {
          const int ss = k & 1;
          if (lane == 0) mbar_wait(&st_empty[ss], ((k >> 1) & 1) ^ 1, ctl, 0x1C0 + ss);
          __syncwarp();  // the statistics stage is free before anyone writes it
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            sStat[(ss * 2 + 0) * kT + j * 32 + lane] = (rl[j] == -INFINITY) ? -INFINITY : -rl[j];
            sStat[(ss * 2 + 1) * kT + j * 32 + lane] = -rd[j];
          }
          const bool finite = __all_sync(0xFFFFFFFFu, rl[0] != -INFINITY && rl[1] != -INFINITY && rl[2] != -INFINITY &&
                                                          rl[3] != -INFINITY);
          if (lane == 0) sFlag[ss] = finite ? 1 : 0;
          __syncwarp();
          if (lane == 0) mbar_arrive(&st_full[ss]);
          load_stats(k + 2, rl, rd);  // consumed two steps from now
        }
      };
      float la[4], da_[4], lb[4], db[4];
      load_stats(0, la, da_);
      load_stats(1, lb, db);
      for (int k = 0; k < n_it; k += 2) {
        step(k, la, da_);
        if (k + 1 < n_it) step(k + 1, lb, db);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    setmaxnreg_dec<kRegsLo>();
    const bool leader = elect_one();  // the whole warp walks the loop; one lane issues
    if (n_it > 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(kT, kT, false, false);  // both operands K-major
      constexpr uint32_t idesc_mn = make_idesc_bf16(kT, kT, false, true);   // B operand MN-major
      const uint64_t r1d = make_smem_desc(smem_u32(sR1), 16, 1024), r2d = make_smem_desc(smem_u32(sR2), 16, 1024);
      uint64_t x1k[NS1], x2k[NS2], x1m[NS1], x2m[NS2];
#pragma unroll
      for (int s = 0; s < NS1; ++s) {
        x1k[s] = make_smem_desc(smem_u32(x1_stage(s)), 16, 1024);
        x1m[s] = make_smem_desc(smem_u32(x1_stage(s)), kT * 128, 1024);
      }
#pragma unroll
      for (int s = 0; s < NS2; ++s) {
        x2k[s] = make_smem_desc(smem_u32(x2_stage(s)), 16, 1024);
        x2m[s] = make_smem_desc(smem_u32(x2_stage(s)), kT * 128, 1024);
      }
      // register selects instead of runtime-indexed arrays (which would live in local memory)
      auto pick1 = [](const uint64_t (&d)[NS1], int st) { return st == 0 ? d[0] : st == 1 ? d[1] : d[2]; };
      auto pick2 = [](const uint64_t (&d)[NS2], int st) { return st == 0 ? d[0] : (st == 1 || NS2 == 2) ? d[1] : d[NS2 - 1]; };
      const uint32_t t1 = tmem_base + kColT1, t2 = tmem_base + kColT2;
      if constexpr (MODE == kDq) {
        mbar_wait(rt_full, 0, ctl, 0x210);
      } else {
        mbar_wait(res_full, 0, ctl, 0x200);
      }
      // T1 = R1 X1^T, T2 = R2 X2^T
      auto gemm_t1 = [&](uint64_t xd) {
        if constexpr (MODE == kDq) gemm_tk(t1, tmem_base + kColR1, xd, idesc_kk, leader);
        else gemm_ss(t1, r1d, xd, idesc_kk, leader);
      };
      auto gemm_t2 = [&](uint64_t xd) {
        if constexpr (MODE == kDq) gemm_tk(t2, tmem_base + kColR2, xd, idesc_kk, leader);
        else gemm_ss(t2, r2d, xd, idesc_kk, leader);
      };
      mbar_wait(&x_full[0], 0, ctl, 0x300);
      tc_fence_after_sync();
      gemm_t1(x1k[0]);
      if (leader) umma_commit(t1_full);
      mbar_wait(&x2_full[0], 0, ctl, 0x380);
      tc_fence_after_sync();
      gemm_t2(x2k[0]);
      if (leader) umma_commit(t2_full);
      if constexpr (MODE == kDq) {
        if (leader) umma_commit(&x2_empty[0]);  // V_0 is only read by dP(0)
      }
      for (int k = 0; k < n_it; ++k) {
        const int s1 = k % NS1, sn1 = (k + 1) % NS1;  // stages of iterations k and k + 1 in either ring
        const int s2 = k % NS2, sn2 = (k + 1) % NS2;
        const uint32_t ph1 = static_cast<uint32_t>((k + 1) / NS1) & 1u;  // phases of the "full" barriers of sn1, sn2
        const uint32_t ph2 = static_cast<uint32_t>((k + 1) / NS2) & 1u;
        const bool more = k + 1 < n_it;
        if constexpr (MODE == kDkDv) {
          mbar_wait(ph_full, k & 1, ctl, 0x480);
          tc_fence_after_sync();
          gemm_ts<1>(tmem_base + kColAcc, t1, pick2(x2m, s2), idesc_mn, k > 0, leader);  // dV += P^T dO_i, first half
          mbar_wait(p_full, k & 1, ctl, 0x400);
          tc_fence_after_sync();
          gemm_ts<2>(tmem_base + kColAcc, t1, pick2(x2m, s2), idesc_mn, true, leader);
          if (leader) umma_commit(&x2_empty[s2]);  // last use of dO_i
          if (more) {
            mbar_wait(&x_full[sn1], ph1, ctl, 0x300 + sn1);
            tc_fence_after_sync();
            gemm_t1(pick1(x1k, sn1));  // S^T(k+1)
            if (leader) umma_commit(t1_full);
          }
          mbar_wait(ds_full, k & 1, ctl, 0x500);
          tc_fence_after_sync();
          gemm_ts(tmem_base + kColAcc2, t2, pick1(x1m, s1), idesc_mn, k > 0, leader);  // dK += dS^T Q_i
          if (leader) umma_commit(&x_empty[s1]);
          if (more) {
            mbar_wait(&x2_full[sn2], ph2, ctl, 0x380 + sn2);
            tc_fence_after_sync();
            gemm_t2(pick2(x2k, sn2));  // dP^T(k+1)
            if (leader) umma_commit(t2_full);
          }
        } else {
          if (more) {
            mbar_wait(&x_full[sn1], ph1, ctl, 0x300 + sn1);
            mbar_wait(p_full, k & 1, ctl, 0x400);  // T1 of iteration k has been read
            tc_fence_after_sync();
            gemm_t1(pick1(x1k, sn1));  // S(k+1)
            if (leader) umma_commit(t1_full);
          }
          mbar_wait(ds_full, k & 1, ctl, 0x500);
          tc_fence_after_sync();
          gemm_ts(tmem_base + kColAcc, t2, pick1(x1m, s1), idesc_mn, k > 0, leader);  // dQ += dS K_j
          if (leader) umma_commit(&x_empty[s1]);
          if (more) {
            mbar_wait(&x2_full[sn2], ph2, ctl, 0x380 + sn2);
            tc_fence_after_sync();
            gemm_t2(pick2(x2k, sn2));  // dP(k+1)
            if (leader) umma_commit(t2_full);
            if (leader) umma_commit(&x2_empty[sn2]);  // V_j is only read by dP
          }
        }
      }
      if (leader) umma_commit(acc_full);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ compute
    setmaxnreg_inc<kRegsHi>();
    const int h = (warp - 4) >> 2;                  // column half
    const int lane_row = ((warp & 3) << 5) + lane;  // TMEM lane = row of the resident tile
    const int res_row = r0 + lane_row;              // key (kDkDv) or query (kDq) position
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const uint32_t t1 = tmem_base + lane_addr + kColT1 + h * 64, t2 = tmem_base + lane_addr + kColT2 + h * 64;
    const float c = p.scale_log2;
    const uint64_t c2 = f2_pack(c, c);
    float my_lse = INFINITY, my_delta = 0.f;
    if constexpr (MODE == kDq) {
      if (res_row < p.Sq && n_it > 0) {
        my_lse = p.lse[batch * p.ls[0] + head * p.ls[1] + res_row];
        my_delta = p.delta[batch * p.dls[0] + head * p.dls[1] + res_row];
        if (my_lse == -INFINITY) my_lse = INFINITY;
      }
    }
    const uint64_t my_nl2 = f2_pack(-my_lse, -my_lse), my_nd2 = f2_pack(-my_delta, -my_delta);
    const bool emu_ok = __all_sync(0xFFFFFFFFu, my_lse != INFINITY);  // warp-uniform
    if constexpr (MODE == kDq) {
      if (n_it > 0) {  // one-time copy of the resident tiles into TMEM: half 0 takes Q, half 1 takes dO
        mbar_wait(res_full, 0, ctl, 0x220);
        copy_row_to_tmem(h == 0 ? sR1 : sR2, lane_row, tmem_base + lane_addr + (h == 0 ? kColR1 : kColR2));
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(rt_full);
      }
    }
    for (int k = 0; k < n_it; ++k) {
      const int s = k & 1;  // statistics stage (mode kDkDv, two-deep ring)
      const int x0 = (it_begin + k - (k / n_div) * n_tile) * kT + h * 64;  // global position of this thread's first column
      if constexpr (MODE == kDkDv) mbar_wait(&st_full[s], (k >> 1) & 1, ctl, 0x600 + s);
      const ulonglong2* st_l = reinterpret_cast<const ulonglong2*>(sStat + (s * 2 + 0) * kT + h * 64);
      const ulonglong2* st_d = reinterpret_cast<const ulonglong2*>(sStat + (s * 2 + 1) * kT + h * 64);
      // key n visible to query m iff n <= m + off
      bool need_mask;
      int lim;  // kDkDv: first visible column; kDq: last visible column (relative to this thread's 64)
      if constexpr (MODE == kDkDv) {
        need_mask = p.causal && (r0 + kT - 1 > x0 + p.causal_off);
        lim = res_row - p.causal_off - x0;
      } else {
        need_mask = p.causal && (x0 + 63 > r0 + p.causal_off);
        lim = res_row + p.causal_off - x0;
      }
      // ---- P = exp2(S c - lse)
      mbar_wait(t1_full, k & 1, ctl, 0x700);
      tc_fence_after_sync();
      uint32_t pv[64];  // scores, then probabilities (fp32 bit patterns)
      tmem_ld32(t1, pv);
      tmem_ld32(t1 + 32, pv + 32);
      tmem_wait_ld();
      if constexpr (MODE == kDq) {  // nothing is written back into T1: the next S may overwrite it right away
        tc_fence_before_sync();
        mbar_arrive(p_full);
      }
      // Masked scores become -inf before the loop, so that the loop itself carries no mask test.
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (MODE == kDkDv ? (j < lim) : (j > lim)) pv[j] = 0xFF800000u;
      }
      // Two copies of the loop (a run-time test inside it costs more than it saves): every fourth (dQ pass) or third
      // (dK/dV pass) pair of exponentials runs on the FMA pipe, unless the tile is masked or holds a row without keys:
      // those need the MUFU's exact 0 for -inf. Measured per tile: 1230 -> 1030 cycles for the 64 exponentials of a
      // thread, which the 16-per-clock MUFU otherwise bounds at 1024.
      auto p_block = [&](auto emu_tag, auto half_tag) {
        constexpr bool EMU = decltype(emu_tag)::value;
        constexpr int I0 = decltype(half_tag)::value * 32;
#pragma unroll
      for (int i = I0; i < I0 + 32; i += 4) {
        uint64_t nl2[2];
        if constexpr (MODE == kDkDv) {
          const ulonglong2 lv = st_l[i >> 2];
          nl2[0] = lv.x; nl2[1] = lv.y;
        } else {
          nl2[0] = nl2[1] = my_nl2;
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int j = i + 2 * u;
          float a0, a1;
          f2_unpack(f2_fma(f2_pack(__uint_as_float(pv[j]), __uint_as_float(pv[j + 1])), c2, nl2[u]), a0, a1);
          float p0, p1;
          constexpr int kEvery = (MODE == kDq) ? 4 : 3;  // one pair in kEvery runs on the FMA pipe
          if (EMU && ((j >> 1) % kEvery) == 0) {
            exp2_poly2(a0, a1, p0, p1);
          } else {
            p0 = fast_exp2(a0);
            p1 = fast_exp2(a1);
          }
          pv[j] = __float_as_uint(p0);
          pv[j + 1] = __float_as_uint(p1);
        }
      }
      };
      bool emu_now = emu_ok && !need_mask;
      if constexpr (MODE == kDkDv) emu_now = sFlag[s] != 0 && !need_mask;  // every query of the tile has a finite lse
      using H0 = std::integral_constant<int, 0>;
      using H1 = std::integral_constant<int, 1>;
      if (emu_now) p_block(std::true_type{}, H0{});
      else p_block(std::false_type{}, H0{});
      if constexpr (MODE == kDkDv) {  // first half of this thread's columns: dV may start on it
        uint32_t pa[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pa[i] = pack_bf16(__uint_as_float(pv[2 * i]), __uint_as_float(pv[2 * i + 1]));
        tmem_st16(t1, pa);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(ph_full);
      }
      if (emu_now) p_block(std::true_type{}, H1{});
      else p_block(std::false_type{}, H1{});
      if constexpr (MODE == kDkDv) {
        uint32_t pa[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pa[i] = pack_bf16(__uint_as_float(pv[32 + 2 * i]), __uint_as_float(pv[32 + 2 * i + 1]));
        tmem_st16(t1 + 16, pa);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(p_full);
      }
      // ---- dS = P (dP - delta)
      mbar_wait(t2_full, k & 1, ctl, 0x800);
      tc_fence_after_sync();
      uint32_t dp[64];
      tmem_ld32(t2, dp);
      tmem_ld32(t2 + 32, dp + 32);
      tmem_wait_ld();
      uint32_t da[32];
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        uint64_t nd2[2];
        if constexpr (MODE == kDkDv) {
          const ulonglong2 dv = st_d[i >> 2];
          nd2[0] = dv.x; nd2[1] = dv.y;
        } else {
          nd2[0] = nd2[1] = my_nd2;
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int j = i + 2 * u;
          float g0, g1;
          f2_unpack(f2_mul(f2_pack(__uint_as_float(pv[j]), __uint_as_float(pv[j + 1])),
                           f2_add(f2_pack(__uint_as_float(dp[j]), __uint_as_float(dp[j + 1])), nd2[u])), g0, g1);
          da[j >> 1] = pack_bf16(g0, g1);
        }
      }
      if constexpr (MODE == kDkDv) mbar_arrive(&st_empty[s]);  // last read of this iteration's statistics
      tmem_st32(t2, da);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(ds_full);
    }

    // ---- write-out. dQ as a final result: one CTA owns the whole row block, so it is stored as bf16 directly
    //      (zeros where the block sees no key); everything else: accumulators -> scaled fp32 atomics
    if (MODE == kDq && p.dq_store_bf16) {
      if (n_it > 0) {
        mbar_wait(acc_full, 0, ctl, 0x900);
        tc_fence_after_sync();
      }
      __nv_bfloat16* dstb = reinterpret_cast<__nv_bfloat16*>(p.dq_acc) + batch * p.dqs[0] +
                            static_cast<int64_t>(res_row) * p.dqs[1] + head * p.dqs[2] + h * 64;
      const uint32_t src = tmem_base + lane_addr + kColAcc + h * 64;
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t r[32];
        if (n_it > 0) {
          tmem_ld32(src + cc * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (res_row < p.Sq) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *(reinterpret_cast<uint4*>(dstb + cc * 32) + i) = make_uint4(
                pack_bf16(__uint_as_float(r[8 * i]) * p.scale, __uint_as_float(r[8 * i + 1]) * p.scale),
                pack_bf16(__uint_as_float(r[8 * i + 2]) * p.scale, __uint_as_float(r[8 * i + 3]) * p.scale),
                pack_bf16(__uint_as_float(r[8 * i + 4]) * p.scale, __uint_as_float(r[8 * i + 5]) * p.scale),
                pack_bf16(__uint_as_float(r[8 * i + 6]) * p.scale, __uint_as_float(r[8 * i + 7]) * p.scale));
        }
      }
    } else if (n_it > 0) {
      mbar_wait(acc_full, 0, ctl, 0x900);
      tc_fence_after_sync();
      float* dst;
      uint32_t src;
      float scl;
      int ncols;
      bool ok;
      if constexpr (MODE == kDkDv) {
        ok = res_row < p.Sk;
        ncols = 128;
        if (h == 0) {
          dst = p.dv_acc + batch * p.dvs[0] + static_cast<int64_t>(res_row) * p.dvs[1] + kv_head * p.dvs[2];
          src = tmem_base + lane_addr + kColAcc;
          scl = 1.0f;
        } else {
          dst = p.dk_acc + batch * p.dks[0] + static_cast<int64_t>(res_row) * p.dks[1] + kv_head * p.dks[2];
          src = tmem_base + lane_addr + kColAcc2;
          scl = p.scale;
        }
      } else {
        ok = res_row < p.Sq;
        ncols = 64;
        dst = p.dq_acc + batch * p.dqs[0] + static_cast<int64_t>(res_row) * p.dqs[1] + head * p.dqs[2] + h * 64;
        src = tmem_base + lane_addr + kColAcc + h * 64;
        scl = p.scale;
      }
      for (int cc = 0; cc < ncols / 32; ++cc) {
        uint32_t r[32];
        tmem_ld32(src + cc * 32, r);
        tmem_wait_ld();
        if (ok) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            atomicAdd(reinterpret_cast<float4*>(dst + cc * 32) + i,
                      make_float4(__uint_as_float(r[4 * i]) * scl, __uint_as_float(r[4 * i + 1]) * scl,
                                  __uint_as_float(r[4 * i + 2]) * scl, __uint_as_float(r[4 * i + 3]) * scl));
        }
      }
    }
  } else {
    setmaxnreg_dec<kRegsLo>();  // warps 2 and 3 only give their registers away
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    // Something gave up waiting: let copies and MMAs still in flight drain before the
    // shared memory and TMEM of this CTA are handed back.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) __nanosleep(1000);
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int MODE>
static int launch(const pith_attn_bwd_args* a, const BwdParams& p, cudaStream_t st) {
  CUtensorMap tq, tk, tv, tdo;
  if (int rc = make_tensor_map(&tq, a->q, 2, a->B, a->Sq, a->Hq, a->Dqk, a->q_stride, 64, kT)) return rc;
  if (int rc = make_tensor_map(&tdo, a->dout, 2, a->B, a->Sq, a->Hq, a->Dv, a->do_stride, 64, kT)) return rc;
  if (int rc = make_tensor_map(&tk, a->k, 2, a->B, a->Sk, a->Hkv, a->Dqk, a->k_stride, 64, kT)) return rc;
  if (int rc = make_tensor_map(&tv, a->v, 2, a->B, a->Sk, a->Hkv, a->Dv, a->v_stride, 64, kT)) return rc;
  auto kern = attn_bwd128_kernel<MODE>;
  PITH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kAlloc));
  if (MODE == kDkDv) {
    // Query heads of one GQA group per CTA (1, 2 or 4): each CTA pays ~1700 cycles of prologue and ~8700 of fp32
    // write-out around ~2650 cycles per streamed tile, so fewer, longer CTAs win as long as the launch stays balanced.
    // Non-causal: all CTAs are equal, the cost is waves x CTA length. Causal: CTAs go heaviest first, the cost is the
    // work per SM as long as the heaviest CTA stays below 0.6 of it.
    const int tiles = (a->Sk + kT - 1) / kT, qtiles = (a->Sq + kT - 1) / kT, group = a->Hq / a->Hkv;
    constexpr double kIter = 2650.0, kFixed = 10400.0, kSMs = 148.0;
    double iters = 0.0, heaviest = 0.0;  // streamed tiles over the key tiles of one head; of the heaviest key tile
    for (int t = 0; t < tiles; ++t) {
      const int first = a->causal ? (t * kT - a->causal_offset > 0 ? (t * kT - a->causal_offset) / kT : 0) : 0;
      const double n = qtiles > first ? qtiles - first : 0;
      iters += n;
      heaviest = n > heaviest ? n : heaviest;
    }
    BwdParams pk = p;
    pk.hpc = 1;
    double best = 0.0;
    for (int hpc = 1; hpc <= 4; hpc *= 2) {
      if (group % hpc != 0) break;
      const double ctas = static_cast<double>(tiles) * a->Hq * a->B / hpc;
      double cost;
      if (!a->causal) {
        const double waves = static_cast<double>(static_cast<int64_t>((ctas + kSMs - 1) / kSMs));
        cost = waves * (hpc * heaviest * kIter + kFixed);
      } else {
        cost = (static_cast<double>(a->Hq) * a->B * iters * kIter + ctas * kFixed) / kSMs;
        if (hpc > 1 && hpc * heaviest * kIter > 0.6 * cost) break;
      }
      if (hpc == 1 || cost < best) {
        best = cost;
        pk.hpc = hpc;
      }
    }
    dim3 grid(tiles, a->Hq / pk.hpc, a->B);
    kern<<<grid, kThreads, Smem::kAlloc, st>>>(tk, tv, tq, tdo, pk);
  } else {
    dim3 grid((a->Sq + kT - 1) / kT, a->Hq, a->B);
    kern<<<grid, kThreads, Smem::kAlloc, st>>>(tq, tdo, tk, tv, p);
  }
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace bwd128

int launch_bwd_d128(const pith_attn_bwd_args* a, const BwdParams& p, int mode, cudaStream_t st) {
  return mode == kDkDv ? bwd128::launch<kDkDv>(a, p, st) : bwd128::launch<kDq>(a, p, st);
}

}  // namespace pith
