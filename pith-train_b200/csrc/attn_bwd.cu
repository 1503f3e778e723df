// Attention backward for sm_100a, generic variant (used for the MLA head dimensions 192 / 128; head
// dimension 128 takes the wider-tile kernel in attn_bwd128.cu). One kernel template, two modes, both built from the same
// pipeline: a 128-row tile stays resident in shared memory, 64-row tiles stream past it through
// a TMA ring, tcgen05 MMAs produce two [128 x 64] fp32 tiles in TMEM, two warpgroups turn them
// into bf16 operands (written back into TMEM) and a second round of MMAs accumulates the result.
//
//   mode kDkDv: resident K_n, V_n (128 keys); streamed Q_i, dO_i (64 queries)
//       T1 = K Q_i^T (= S^T)      T2 = V dO_i^T (= dP^T)          lane = key, column = query
//       A1 = P^T = exp2(T1 c - lse)     A2 = dS^T = P^T (T2 - delta)
//       dV += A1 dO_i             dK += A2 Q_i
//   mode kDq:   resident Q_m, dO_m (128 queries); streamed K_j, V_j (64 keys)
//       T1 = Q K_j^T (= S)        T2 = dO V_j^T (= dP)            lane = query, column = key
//       A2 = dS = exp2(T1 c - lse) (T2 - delta)
//       dQ += A2 K_j
// lse is the log2-domain LSE of the COMPLETE softmax row and delta = rowsum(O dO), so one
// (Q block, KV block) pair of a ring step yields exactly its share of the gradients.
// Results are scaled (dK, dQ by softmax_scale) and added to fp32 accumulators with vector
// atomics, so ring steps and the query heads of a GQA group round to bf16 only once.
//
// Warp roles (384 threads): warp 0 TMA producer (+ the per-query statistics of the streamed tile
// in mode kDkDv, loaded two iterations ahead), warp 1 MMA issuer, warps 4..7 / 8..11 two compute groups.
//   mode kDq: two TMEM buffers; the groups alternate iterations, so the tensor core works on one iteration
//     while the other is in the exponentials.
//   mode kDkDv: the 192 + 128 accumulator columns leave room for one buffer, so both groups work on every
//     tile (32 of its 64 columns each), the packed operands A1 / A2 get 64 columns of their own, and the next
//     tile's T GEMMs are issued as soon as the buffer has been loaded into registers.
// The two streamed tensors have separate TMA rings (X1: four stages, X2: three).
//
// TMEM columns, mode kDq: buffer b at [128 b, 128 b + 128): T1 in the first 64 columns, T2 in the last 64,
// A2 (packed bf16) overlays the first 32 columns of T2; dQ accumulator at [256, 448).
// Mode kDkDv: T1 [0, 64), T2 [64, 128), A1 [128, 160), A2 [160, 192), dV [192, 320), dK [320, 512).
#include "../../include/pith_b200.h"
#include "common.cuh"
#include <mutex>

#include "attn_bwd_common.h"
#include "host_common.h"

namespace pith {

constexpr int kBwdThreads = 384;
constexpr int kBwdRegsLo = 72;   // producer / MMA-issuer warpgroup
constexpr int kBwdRegsHi = 208;  // compute warpgroups (128 * 72 + 256 * 208 <= 384 * 168, the launch allocation)
constexpr int kRes = 128;  // rows of the resident tile (= TMEM lanes)
constexpr int kStr = 64;   // rows of a streamed tile (= columns of T1 / T2)


template <int DQK, int MODE>
struct BwdCfg {
  static constexpr int NBUF = (MODE == kDkDv && DQK == 192) ? 1 : 2;
  // Ring depths: X1 (Q_i / K_j) is read by the first GEMM of an iteration and by its last, X2 (dO_i / V_j) is released
  // earlier; a reload is a TMA round trip of ~2000 cycles, more than an iteration, so X1 gets the deeper ring.
  static constexpr int NS1 = 4;
  static constexpr int NS2 = 3;
  static constexpr int kR1 = kRes * DQK * 2;
  static constexpr int kR2 = kRes * 128 * 2;
  static constexpr int kX1 = kStr * DQK * 2;
  static constexpr int kX2 = kStr * 128 * 2;
  static constexpr int kR1Off = 0;
  static constexpr int kR2Off = kR1Off + kR1;
  static constexpr int kX1Off = kR2Off + kR2;
  static constexpr int kX2Off = kX1Off + NS1 * kX1;
  static constexpr int kStatOff = kX2Off + NS2 * kX2;        // [NS1][2][64] floats
  static constexpr int kBarOff = kStatOff + NS1 * 2 * kStr * 4;
  static constexpr int kNumBars = 1 + 2 * NS1 + 2 * NS2 + 2 + 2 + 1 + 2;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;
  static constexpr int kAlloc = kTotal;  // no slack: the kernel checks that the dynamic window starts 1024-aligned
  static_assert(kAlloc <= 232448, "shared memory budget");
  // With a single buffer (the 192 + 128 accumulator columns of mode kDkDv leave 192), the packed operands A1 / A2 get
  // 64 columns of their own behind it: the next iteration's T GEMMs may overwrite the buffer as soon as the compute
  // group has loaded it, instead of after the accumulating GEMMs have read A1 / A2 out of it.
  static constexpr bool kSplitA = NBUF == 1;
  static constexpr int kACol = 128;
  static constexpr int kAccCol = kSplitA ? 192 : NBUF * 128;  // first accumulator column
};

template <int DQK, int MODE>
__global__ void __launch_bounds__(kBwdThreads, 1)
    attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_r1, const __grid_constant__ CUtensorMap tm_r2,
                    const __grid_constant__ CUtensorMap tm_x1, const __grid_constant__ CUtensorMap tm_x2,
                    const BwdParams p) {
  using C = BwdCfg<DQK, MODE>;
  constexpr int NBUF = C::NBUF, NS1 = C::NS1, NS2 = C::NS2;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sR1 = smem + C::kR1Off;
  uint8_t* sR2 = smem + C::kR2Off;
  uint8_t* sX1 = smem + C::kX1Off;
  uint8_t* sX2 = smem + C::kX2Off;
  float* sStat = reinterpret_cast<float*>(smem + C::kStatOff);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kBarOff);
  uint64_t* res_full = bars;
  uint64_t* x_full = bars + 1;        // X1 (+ statistics in kDkDv)
  uint64_t* x_empty = x_full + NS1;
  uint64_t* x2_full = x_empty + NS1;  // X2
  uint64_t* x2_empty = x2_full + NS2;
  uint64_t* t_full = x2_empty + NS2;  // [2], by compute group
  uint64_t* a_full = t_full + 2;     // [2]
  uint64_t* acc_full = a_full + 2;
  uint64_t* t_read = acc_full + 1;  // kSplitA: the buffer has been loaded into registers
  uint64_t* a_free = t_read + 1;    // kSplitA: the accumulating GEMMs have read A1 / A2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortCtl ctl{p.status, abort_flag};

  int tile_i, head;
  launch_order(blockIdx.x, gridDim.x, p.causal != 0, tile_i, head);
  const int batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  // Tile of the resident operand and the range of streamed tiles it meets.
  int r0, it_begin, it_end;
  if constexpr (MODE == kDkDv) {
    r0 = tile_i * kRes;  // first key; small r0 = most work, launched first
    it_begin = p.causal ? max(0, r0 - p.causal_off) / kStr : 0;
    it_end = (p.Sq + kStr - 1) / kStr;
  } else {
    r0 = (gridDim.x - 1 - tile_i) * kRes;  // first query; late queries first
    it_begin = 0;
    it_end = (p.Sk + kStr - 1) / kStr;
    if (p.causal) {
      const int last_key = min(r0 + kRes - 1, p.Sq - 1) + p.causal_off;
      it_end = last_key < 0 ? 0 : min(it_end, last_key / kStr + 1);
    }
  }
  int n_it = max(0, it_end - it_begin);

  if (threadIdx.x == 0) {
    // a launch that finds an error already recorded (by an earlier CTA or launch) does no work
    *abort_flag = (p.status != nullptr && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) ? 1u : 0u;
    mbar_init(res_full, 1);
    for (int i = 0; i < NS1; ++i) {
      mbar_init(&x_full[i], MODE == kDkDv ? 2 : 1);
      mbar_init(&x_empty[i], 1);
    }
    for (int i = 0; i < NS2; ++i) {
      mbar_init(&x2_full[i], 1);
      mbar_init(&x2_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&t_full[i], 1);
      mbar_init(&a_full[i], C::kSplitA ? 256 : 128);
    }
    mbar_init(acc_full, 1);
    mbar_init(t_read, 256);
    mbar_init(a_free, 1);
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
  const int x_head = (MODE == kDkDv) ? head : kv_head;   // head index of the streamed tensors

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    setmaxnreg_dec<kBwdRegsLo>();
    if (n_it > 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tm_r1);
        tma_prefetch_desc(&tm_r2);
        tma_prefetch_desc(&tm_x1);
        tma_prefetch_desc(&tm_x2);
        mbar_arrive_expect_tx(res_full, C::kR1 + C::kR2);
#pragma unroll
        for (int sub = 0; sub < DQK / 64; ++sub)
          tma_load_4d(sR1 + sub * (kRes * 128), &tm_r1, res_full, sub * 64, r1_head, r0, batch);
#pragma unroll
        for (int sub = 0; sub < 2; ++sub)
          tma_load_4d(sR2 + sub * (kRes * 128), &tm_r2, res_full, sub * 64, r1_head, r0, batch);
      }
      // Statistics of the 64 streamed queries (kDkDv): raw lse / delta of iteration k are loaded two iterations ahead
      // into registers (a plain global load takes thousands of cycles next to the TMA traffic, and the stage's "full"
      // barrier waits for them) and written to the stage as -lse (+inf -> -inf where the row does not exist or saw
      // no key) and -delta.
      auto load_stats = [&](int k, float (&rl)[2], float (&rd)[2]) {
        if constexpr (MODE == kDkDv) {
          const int x0 = (it_begin + k) * kStr;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int m = x0 + j * 32 + lane;
            rl[j] = INFINITY;
            rd[j] = 0.f;
            if (k < n_it && m < p.Sq) {
              rl[j] = p.lse[batch * p.ls[0] + head * p.ls[1] + m];
              rd[j] = p.delta[batch * p.dls[0] + head * p.dls[1] + m];
              if (rl[j] == -INFINITY) rl[j] = INFINITY;
            }
          }
        }
      };
      auto step = [&](int k, float (&rl)[2], float (&rd)[2]) {
        const int s = k % NS1, s2 = k % NS2;
        const int x0 = (it_begin + k) * kStr;
        if (lane == 0) {
          mbar_wait(&x_empty[s], ((k / NS1) & 1) ^ 1, ctl, 0x100 + s);
          mbar_arrive_expect_tx(&x_full[s], C::kX1);
#pragma unroll
          for (int sub = 0; sub < DQK / 64; ++sub)
            tma_load_4d(sX1 + s * C::kX1 + sub * (kStr * 128), &tm_x1, &x_full[s], sub * 64, x_head, x0, batch);
          mbar_wait(&x2_empty[s2], ((k / NS2) & 1) ^ 1, ctl, 0x180 + s2);
          mbar_arrive_expect_tx(&x2_full[s2], C::kX2);
#pragma unroll
          for (int sub = 0; sub < 2; ++sub)
            tma_load_4d(sX2 + s2 * C::kX2 + sub * (kStr * 128), &tm_x2, &x2_full[s2], sub * 64, x_head, x0, batch);
        }
        __syncwarp();  // the X1 stage is free (lane 0 saw x_empty) before anyone writes its statistics
        if constexpr (MODE == kDkDv) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            sStat[(s * 2 + 0) * kStr + j * 32 + lane] = -rl[j];  // stored negated: the consumers only ever add them
            sStat[(s * 2 + 1) * kStr + j * 32 + lane] = -rd[j];
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&x_full[s]);
          load_stats(k + 2, rl, rd);  // consumed two steps from now
        }
      };
      float la[2], da_[2], lb[2], db[2];
      load_stats(0, la, da_);
      load_stats(1, lb, db);
      for (int k = 0; k < n_it; k += 2) {
        step(k, la, da_);
        if (k + 1 < n_it) step(k + 1, lb, db);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    setmaxnreg_dec<kBwdRegsLo>();
    const bool leader = elect_one();  // the whole warp walks the loop; one lane issues
    if (n_it > 0) {
      constexpr uint32_t idesc_t = make_idesc_bf16(kRes, kStr, false, false);
      constexpr uint32_t idesc_dv = make_idesc_bf16(kRes, 128, false, true);
      constexpr uint32_t idesc_dqk = make_idesc_bf16(kRes, DQK, false, true);
      // K-major views (T GEMMs) and MN-major views (accumulating GEMMs) of the tiles; later K-steps and ring
      // stages only move the start-address field.
      const uint64_t r1d = make_smem_desc(smem_u32(sR1), 16, 1024), r2d = make_smem_desc(smem_u32(sR2), 16, 1024);
      const uint64_t x1k = make_smem_desc(smem_u32(sX1), 16, 1024), x2k = make_smem_desc(smem_u32(sX2), 16, 1024);
      const uint64_t x1m = make_smem_desc(smem_u32(sX1), kStr * 128, 1024);
      const uint64_t x2m = make_smem_desc(smem_u32(sX2), kStr * 128, 1024);
      mbar_wait(res_full, 0, ctl, 0x200);
      auto issue_t = [&](int k) {
        const int s = k % NS1, s2 = k % NS2, b = k % NBUF;
        mbar_wait(&x_full[s], (k / NS1) & 1, ctl, 0x300 + s);
        tc_fence_after_sync();
        const uint32_t t1 = tmem_base + b * 128, t2 = t1 + 64;
        const uint64_t x1s = desc_advance(x1k, s * C::kX1), x2s = desc_advance(x2k, s2 * C::kX2);
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk) {
          const uint32_t sub = kk >> 2, off = (kk & 3) * 32;
          if (leader)
            umma_ss(t1, desc_advance(r1d, sub * (kRes * 128) + off), desc_advance(x1s, sub * (kStr * 128) + off), idesc_t,
                    kk > 0 ? 1u : 0u);
        }
        mbar_wait(&x2_full[s2], (k / NS2) & 1, ctl, 0x380 + s2);
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {
          const uint32_t sub = kk >> 2, off = (kk & 3) * 32;
          if (leader)
            umma_ss(t2, desc_advance(r2d, sub * (kRes * 128) + off), desc_advance(x2s, sub * (kStr * 128) + off), idesc_t,
                    kk > 0 ? 1u : 0u);
        }
        if (leader) umma_commit(&t_full[C::kSplitA ? 0 : (k & 1)]);
        if (MODE == kDq && leader) umma_commit(&x2_empty[s2]);  // V_j is only read by dP
      };
      auto issue_acc = [&](int k) {
        const int s = k % NS1, s2 = k % NS2, b = k % NBUF;
        if constexpr (C::kSplitA) mbar_wait(&a_full[0], k & 1, ctl, 0x400);
        else mbar_wait(&a_full[k & 1], (k >> 1) & 1, ctl, 0x400 + (k & 1));
        tc_fence_after_sync();
        const uint32_t a1 = C::kSplitA ? tmem_base + C::kACol : tmem_base + b * 128, a2 = a1 + (C::kSplitA ? 32 : 64);
        const uint32_t acc = k > 0 ? 1u : 0u;
        const uint64_t x1s = desc_advance(x1m, s * C::kX1), x2s = desc_advance(x2m, s2 * C::kX2);
        if constexpr (MODE == kDkDv) {
#pragma unroll
          for (int kk = 0; kk < kStr / 16; ++kk)  // dV += P^T dO_i
            if (leader)
              umma_ts(tmem_base + C::kAccCol, a1 + kk * 8, desc_advance(x2s, kk * 2048), idesc_dv, acc | (kk > 0 ? 1u : 0u));
          if (leader) umma_commit(&x2_empty[s2]);  // last use of dO_i
#pragma unroll
          for (int kk = 0; kk < kStr / 16; ++kk)  // dK += dS^T Q_i
            if (leader)
              umma_ts(tmem_base + C::kAccCol + 128, a2 + kk * 8, desc_advance(x1s, kk * 2048), idesc_dqk,
                      acc | (kk > 0 ? 1u : 0u));
        } else {
#pragma unroll
          for (int kk = 0; kk < kStr / 16; ++kk)  // dQ += dS K_j
            if (leader)
              umma_ts(tmem_base + C::kAccCol, a2 + kk * 8, desc_advance(x1s, kk * 2048), idesc_dqk, acc | (kk > 0 ? 1u : 0u));
        }
        if (leader) umma_commit(&x_empty[s]);
        if (C::kSplitA && leader) umma_commit(a_free);
      };
      issue_t(0);
      if constexpr (C::kSplitA) {
        for (int k = 0; k < n_it; ++k) {
          if (k + 1 < n_it) {
            mbar_wait(t_read, k & 1, ctl, 0x480);
            tc_fence_after_sync();
            issue_t(k + 1);
          }
          issue_acc(k);
        }
      } else {
        for (int k = 0; k < n_it; ++k) {
          if (k + 1 < n_it) issue_t(k + 1);
          issue_acc(k);
        }
      }
      if (leader) umma_commit(acc_full);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ compute groups
    setmaxnreg_inc<kBwdRegsHi>();
    const int w = (warp - 4) >> 2;
    const int lane_row = ((warp & 3) << 5) + lane;  // TMEM lane = row of the resident tile
    const int res_row = r0 + lane_row;              // key (kDkDv) or query (kDq) position
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const float c = p.scale_log2;
    float my_lse = INFINITY, my_delta = 0.f;
    if constexpr (MODE == kDq) {
      if (res_row < p.Sq && n_it > 0) {
        my_lse = p.lse[batch * p.ls[0] + head * p.ls[1] + res_row];
        my_delta = p.delta[batch * p.dls[0] + head * p.dls[1] + res_row];
        if (my_lse == -INFINITY) my_lse = INFINITY;
      }
    }
    const uint64_t my_nl2 = f2_pack(-my_lse, -my_lse), my_nd2 = f2_pack(-my_delta, -my_delta);
    if constexpr (C::kSplitA) {
      // Both groups work on every tile, 32 of its 64 columns each: half the latency from the score GEMMs to the
      // accumulating GEMMs, which is what the single buffer makes the iteration wait for.
      const uint64_t c2 = f2_pack(c, c);
      const uint32_t t1 = tmem_base + lane_addr + w * 32, t2 = t1 + 64;
      const uint32_t ta = tmem_base + lane_addr + C::kACol + w * 16;
      for (int k = 0; k < n_it; ++k) {
        const int s = k % NS1;
        const int x0 = (it_begin + k) * kStr + w * 32;  // global position of this thread's first column
        mbar_wait(&x_full[s], (k / NS1) & 1, ctl, 0x500 + s);
        mbar_wait(&t_full[0], k & 1, ctl, 0x600);
        tc_fence_after_sync();
        uint32_t s1[32], s2[32];
        tmem_ld32(t1, s1);
        tmem_ld32(t2, s2);
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(t_read);
        const bool need_mask = p.causal && (r0 + kRes - 1 > x0 + p.causal_off);
        const int lim = res_row - p.causal_off - x0;  // column i visible iff i >= lim
        const uint64_t* st_l = reinterpret_cast<const uint64_t*>(sStat + (s * 2 + 0) * kStr + w * 32);
        const uint64_t* st_d = reinterpret_cast<const uint64_t*>(sStat + (s * 2 + 1) * kStr + w * 32);
        uint32_t pa[16], da[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const uint64_t nl2 = st_l[i >> 1], nd2 = st_d[i >> 1];
          float e0, e1;
          f2_unpack(f2_fma(f2_pack(__uint_as_float(s1[i]), __uint_as_float(s1[i + 1])), c2, nl2), e0, e1);
          float p0 = fast_exp2(e0), p1 = fast_exp2(e1);
          if (need_mask) {
            if (i < lim) p0 = 0.f;
            if (i + 1 < lim) p1 = 0.f;
          }
          float g0, g1;
          f2_unpack(f2_mul(f2_pack(p0, p1), f2_add(f2_pack(__uint_as_float(s2[i]), __uint_as_float(s2[i + 1])), nd2)), g0, g1);
          pa[i >> 1] = pack_bf16(p0, p1);
          da[i >> 1] = pack_bf16(g0, g1);
        }
        if (k > 0) {
          mbar_wait(a_free, (k - 1) & 1, ctl, 0x680);
          tc_fence_after_sync();
        }
        tmem_st16(ta, pa);
        tmem_st16(ta + 32, da);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&a_full[0]);
      }
    } else {
    // two buffers: the groups alternate iterations
    for (int k = w; k < n_it; k += 2) {
      const int s = k % NS1, b = k % NBUF;
      const int x0 = (it_begin + k) * kStr;
      if constexpr (MODE == kDkDv) mbar_wait(&x_full[s], (k / NS1) & 1, ctl, 0x500 + s);
      mbar_wait(&t_full[w], (k >> 1) & 1, ctl, 0x600 + w);
      tc_fence_after_sync();
      const uint32_t t1 = tmem_base + lane_addr + b * 128, t2 = t1 + 64;
      uint32_t s1[kStr], s2[kStr];
      tmem_ld32(t1, s1);
      tmem_ld32(t1 + 32, s1 + 32);
      tmem_ld32(t2, s2);
      tmem_ld32(t2 + 32, s2 + 32);
      tmem_wait_ld();
      // key n visible to query m iff n <= m + off
      bool need_mask;
      int lim;  // kDkDv: first visible column (query) index; kDq: last visible column (key) index
      if constexpr (MODE == kDkDv) {
        need_mask = p.causal && (r0 + kRes - 1 > x0 + p.causal_off);
        lim = res_row - p.causal_off - x0;  // column i visible iff i >= lim
      } else {
        need_mask = p.causal && (x0 + kStr - 1 > r0 + p.causal_off);
        lim = res_row + p.causal_off - x0;  // column i visible iff i <= lim
      }
      const uint64_t* st_l = reinterpret_cast<const uint64_t*>(sStat + (s * 2 + 0) * kStr);  // pairs of -lse
      const uint64_t* st_d = reinterpret_cast<const uint64_t*>(sStat + (s * 2 + 1) * kStr);  // pairs of -delta
      const uint64_t c2 = f2_pack(c, c);
      uint32_t pa[kStr / 2], da[kStr / 2];
#pragma unroll
      for (int i = 0; i < kStr; i += 2) {
        uint64_t nl2, nd2;
        if constexpr (MODE == kDkDv) {
          nl2 = st_l[i >> 1];
          nd2 = st_d[i >> 1];
        } else {
          nl2 = my_nl2;
          nd2 = my_nd2;
        }
        float x0, x1;
        f2_unpack(f2_fma(f2_pack(__uint_as_float(s1[i]), __uint_as_float(s1[i + 1])), c2, nl2), x0, x1);
        float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
        if (need_mask) {
          if constexpr (MODE == kDkDv) {
            if (i < lim) p0 = 0.f;
            if (i + 1 < lim) p1 = 0.f;
          } else {
            if (i > lim) p0 = 0.f;
            if (i + 1 > lim) p1 = 0.f;
          }
        }
        float g0, g1;
        f2_unpack(f2_mul(f2_pack(p0, p1), f2_add(f2_pack(__uint_as_float(s2[i]), __uint_as_float(s2[i + 1])), nd2)), g0, g1);
        pa[i >> 1] = pack_bf16(p0, p1);
        da[i >> 1] = pack_bf16(g0, g1);
      }
      if constexpr (MODE == kDkDv) tmem_st32(t1, pa);
      tmem_st32(t2, da);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&a_full[w]);
    }
    }

    // ---- write-out: accumulators -> scaled fp32 atomics
    if (n_it > 0) {
      mbar_wait(acc_full, 0, ctl, 0x700);
      tc_fence_after_sync();
      if constexpr (MODE == kDkDv) {
        const bool ok = res_row < p.Sk;
        if (w == 0) {
          float* dst = p.dv_acc + batch * p.dvs[0] + static_cast<int64_t>(res_row) * p.dvs[1] + kv_head * p.dvs[2];
#pragma unroll
          for (int cc = 0; cc < 128 / 32; ++cc) {
            uint32_t r[32];
            tmem_ld32(tmem_base + lane_addr + C::kAccCol + cc * 32, r);
            tmem_wait_ld();
            if (ok) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                atomicAdd(reinterpret_cast<float4*>(dst + cc * 32) + i,
                          make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                      __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])));
            }
          }
        } else {
          float* dst = p.dk_acc + batch * p.dks[0] + static_cast<int64_t>(res_row) * p.dks[1] + kv_head * p.dks[2];
#pragma unroll
          for (int cc = 0; cc < DQK / 32; ++cc) {
            uint32_t r[32];
            tmem_ld32(tmem_base + lane_addr + C::kAccCol + 128 + cc * 32, r);
            tmem_wait_ld();
            if (ok) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                atomicAdd(reinterpret_cast<float4*>(dst + cc * 32) + i,
                          make_float4(__uint_as_float(r[4 * i]) * p.scale, __uint_as_float(r[4 * i + 1]) * p.scale,
                                      __uint_as_float(r[4 * i + 2]) * p.scale, __uint_as_float(r[4 * i + 3]) * p.scale));
            }
          }
        }
      } else {
        const bool ok = res_row < p.Sq;
        float* dst = p.dq_acc + batch * p.dqs[0] + static_cast<int64_t>(res_row) * p.dqs[1] + head * p.dqs[2];
        constexpr int kHalf = DQK / 64;  // 32-column chunks per group
#pragma unroll
        for (int cc = w * kHalf; cc < (w + 1) * kHalf; ++cc) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_addr + C::kAccCol + cc * 32, r);
          tmem_wait_ld();
          if (ok) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              atomicAdd(reinterpret_cast<float4*>(dst + cc * 32) + i,
                        make_float4(__uint_as_float(r[4 * i]) * p.scale, __uint_as_float(r[4 * i + 1]) * p.scale,
                                    __uint_as_float(r[4 * i + 2]) * p.scale, __uint_as_float(r[4 * i + 3]) * p.scale));
          }
        }
      }
    }
  }

  else {
    setmaxnreg_dec<kBwdRegsLo>();  // warps 2 and 3 only give their registers away
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) __nanosleep(1000);
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int DQK, int MODE>
static int launch_bwd(const pith_attn_bwd_args* a, const BwdParams& p, cudaStream_t st) {
  using C = BwdCfg<DQK, MODE>;
  CUtensorMap r1, r2, x1, x2;
  const int qrows = MODE == kDkDv ? kStr : kRes;
  const int krows = MODE == kDkDv ? kRes : kStr;
  CUtensorMap tq, tk, tv, tdo;
  if (int rc = make_tensor_map(&tq, a->q, 2, a->B, a->Sq, a->Hq, a->Dqk, a->q_stride, 64, qrows)) return rc;
  if (int rc = make_tensor_map(&tdo, a->dout, 2, a->B, a->Sq, a->Hq, a->Dv, a->do_stride, 64, qrows)) return rc;
  if (int rc = make_tensor_map(&tk, a->k, 2, a->B, a->Sk, a->Hkv, a->Dqk, a->k_stride, 64, krows)) return rc;
  if (int rc = make_tensor_map(&tv, a->v, 2, a->B, a->Sk, a->Hkv, a->Dv, a->v_stride, 64, krows)) return rc;
  int tiles;
  if (MODE == kDkDv) {
    r1 = tk; r2 = tv; x1 = tq; x2 = tdo;
    tiles = (a->Sk + kRes - 1) / kRes;
  } else {
    r1 = tq; r2 = tdo; x1 = tk; x2 = tv;
    tiles = (a->Sq + kRes - 1) / kRes;
  }
  auto kern = attn_bwd_kernel<DQK, MODE>;
  PITH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kAlloc));
  dim3 grid(tiles, a->Hq, a->B);
  kern<<<grid, kBwdThreads, C::kAlloc, st>>>(r1, r2, x1, x2, p);
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

static bool f32_rows_ok(const void* base, const int64_t st[3]) {
  return aligned16(base) && st[0] % 4 == 0 && st[1] % 4 == 0 && st[2] % 4 == 0;
}

}  // namespace pith

using namespace pith;

namespace {

// Side stream and events (per device, created on first use, kept until exit) for running the dQ pass beside the
// dK/dV pass.
struct ForkJoin {
  std::mutex mu;
  cudaStream_t side = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};

ForkJoin* fork_join_for_current_device() {
  constexpr int kMaxDevices = 64;
  static ForkJoin table[kMaxDevices];
  static std::mutex table_mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    pith::fail(pith::kErrCuda, "cudaGetDevice failed or device index out of range");
    return nullptr;
  }
  std::lock_guard<std::mutex> guard(table_mu);
  ForkJoin* fj = &table[dev];
  if (fj->side == nullptr) {
    cudaStream_t s = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&e0, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&e1, cudaEventDisableTiming) != cudaSuccess) {
      pith::fail(pith::kErrCuda, "could not create the side stream of the backward: %s",
                 cudaGetErrorString(cudaGetLastError()));
      return nullptr;
    }
    fj->fork = e0;
    fj->join = e1;
    fj->side = s;
  }
  return fj;
}

}  // namespace

extern "C" int pith_attn_bwd(const pith_attn_bwd_args* a, void* stream) {
  PITH_REQUIRE(a != nullptr, "null args");
  PITH_REQUIRE(a->q && a->k && a->v && a->dout && a->lse && a->delta, "null tensor pointer");
  const bool want_dq = a->dq_acc != nullptr;
  const bool want_dkv = a->dk_acc != nullptr;
  PITH_REQUIRE((a->dk_acc == nullptr) == (a->dv_acc == nullptr), "dk_acc and dv_acc must be given together");
  PITH_REQUIRE(want_dq || want_dkv, "no gradient accumulator given");
  PITH_REQUIRE(a->B > 0 && a->Sq > 0 && a->Sk > 0 && a->Hq > 0 && a->Hkv > 0, "bad shape B=%d Sq=%d Sk=%d Hq=%d Hkv=%d",
               a->B, a->Sq, a->Sk, a->Hq, a->Hkv);
  PITH_REQUIRE(a->Hq % a->Hkv == 0, "Hq=%d is not a multiple of Hkv=%d", a->Hq, a->Hkv);
  PITH_REQUIRE(a->Dv == 128 && (a->Dqk == 128 || a->Dqk == 192),
               "unsupported head dims Dqk=%d Dv=%d (supported: 128/128 and 192/128)", a->Dqk, a->Dv);
  PITH_REQUIRE(a->softmax_scale > 0.f, "softmax_scale must be positive");
  PITH_REQUIRE(a->Hq <= 65535 && a->B <= 65535, "Hq and B must fit a grid dimension");
  const bool dq_bf16 = want_dq && (a->flags & PITH_BWD_DQ_STORE_BF16);
  PITH_REQUIRE(!dq_bf16 || a->Dqk == 128, "PITH_BWD_DQ_STORE_BF16 is supported for head_dim 128 only");
  PITH_REQUIRE(!dq_bf16 || (aligned16(a->dq_acc) && a->dq_stride[0] % 8 == 0 && a->dq_stride[1] % 8 == 0 &&
                            a->dq_stride[2] % 8 == 0),
               "the bf16 dQ output must be 16-byte aligned with 16-byte-multiple strides");
  PITH_REQUIRE((!want_dq || dq_bf16 || f32_rows_ok(a->dq_acc, a->dq_stride)) &&
                   (!want_dkv || (f32_rows_ok(a->dk_acc, a->dk_stride) && f32_rows_ok(a->dv_acc, a->dv_stride))),
               "gradient accumulators must be 16-byte aligned with 16-byte-multiple strides");
  if (int rc = require_sm100()) return rc;
  BwdParams p;
  p.lse = a->lse; p.delta = a->delta; p.dq_acc = a->dq_acc; p.dk_acc = a->dk_acc; p.dv_acc = a->dv_acc;
  p.status = a->status;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal ? 1 : 0; p.causal_off = a->causal_offset;
  p.dq_store_bf16 = dq_bf16 ? 1 : 0;
  p.hpc = 1;
  p.scale = a->softmax_scale; p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  for (int i = 0; i < 3; ++i) { p.dqs[i] = a->dq_stride[i]; p.dks[i] = a->dk_stride[i]; p.dvs[i] = a->dv_stride[i]; }
  for (int i = 0; i < 2; ++i) { p.ls[i] = a->lse_stride[i]; p.dls[i] = a->delta_stride[i]; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto launch = [&](BwdMode mode, cudaStream_t s) -> int {
    if (a->Dqk == 128) return launch_bwd_d128(a, p, mode, s);
    return mode == kDkDv ? launch_bwd<192, kDkDv>(a, p, s) : launch_bwd<192, kDq>(a, p, s);
  };
  // Side by side pays when a launch is only a few waves long (its partial last wave is a large share); on long
  // launches of the head_dim-128 kernels the two kernels' interleaved CTAs cost more in L2 locality than the tail
  // gives back (measured, 32 heads: 4096 x 2048 non-causal 0.437 -> 0.421 ms, 4096 x 4096 causal 0.439 -> 0.433 ms,
  // 6144 x 6144 causal 0.889 -> 0.932 ms, 8192 x 8192 causal 1.52 -> 1.68 ms). The Dqk = 192 kernels gain at every
  // size measured (16 heads, 8192 x 8192 causal: 1.052 -> 1.018 ms).
  const double work = static_cast<double>(a->B) * a->Hq * a->Sq * a->Sk * (a->causal ? 0.5 : 1.0);
  const double limit = a->Dqk == 128 ? 4.5e8 : 4.0e9;
  const bool side_by_side = (a->flags & PITH_BWD_CONCURRENT) || (!(a->flags & PITH_BWD_SERIAL) && work <= limit);
  if (!(want_dkv && want_dq) || !side_by_side) {
    if (want_dkv)
      if (int rc = launch(kDkDv, st)) return rc;
    if (want_dq)
      if (int rc = launch(kDq, st)) return rc;
    return kOk;
  }
  // The two passes write disjoint accumulators. Every CTA needs a whole SM, so a lone launch ends with a partial
  // wave; issued on two streams the dQ pass fills the SMs the dK/dV pass leaves idle at its tail.
  ForkJoin* fj = fork_join_for_current_device();
  if (fj == nullptr) return kErrCuda;
  std::lock_guard<std::mutex> guard(fj->mu);  // one fork/join sequence at a time: the events are shared
  PITH_CUDA(cudaEventRecord(fj->fork, st));
  PITH_CUDA(cudaStreamWaitEvent(fj->side, fj->fork, 0));
  // Whatever the launches answer, the side stream is joined back: an enclosing stream capture stays valid.
  int rc = launch(kDkDv, st);
  if (rc == kOk) rc = launch(kDq, fj->side);
  PITH_CUDA(cudaEventRecord(fj->join, fj->side));
  PITH_CUDA(cudaStreamWaitEvent(st, fj->join, 0));
  return rc;
}
