// Shared between the attention-forward kernels (one CTA per two query tiles, and the CTA-pair variant):
// launch parameters, the per-row online softmax over the score tiles in TMEM, and the epilogue
// (normalise, optional merge with a previous partial (O, LSE), store).
#pragma once
#include "../../include/pith_b200.h"
#include "common.cuh"
#include "host_common.h"

namespace pith {

struct FwdParams {
  void* o;
  float* lse;
  const float* prev_o;
  const float* prev_lse;
  uint32_t* status;
  int B, Sq, Sk, Hq, Hkv;
  int causal, causal_off;
  int o_fp32, lse_natural;
  float scale_log2;
  int64_t os[3], pos[3];
  int64_t ls[2], pls[2];
};

constexpr int kFwdThreads = 384;
constexpr int kBM = 128;  // query rows per tile
constexpr int kDV = 128;
// Register budget after setmaxnreg: 128 * lo + 256 * hi must stay within the 384 * 168 registers the CTA is launched
// with (a larger request makes setmaxnreg.inc wait forever). 80 / 208 measured 3 % faster than 64 / 216: the MMA
// issuer keeps its descriptors in registers.
constexpr int kFwdRegsLo = 80;   // producer / MMA issuer warpgroup
constexpr int kFwdRegsHi = 208;  // softmax warpgroups: one 128-column score row per thread
static_assert(128 * kFwdRegsLo + 256 * kFwdRegsHi <= kFwdThreads * 168, "setmaxnreg budget exceeds the launch allocation");

// Host side of pith_attn_fwd: fills FwdParams after the argument checks. Defined in attn_fwd.cu.
// The CTA-pair kernel (attn_fwd_pair.cu): pairs of CTAs share every K/V block through one 256-row MMA.
int launch_fwd_pair(const pith_attn_fwd_args* a, const FwdParams& p, cudaStream_t st);

// One softmax warpgroup: thread = query row = TMEM lane. Walks the `nb` score tiles of its query tile
// (S at tS, 128 fp32 columns, P written back over its first 64 columns as packed bf16), keeps the running
// maximum / sum, rescales O (at tO) only when the maximum grows by more than 2^8, then normalises, merges and
// stores. `arrive_p()` tells the MMA issuer that P (and the rescaled O) of this row are in TMEM; `arrive_half()` is
// called when the first 64 keys' P is there (the issuer may start the first half of the PV GEMM under the second
// half of the exponentials; pass a no-op where that is not used).
//   tile_row0 = first query row of the tile, row = this thread's query row (both relative to the Q block).
template <int BN, class ArriveP, class ArriveHalf>
__device__ __forceinline__ void fwd_softmax_rows(const FwdParams& p, const AbortCtl& ctl, uint64_t* s_full,
                                                 uint64_t* o_full, ArriveP arrive_p, ArriveHalf arrive_half, uint32_t tS,
                                                 uint32_t tO,
                                                 int tile_row0, int row, int nb, int head, int batch, uint32_t tag) {
  const float c = p.scale_log2;
  float m_used = -INFINITY;
  float l = 0.f;
  const int64_t po_off = batch * p.pos[0] + static_cast<int64_t>(row) * p.pos[1] + head * p.pos[2];
  for (int j = 0; j < nb; ++j) {
    mbar_wait(s_full, j & 1, ctl, 0x700 + tag);
    tc_fence_after_sync();
    uint32_t sr[BN];
#pragma unroll
    for (int cchunk = 0; cchunk < BN / 32; ++cchunk) tmem_ld32(tS + cchunk * 32, sr + cchunk * 32);
    tmem_wait_ld();
    const int n0 = j * BN;
    const bool need_mask = (p.causal && (n0 + BN - 1 > tile_row0 + p.causal_off)) || (n0 + BN > p.Sk);
    if (need_mask) {
      const int limit = p.causal ? min(p.Sk - 1, row + p.causal_off) : p.Sk - 1;  // last visible key
#pragma unroll
      for (int i = 0; i < BN; ++i)
        if (n0 + i > limit) sr[i] = 0xFF800000u;  // -inf
    }
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // independent chains
#pragma unroll
    for (int i = 0; i < BN; i += 8) {
#pragma unroll
      for (int u = 0; u < 4; ++u)
        mx[u] = fmax3(mx[u], __uint_as_float(sr[i + 2 * u]), __uint_as_float(sr[i + 2 * u + 1]));
    }
    const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
    const float m_new = fmaxf(m_used, m_blk);
    if (j == 0) {
      m_used = m_new;
    } else {
      const bool need = (m_new - m_used) * c > 8.0f;
      if (__any_sync(0xFFFFFFFFu, need)) {
        const float alpha = need ? fast_exp2((m_used - m_new) * c) : 1.0f;
        if (need) m_used = m_new;
        l *= alpha;
#pragma unroll
        for (int cchunk = 0; cchunk < kDV / 32; ++cchunk) {
          uint32_t orr[32];
          tmem_ld32(tO + cchunk * 32, orr);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
          tmem_st32(tO + cchunk * 32, orr);
        }
      }
    }
    const float mc = (m_used == -INFINITY) ? 0.f : m_used * c;
    // scale and sum with fma.f32x2 / add.f32x2: two floats per instruction, four independent partial sums
    const uint64_t c2 = f2_pack(c, c), nmc2 = f2_pack(-mc, -mc);
    uint64_t ls2[2] = {0ull, 0ull};
#pragma unroll
    for (int cchunk = 0; cchunk < BN / 64; ++cchunk) {
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(sr[cchunk * 64 + 2 * i]),
                                           __uint_as_float(sr[cchunk * 64 + 2 * i + 1])), c2, nmc2);
        float x0, x1;
        f2_unpack(x2, x0, x1);
        const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
        ls2[i & 1] = f2_add(ls2[i & 1], f2_pack(p0, p1));
        pk[i] = pack_bf16(p0, p1);
      }
      tmem_st32(tS + cchunk * 32, pk);
      if (cchunk == 0 && BN / 64 > 1) {
        tmem_wait_st();
        tc_fence_before_sync();
        arrive_half();
      }
    }
    float la, lb, lc, ld;
    f2_unpack(ls2[0], la, lb);
    f2_unpack(ls2[1], lc, ld);
    l += (la + lb) + (lc + ld);
    tmem_wait_st();
    tc_fence_before_sync();
    arrive_p();
  }

  // ---- epilogue: normalise, optional merge with a previous partial, store
  const bool row_ok = row < p.Sq;
  // the previous partial's LSE and first 32 columns are requested before the wait for the last PV GEMM; each later
  // chunk is requested before the chunk in front of it is processed
  const bool merge = p.prev_o != nullptr;
  float pl = -INFINITY;
  float4 pq[8];
  const float4* pp = reinterpret_cast<const float4*>(p.prev_o + po_off);
  if (merge && row_ok) {
    pl = p.prev_lse[batch * p.pls[0] + head * p.pls[1] + row];
#pragma unroll
    for (int i = 0; i < 8; ++i) pq[i] = pp[i];
  }
  if (nb > 0) {
    mbar_wait(o_full, 0, ctl, 0x800 + tag);
    tc_fence_after_sync();
  }
  float inv = (l > 0.f) ? 1.0f / l : 0.f;
  float lse2 = (l > 0.f) ? fmaf(m_used, c, fast_log2(l)) : -INFINITY;
  float w_prev = 0.f;
  if (merge) {
    const float mx = fmaxf(pl, lse2);
    if (mx > -INFINITY) {
      const float e1 = exp2f(pl - mx), e2 = exp2f(lse2 - mx);
      const float den = e1 + e2;
      w_prev = e1 / den;
      inv *= e2 / den;
      lse2 = mx + log2f(den);
    }
  }
  if (row_ok) p.lse[batch * p.ls[0] + head * p.ls[1] + row] = p.lse_natural ? lse2 * 0.6931471805599453f : lse2;
  const int64_t o_off = batch * p.os[0] + static_cast<int64_t>(row) * p.os[1] + head * p.os[2];
#pragma unroll
  for (int cchunk = 0; cchunk < kDV / 32; ++cchunk) {
    uint32_t orr[32];
    if (nb > 0) {
      tmem_ld32(tO + cchunk * 32, orr);
      tmem_wait_ld();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) orr[i] = 0u;
    }
    if (row_ok) {
      float ov[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) ov[i] = __uint_as_float(orr[i]) * inv;
      if (merge) {
        float4 cur[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) cur[i] = pq[i];
        if (cchunk + 1 < kDV / 32) {
#pragma unroll
          for (int i = 0; i < 8; ++i) pq[i] = pp[(cchunk + 1) * 8 + i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 x = cur[i];
          ov[4 * i] = fmaf(w_prev, x.x, ov[4 * i]);
          ov[4 * i + 1] = fmaf(w_prev, x.y, ov[4 * i + 1]);
          ov[4 * i + 2] = fmaf(w_prev, x.z, ov[4 * i + 2]);
          ov[4 * i + 3] = fmaf(w_prev, x.w, ov[4 * i + 3]);
        }
      }
      if (p.o_fp32) {
        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.o) + o_off + cchunk * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = make_float4(ov[4 * i], ov[4 * i + 1], ov[4 * i + 2], ov[4 * i + 3]);
      } else {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.o) + o_off + cchunk * 32);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          dst[i] = make_uint4(pack_bf16(ov[8 * i], ov[8 * i + 1]), pack_bf16(ov[8 * i + 2], ov[8 * i + 3]),
                              pack_bf16(ov[8 * i + 4], ov[8 * i + 5]), pack_bf16(ov[8 * i + 6], ov[8 * i + 7]));
      }
    }
  }
}

}  // namespace pith
