// Attention forward on CTA pairs (sm_100a, tcgen05 with cta_group::2).
//
// Two CTAs (a cluster of 2) run every MMA together: the accumulator has 256 rows, 128 in each CTA's TMEM, each CTA
// supplies its own 128 rows of the A operand (Q from its shared memory, P from its TMEM) and only HALF of the B
// operand: 64 of the block's 128 keys for S = Q K^T, 64 of the 128 value columns for O += P V. What that buys is
// capacity, not MMA rate (a cta_group::2 MMA costs the same 64 cycles per K-step as a single-CTA one, and the single-CTA
// kernel is not short of shared-memory bandwidth): K/V stages are half as large, so the 192-wide MLA heads get a
// second V stage that does not fit next to 96 KB of Q in one CTA, and the L2 -> SM stream per CTA halves. Measured:
// faster for Dqk = 192 (0.338 -> 0.269 ms at 16 heads x 8192^2 causal), slower for Dqk = 128 (0.431 -> 0.477 ms),
// which therefore stays on the single-CTA kernel.
//
// A pair owns 512 consecutive query rows of one (batch, head): CTA c holds rows [(2t + c) * 128, +128) as its
// tile t (t = 0, 1), so that tile t of both CTAs forms one 256-row MMA. Warp roles as in the single-CTA kernel
// (warp 0 TMA producer, warp 1 MMA issuer, warps 4..7 / 8..11 softmax of tile 0 / 1), with these differences:
//   * only rank 0 issues MMAs; its commits arrive on the barriers of both CTAs;
//   * both producers load their halves into their own shared memory, the bytes are counted by rank 0's
//     "full" barriers (plain TMA loads with a remote barrier: no multicast);
//   * the softmax threads of both CTAs arrive on rank 0's "P ready" barriers (256 arrivals each).
// Under a causal mask rank 0's tiles end one block before rank 1's; they run the extra, fully masked block.
// Every wait is bounded; the two CTAs meet at a cluster barrier before the TMEM is released.
#include "attn_fwd_common.cuh"

namespace pith {

constexpr int kPairBN = 128;  // keys per block (64 per CTA)

template <int DQK, int KST, int VST>
struct FwdPairSmem {
  static constexpr int kQTile = kBM * DQK * 2;          // one 128-row Q tile
  static constexpr int kKHalf = (kPairBN / 2) * DQK * 2;  // this CTA's 64 keys of a block
  static constexpr int kVHalf = kPairBN * (kDV / 2) * 2;  // this CTA's 64 value columns of a block
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + 2 * kQTile;
  static constexpr int kVOff = kKOff + KST * kKHalf;
  static constexpr int kBarOff = kVOff + VST * kVHalf;
  static constexpr int kNumBars = 1 + 2 * KST + 2 * VST + 8;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;
  static constexpr int kAlloc = kTotal + 1024;
};

// S[256 x 128] = Q[256 x DQK] K_blk[128 x DQK]^T over the pair. Per CTA: Q tile = DQK/64 sub-tiles of
// [128][64] (16 KB apart), K half = DQK/64 sub-tiles of [64][64] (8 KB apart), all K-major, 128-byte swizzle.
template <int DQK>
__device__ __forceinline__ void issue_qk_pair(uint32_t d_tmem, uint64_t qdesc, uint64_t kdesc, uint32_t idesc,
                                              bool leader) {
#pragma unroll
  for (int kk = 0; kk < DQK / 16; ++kk) {
    const uint32_t sub = kk >> 2, off = (kk & 3) * 32;
    if (leader)
      umma_ss_pair(d_tmem, desc_advance(qdesc, sub * (kBM * 128) + off),
                   desc_advance(kdesc, sub * ((kPairBN / 2) * 128) + off), idesc, kk > 0 ? 1u : 0u);
  }
}
// O[256 x 128] (+)= P[256 x 128] (bf16 in each CTA's TMEM) V_blk[128 x 128]; per CTA V half = [128 keys][64 columns]
// MN-major (one 64-wide column block), 16 keys = 2048 bytes per K-step.
// K-steps [K0, K1) of the block's 8: the first half can run as soon as the first 64 keys' P has been stored.
template <int K0, int K1>
__device__ __forceinline__ void issue_pv_pair(uint32_t d_tmem, uint32_t p_tmem, uint64_t vdesc, uint32_t idesc,
                                              bool acc, bool leader) {
#pragma unroll
  for (int kk = K0; kk < K1; ++kk)
    if (leader) umma_ts_pair(d_tmem, p_tmem + kk * 8, desc_advance(vdesc, kk * 2048), idesc, (acc || kk > 0) ? 1u : 0u);
}

template <int DQK, int KST, int VST>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kFwdThreads, 1)
    attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using L = FwdPairSmem<DQK, KST, VST>;
  constexpr int BN = kPairBN;
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared memory window starts at the same offset in both CTAs, so the aligned offsets agree too
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kQOff;
  uint8_t* sK = smem + L::kKOff;
  uint8_t* sV = smem + L::kVOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;            // rank 0 only
  uint64_t* k_full = bars + 1;        // rank 0 only
  uint64_t* k_empty = k_full + KST;   // both
  uint64_t* v_full = k_empty + KST;   // rank 0 only
  uint64_t* v_empty = v_full + VST;   // both
  uint64_t* s_full = v_empty + VST;   // [2] both
  uint64_t* p_full = s_full + 2;      // [2] rank 0 only, 256 arrivals
  uint64_t* o_full = p_full + 2;      // [2] both
  uint64_t* ph_full = o_full + 2;     // [2] rank 0 only, 256 arrivals: P of the block's first 64 keys is in TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortCtl ctl{p.status, abort_flag};
  const uint32_t rank = cluster_ctarank();

  // Heaviest (latest) query rows first.
  const int npairs = gridDim.x >> 1;
  int tile_i, head;
  launch_order(blockIdx.x >> 1, npairs, p.causal != 0, tile_i, head);  // both CTAs of a pair map to the same (pair, head)
  const int qpair = npairs - 1 - tile_i;
  const int batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int m_base = qpair * (4 * kBM);

  // Trip counts are a property of the PAIR's tile t (rows [m_base + 2t*128, +256)): both CTAs compute the same.
  int nblk[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int lo = m_base + 2 * t * kBM;
    int kv_end = p.Sk;
    if (p.causal) {
      const int hi = min(lo + 2 * kBM - 1, p.Sq - 1);
      kv_end = min(p.Sk, hi + p.causal_off + 1);
    }
    nblk[t] = (lo < p.Sq && kv_end > 0) ? (kv_end + BN - 1) / BN : 0;
  }
  int nmax = max(nblk[0], nblk[1]);

  if (threadIdx.x == 0) {
    // a launch that finds an error already recorded (by an earlier CTA or launch) does no work
    *abort_flag = (p.status != nullptr && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) ? 1u : 0u;
    mbar_init(q_full, 1);
    for (int i = 0; i < KST; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < VST; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_full[t], 256); mbar_init(&o_full[t], 1); mbar_init(&ph_full[t], 256); }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (*abort_flag != 0u) nblk[0] = nblk[1] = nmax = 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    setmaxnreg_dec<kFwdRegsLo>();
    if (lane == 0 && nmax > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      const uint32_t q_full0 = mapa_u32(smem_u32(q_full), 0);
      if (rank == 0) mbar_arrive_expect_tx(q_full, 2 * 2 * L::kQTile);  // both CTAs' tiles
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int sub = 0; sub < DQK / 64; ++sub)
          tma_load_4d_pair(sQ + t * L::kQTile + sub * (kBM * 128), &tm_q, q_full0, sub * 64, head,
                           m_base + (2 * t + static_cast<int>(rank)) * kBM, batch);
      for (int j = 0; j < nmax; ++j) {
        const int ks = j % KST, vs = j % VST;
        mbar_wait(&k_empty[ks], ((j / KST) & 1) ^ 1, ctl, 0x100 + ks);
        if (rank == 0) mbar_arrive_expect_tx(&k_full[ks], 2 * L::kKHalf);
        const uint32_t kf0 = mapa_u32(smem_u32(&k_full[ks]), 0);
#pragma unroll
        for (int sub = 0; sub < DQK / 64; ++sub)
          tma_load_4d_pair(sK + ks * L::kKHalf + sub * ((BN / 2) * 128), &tm_k, kf0, sub * 64, kv_head,
                           j * BN + static_cast<int>(rank) * (BN / 2), batch);
        mbar_wait(&v_empty[vs], ((j / VST) & 1) ^ 1, ctl, 0x200 + vs);
        if (rank == 0) mbar_arrive_expect_tx(&v_full[vs], 2 * L::kVHalf);
        const uint32_t vf0 = mapa_u32(smem_u32(&v_full[vs]), 0);
        tma_load_4d_pair(sV + vs * L::kVHalf, &tm_v, vf0, static_cast<int>(rank) * (kDV / 2), kv_head, j * BN, batch);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (rank 0 only)
    setmaxnreg_dec<kFwdRegsLo>();
    const bool leader = elect_one();  // the whole warp walks the loop; one lane issues
    if (rank == 0 && nmax > 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(2 * kBM, BN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(2 * kBM, kDV, false, true);
      uint64_t qd[2], kd[KST], vd[VST];
#pragma unroll
      for (int t = 0; t < 2; ++t) qd[t] = make_smem_desc(smem_u32(sQ) + t * L::kQTile, 16, 1024);
#pragma unroll
      for (int i = 0; i < KST; ++i) kd[i] = make_smem_desc(smem_u32(sK) + i * L::kKHalf, 16, 1024);
#pragma unroll
      for (int i = 0; i < VST; ++i) vd[i] = make_smem_desc(smem_u32(sV) + i * L::kVHalf, BN * 128, 1024);
      mbar_wait(q_full, 0, ctl, 0x300);
      mbar_wait(&k_full[0], 0, ctl, 0x400);
      tc_fence_after_sync();
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (nblk[t] > 0) {
          issue_qk_pair<DQK>(tmem_base + t * 128, qd[t], kd[0], idesc_qk, leader);
          if (leader) umma_commit_pair(&s_full[t]);
        }
      }
      if (leader) umma_commit_pair(&k_empty[0]);
      for (int j = 0; j < nmax; ++j) {
        const int vs = j % VST;
        const bool have_next = j + 1 < nmax;
        const int ks = (j + 1) % KST;
        mbar_wait(&v_full[vs], (j / VST) & 1, ctl, 0x500 + vs);
        if (have_next) mbar_wait(&k_full[ks], ((j + 1) / KST) & 1, ctl, 0x400 + ks);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j < nblk[t]) {
            mbar_wait(&ph_full[t], j & 1, ctl, 0x680 + t);
            tc_fence_after_sync();
            issue_pv_pair<0, 4>(tmem_base + 256 + t * 128, tmem_base + t * 128, vd[vs], idesc_pv, j > 0, leader);
            mbar_wait(&p_full[t], j & 1, ctl, 0x600 + t);
            tc_fence_after_sync();
            issue_pv_pair<4, 8>(tmem_base + 256 + t * 128, tmem_base + t * 128, vd[vs], idesc_pv, true, leader);
            if (j + 1 < nblk[t]) {
              issue_qk_pair<DQK>(tmem_base + t * 128, qd[t], kd[ks], idesc_qk, leader);
              if (leader) umma_commit_pair(&s_full[t]);
            } else {
              if (leader) umma_commit_pair(&o_full[t]);
            }
          }
        }
        if (leader) umma_commit_pair(&v_empty[vs]);
        if (have_next) if (leader) umma_commit_pair(&k_empty[ks]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax + epilogue (both CTAs)
    setmaxnreg_inc<kFwdRegsHi>();
    const int t = (warp - 4) >> 2;                      // query tile of this warpgroup
    const int row_in_tile = ((warp & 3) << 5) + lane;   // TMEM lane == query row
    const int tile_row0 = m_base + (2 * t + static_cast<int>(rank)) * kBM;
    const int row = tile_row0 + row_in_tile;            // query position inside this call's Q block
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const uint32_t tS = tmem_base + lane_addr + t * 128;
    const uint32_t tO = tmem_base + lane_addr + 256 + t * 128;
    const uint32_t pf0 = mapa_u32(smem_u32(&p_full[t]), 0);
    const uint32_t ph0 = mapa_u32(smem_u32(&ph_full[t]), 0);
    fwd_softmax_rows<BN>(p, ctl, &s_full[t], &o_full[t], [pf0] { mbar_arrive_cluster(pf0); },
                         [ph0] { mbar_arrive_cluster(ph0); }, tS, tO, tile_row0, row, nblk[t], head, batch, t);
  } else {
    setmaxnreg_dec<kFwdRegsLo>();  // warps 2 and 3 only give their registers away
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA's shared memory / TMEM goes away while the pair's MMAs may still touch it
  if (*abort_flag != 0u) {
    // Something gave up waiting: let copies and MMAs still in flight drain before the
    // shared memory and TMEM of this CTA are handed back.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int DQK, int KST, int VST>
static int launch_pair(const pith_attn_fwd_args* a, const FwdParams& p, cudaStream_t st) {
  using L = FwdPairSmem<DQK, KST, VST>;
  static_assert(L::kAlloc <= 232448, "shared memory budget");
  CUtensorMap tq, tk, tv;
  if (int rc = make_tensor_map(&tq, a->q, 2, a->B, a->Sq, a->Hq, a->Dqk, a->q_stride, 64, kBM)) return rc;
  if (int rc = make_tensor_map(&tk, a->k, 2, a->B, a->Sk, a->Hkv, a->Dqk, a->k_stride, 64, kPairBN / 2)) return rc;
  if (int rc = make_tensor_map(&tv, a->v, 2, a->B, a->Sk, a->Hkv, a->Dv, a->v_stride, 64, kPairBN)) return rc;
  auto kern = attn_fwd_pair_kernel<DQK, KST, VST>;
  // per call: the attribute belongs to the current device, and a process may use several
  PITH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
  const int npairs = (a->Sq + 4 * kBM - 1) / (4 * kBM);
  dim3 grid(2 * npairs, a->Hq, a->B);  // cluster dimension (2, 1, 1) is a compile-time attribute of the kernel
  kern<<<grid, kFwdThreads, L::kAlloc, st>>>(tq, tk, tv, p);
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

int launch_fwd_pair(const pith_attn_fwd_args* a, const FwdParams& p, cudaStream_t st) {
  if (a->Dqk == 128) return launch_pair<128, 2, 2>(a, p, st);
  return launch_pair<192, 2, 2>(a, p, st);
}

}  // namespace pith
