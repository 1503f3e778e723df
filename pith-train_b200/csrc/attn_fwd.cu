// Attention forward for sm_100a: S = Q K^T and O += P V run on tcgen05 with fp32 accumulators
// in TMEM; Q/K/V tiles arrive through TMA into 128-byte-swizzled shared memory.
//
// One CTA owns two 128-row query tiles of one (batch, query head) and walks the key/value
// blocks they need. Warp roles (384 threads):
//   warp 0        TMA producer: Q once, then K and V blocks through KST / VST-deep rings
//   warp 1        tcgen05 issuer (the warp walks the loop converged, one elected lane issues):
//                 S_t = Q_t K_j^T, O_t += P_t V_j; the PV GEMM starts on the first 64 keys' P while the second
//                 64 are still being exponentiated
//   warps 4..7    softmax group of tile 0, one thread per query row (= TMEM lane)
//   warps 8..11   softmax group of tile 1
// The two softmax groups alternate with the tensor core: while group 0 turns S_0 into P_0
// the tensor core works on tile 1 and vice versa.
//
// TMEM columns (512, fp32): [0,128) S_0 (P_0 packed bf16 overlays [0,64)), [128,256) S_1 / P_1,
// [256,384) O_0, [384,512) O_1.
//
// Softmax runs in the exp2 domain; the running maximum is only moved when it grows by more than
// 2^8 (warp-uniform decision), which keeps the O rescale off the common path. The epilogue
// normalises, optionally merges a previous partial (O, LSE) (the ring's online-softmax combine)
// and writes bf16 or fp32 O plus the log2-domain LSE. Causal launches take their (tile, head) from launch_order()
// (heads in groups of eight, heaviest tiles first).
#include "attn_fwd_common.cuh"

namespace pith {

template <int DQK, int BN, int KST, int VST>
struct FwdSmem {
  static constexpr int kQTile = kBM * DQK * 2;  // bytes of one Q tile
  static constexpr int kKTile = BN * DQK * 2;
  static constexpr int kVTile = BN * kDV * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + 2 * kQTile;
  static constexpr int kVOff = kKOff + KST * kKTile;
  static constexpr int kBarOff = kVOff + VST * kVTile;
  static constexpr int kNumBars = 1 + 2 * KST + 2 * VST + 8;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16;
  static constexpr int kAlloc = kTotal;  // no slack: the kernel checks that the dynamic window starts 1024-aligned
};

// S[128 x BN] = Q_tile[128 x DQK] * K_blk[BN x DQK]^T, both operands K-major in shared memory.
// qdesc / kdesc describe the first [rows][64] sub-tile; later K-steps only move the start address.
template <int DQK, int BN>
__device__ __forceinline__ void issue_qk(uint32_t d_tmem, uint64_t qdesc, uint64_t kdesc, uint32_t idesc, bool leader) {
#pragma unroll
  for (int kk = 0; kk < DQK / 16; ++kk) {
    const uint32_t sub = kk >> 2, off = (kk & 3) * 32;
    if (leader)
      umma_ss(d_tmem, desc_advance(qdesc, sub * (kBM * 128) + off), desc_advance(kdesc, sub * (BN * 128) + off), idesc,
              kk > 0 ? 1u : 0u);
  }
}

// O[128 x 128] (+)= P[128 x BN] (bf16 in TMEM) * V_blk[BN x 128] (MN-major in shared memory:
// two [BN][64] column blocks, BN * 128 bytes apart).
// K-steps [K0, K1) of the block's BN / 16: the first half can run as soon as the first 64 keys' P has been stored.
template <int K0, int K1>
__device__ __forceinline__ void issue_pv(uint32_t d_tmem, uint32_t p_tmem, uint64_t vdesc, uint32_t idesc, bool acc,
                                         bool leader) {
#pragma unroll
  for (int kk = K0; kk < K1; ++kk)
    if (leader) umma_ts(d_tmem, p_tmem + kk * 8, desc_advance(vdesc, kk * 2048), idesc, (acc || kk > 0) ? 1u : 0u);
}

template <int DQK, int BN, int KST, int VST>
__global__ void __launch_bounds__(kFwdThreads, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using L = FwdSmem<DQK, BN, KST, VST>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem + L::kQOff;
  uint8_t* sK = smem + L::kKOff;
  uint8_t* sV = smem + L::kVOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + KST;
  uint64_t* v_full = k_empty + KST;
  uint64_t* v_empty = v_full + VST;
  uint64_t* s_full = v_empty + VST;  // [2]
  uint64_t* p_full = s_full + 2;     // [2]
  uint64_t* o_full = p_full + 2;     // [2]
  uint64_t* ph_full = o_full + 2;    // [2] P of the block's first 64 keys is in TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AbortCtl ctl{p.status, abort_flag};

  // Heaviest (latest) query tiles first.
  int tile_i, head;
  launch_order(blockIdx.x, gridDim.x, p.causal != 0, tile_i, head);
  const int qblk = gridDim.x - 1 - tile_i;
  const int batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int m0 = qblk * (2 * kBM);

  int nblk[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int lo = m0 + t * kBM;
    int kv_end = p.Sk;
    if (p.causal) {
      const int hi = min(lo + kBM - 1, p.Sq - 1);
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
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_full[t], 128); mbar_init(&o_full[t], 1); mbar_init(&ph_full[t], 128); }
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
    if (threadIdx.x == 0) report_error(ctl, 0xA1u, smem_u32(smem));
    nblk[0] = nblk[1] = nmax = 0;
  }
  if (*abort_flag != 0u) nblk[0] = nblk[1] = nmax = 0;

  // Register budget: the four warps of warpgroup 0 (producer, MMA issuer, two idle) need few registers,
  // the softmax groups hold a whole 128-column score row each.
  // (each role branch below starts with its own setmaxnreg so that the limit holds for exactly that code)
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    setmaxnreg_dec<kFwdRegsLo>();
    if (lane == 0 && nmax > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_arrive_expect_tx(q_full, 2 * L::kQTile);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int sub = 0; sub < DQK / 64; ++sub)
          tma_load_4d(sQ + t * L::kQTile + sub * (kBM * 128), &tm_q, q_full, sub * 64, head, m0 + t * kBM, batch);
      for (int j = 0; j < nmax; ++j) {
        const int ks = j % KST, vs = j % VST;
        mbar_wait(&k_empty[ks], ((j / KST) & 1) ^ 1, ctl, 0x100 + ks);
        mbar_arrive_expect_tx(&k_full[ks], L::kKTile);
#pragma unroll
        for (int sub = 0; sub < DQK / 64; ++sub)
          tma_load_4d(sK + ks * L::kKTile + sub * (BN * 128), &tm_k, &k_full[ks], sub * 64, kv_head, j * BN, batch);
        mbar_wait(&v_empty[vs], ((j / VST) & 1) ^ 1, ctl, 0x200 + vs);
        mbar_arrive_expect_tx(&v_full[vs], L::kVTile);
#pragma unroll
        for (int sub = 0; sub < kDV / 64; ++sub)
          tma_load_4d(sV + vs * L::kVTile + sub * (BN * 128), &tm_v, &v_full[vs], sub * 64, kv_head, j * BN, batch);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    setmaxnreg_dec<kFwdRegsLo>();
    const bool leader = elect_one();  // the whole warp walks the loop; one lane issues
    if (nmax > 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(kBM, BN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(kBM, kDV, false, true);
      uint64_t qd[2], kd[KST], vd[VST];
#pragma unroll
      for (int t = 0; t < 2; ++t) qd[t] = make_smem_desc(smem_u32(sQ) + t * L::kQTile, 16, 1024);
#pragma unroll
      for (int i = 0; i < KST; ++i) kd[i] = make_smem_desc(smem_u32(sK) + i * L::kKTile, 16, 1024);
#pragma unroll
      for (int i = 0; i < VST; ++i) vd[i] = make_smem_desc(smem_u32(sV) + i * L::kVTile, BN * 128, 1024);
      mbar_wait(q_full, 0, ctl, 0x300);
      mbar_wait(&k_full[0], 0, ctl, 0x400);
      tc_fence_after_sync();
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (nblk[t] > 0) {
          issue_qk<DQK, BN>(tmem_base + t * 128, qd[t], kd[0], idesc_qk, leader);
          if (leader) umma_commit(&s_full[t]);
        }
      }
      if (leader) umma_commit(&k_empty[0]);
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
            issue_pv<0, BN / 32>(tmem_base + 256 + t * 128, tmem_base + t * 128, vd[vs], idesc_pv, j > 0, leader);
            mbar_wait(&p_full[t], j & 1, ctl, 0x600 + t);
            tc_fence_after_sync();
            issue_pv<BN / 32, BN / 16>(tmem_base + 256 + t * 128, tmem_base + t * 128, vd[vs], idesc_pv, true, leader);
            if (j + 1 < nblk[t]) {
              issue_qk<DQK, BN>(tmem_base + t * 128, qd[t], kd[ks], idesc_qk, leader);
              if (leader) umma_commit(&s_full[t]);
            } else {
              if (leader) umma_commit(&o_full[t]);
            }
          }
        }
        if (leader) umma_commit(&v_empty[vs]);
        if (have_next) if (leader) umma_commit(&k_empty[ks]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax + epilogue
    setmaxnreg_inc<kFwdRegsHi>();
    const int t = (warp - 4) >> 2;                 // query tile of this warpgroup
    const int row_in_tile = ((warp & 3) << 5) + lane;  // TMEM lane == query row
    const int row = m0 + t * kBM + row_in_tile;    // query position inside this call's Q block
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const uint32_t tS = tmem_base + lane_addr + t * 128;
    const uint32_t tO = tmem_base + lane_addr + 256 + t * 128;
    uint64_t* pf = &p_full[t];
    uint64_t* ph = &ph_full[t];
    fwd_softmax_rows<BN>(p, ctl, &s_full[t], &o_full[t], [pf] { mbar_arrive(pf); }, [ph] { mbar_arrive(ph); }, tS, tO,
                         m0 + t * kBM, row, nblk[t], head, batch, t);
  } else {
    setmaxnreg_dec<kFwdRegsLo>();  // warps 2 and 3 only give their registers away
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
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int DQK, int BN, int KST, int VST>
static int launch_fwd(const pith_attn_fwd_args* a, const FwdParams& p, cudaStream_t st) {
  using L = FwdSmem<DQK, BN, KST, VST>;
  CUtensorMap tq, tk, tv;
  if (int rc = make_tensor_map(&tq, a->q, 2, a->B, a->Sq, a->Hq, a->Dqk, a->q_stride, 64, kBM)) return rc;
  if (int rc = make_tensor_map(&tk, a->k, 2, a->B, a->Sk, a->Hkv, a->Dqk, a->k_stride, 64, BN)) return rc;
  if (int rc = make_tensor_map(&tv, a->v, 2, a->B, a->Sk, a->Hkv, a->Dv, a->v_stride, 64, BN)) return rc;
  auto kern = attn_fwd_kernel<DQK, BN, KST, VST>;
  // per call: the attribute belongs to the current device, and a process may use several
  PITH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc));
  dim3 grid((a->Sq + 2 * kBM - 1) / (2 * kBM), a->Hq, a->B);
  kern<<<grid, kFwdThreads, L::kAlloc, st>>>(tq, tk, tv, p);
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace pith

using namespace pith;

extern "C" int pith_attn_fwd(const pith_attn_fwd_args* a, void* stream) {
  PITH_REQUIRE(a != nullptr, "null args");
  PITH_REQUIRE(a->q && a->k && a->v && a->o && a->lse, "null tensor pointer");
  PITH_REQUIRE(a->B > 0 && a->Sq > 0 && a->Sk > 0 && a->Hq > 0 && a->Hkv > 0, "bad shape B=%d Sq=%d Sk=%d Hq=%d Hkv=%d",
               a->B, a->Sq, a->Sk, a->Hq, a->Hkv);
  PITH_REQUIRE(a->Hq % a->Hkv == 0, "Hq=%d is not a multiple of Hkv=%d", a->Hq, a->Hkv);
  PITH_REQUIRE(a->Dv == 128 && (a->Dqk == 128 || a->Dqk == 192),
               "unsupported head dims Dqk=%d Dv=%d (supported: 128/128 and 192/128)", a->Dqk, a->Dv);
  PITH_REQUIRE((a->prev_o == nullptr) == (a->prev_lse == nullptr), "prev_o and prev_lse must be given together");
  PITH_REQUIRE(a->softmax_scale > 0.f, "softmax_scale must be positive");
  PITH_REQUIRE(a->Hq <= 65535 && a->B <= 65535, "Hq and B must fit a grid dimension");
  const bool o32 = (a->flags & PITH_FWD_O_FP32) != 0;
  const int oeb = o32 ? 4 : 2;
  PITH_REQUIRE(aligned16(a->o) && (a->o_stride[0] * oeb) % 16 == 0 && (a->o_stride[1] * oeb) % 16 == 0 &&
                   (a->o_stride[2] * oeb) % 16 == 0,
               "o must be 16-byte aligned with 16-byte-multiple strides");
  if (a->prev_o)
    PITH_REQUIRE(aligned16(a->prev_o) && a->prev_o_stride[0] % 4 == 0 && a->prev_o_stride[1] % 4 == 0 &&
                     a->prev_o_stride[2] % 4 == 0,
                 "prev_o must be 16-byte aligned with 16-byte-multiple strides");
  if (int rc = require_sm100()) return rc;
  FwdParams p;
  p.o = a->o; p.lse = a->lse; p.prev_o = a->prev_o; p.prev_lse = a->prev_lse; p.status = a->status;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal ? 1 : 0; p.causal_off = a->causal_offset;
  p.o_fp32 = o32 ? 1 : 0; p.lse_natural = (a->flags & PITH_FWD_LSE_NATURAL) ? 1 : 0;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  for (int i = 0; i < 3; ++i) { p.os[i] = a->o_stride[i]; p.pos[i] = a->prev_o ? a->prev_o_stride[i] : 0; }
  for (int i = 0; i < 2; ++i) { p.ls[i] = a->lse_stride[i]; p.pls[i] = a->prev_lse ? a->prev_lse_stride[i] : 0; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PITH_REQUIRE(!((a->flags & PITH_FWD_SINGLE_CTA) && (a->flags & PITH_FWD_CTA_PAIR)),
               "PITH_FWD_SINGLE_CTA and PITH_FWD_CTA_PAIR exclude each other");
  const bool pair = (a->flags & PITH_FWD_CTA_PAIR) || (!(a->flags & PITH_FWD_SINGLE_CTA) && a->Dqk == 192);
  if (pair) return launch_fwd_pair(a, p, st);
  if (a->Dqk == 128) return launch_fwd<128, 128, 2, 2>(a, p, st);
  return launch_fwd<192, 128, 2, 1>(a, p, st);
}
