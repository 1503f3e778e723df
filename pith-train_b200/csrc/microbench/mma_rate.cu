// Micro-benchmark behind the kernels' design notes: how many cycles a tcgen05.mma takes when one lane issues
// the attention kernels' MMA sequences back to back, alone and next to the other traffic those kernels generate.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I.. -I../../../include \
//        -o mma_rate mma_rate.cu ../host_common.cu && ./mma_rate
//
// Part 1: M = 128 (256 over a CTA pair), K = 16, N = 64 / 128 / 256, operands from shared memory (SS) or A from
//         TMEM (TS), one or two accumulators.
// Part 2: the forward kernel's sequence per iteration (PV0 QK0 PV1 QK1 = 32 MMAs, ideal 2048 cycles) with, beside
//         it: TMA loads into other buffers, warps spinning on an mbarrier, tcgen05.ld/st, MUFU and shared-memory
//         stores; then with a commit after every group, with a satisfied mbarrier wait + fence before every group, and
//         with a full drain (commit + wait) once per iteration.
// Every wait is bounded; nothing here can spin forever. Not part of the library: nothing links or imports it.
#include <cstdio>
#include "common.cuh"
#include "host_common.h"
using namespace pith;

struct Res { long long cyc; int n; };
constexpr int kSmem = 202 * 1024;

// ---------------------------------------------------------------------------------------------- part 1
template <int TS, int N, int NBUF, int PAIR, int BK>
__global__ void __launch_bounds__(128, 1) rate_kernel(Res* out, int reps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot, aflag;
  const int warp = threadIdx.x >> 5;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { aflag = 0; mbar_init(&bar, 1); mbar_fence_init(); }
  if (warp == 0) { if (PAIR) { tmem_alloc_pair(&slot, 512); tmem_relinquish_pair(); } else { tmem_alloc(&slot, 512); tmem_relinquish(); } }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tb = slot;
  AbortCtl ctl{nullptr, &aflag};
  if (threadIdx.x == 32 && rank == 0) {
    const uint32_t idesc = make_idesc_bf16(PAIR ? 256 : 128, N, false, BK ? false : true);
    const uint64_t ad = make_smem_desc(smem_u32(smem), 16, 1024);
    const uint64_t bdk = make_smem_desc(smem_u32(smem) + 65536, 16, 1024);
    const uint64_t bdm = make_smem_desc(smem_u32(smem) + 65536, 128 * 128, 1024);
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
      const uint32_t d = tb + (NBUF == 1 ? 0 : (r % NBUF) * N);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t aoff = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
        const uint32_t boff = BK ? (kk >> 2) * ((PAIR ? N / 2 : N) * 128) + (kk & 3) * 32 : kk * 2048;
        const uint64_t bd = desc_advance(BK ? bdk : bdm, boff);
        if (TS) { if (PAIR) umma_ts_pair(d, tb + 384 + kk * 8, bd, idesc, kk > 0); else umma_ts(d, tb + 384 + kk * 8, bd, idesc, kk > 0); }
        else    { if (PAIR) umma_ss_pair(d, desc_advance(ad, aoff), bd, idesc, kk > 0); else umma_ss(d, desc_advance(ad, aoff), bd, idesc, kk > 0); }
      }
    }
    if (PAIR) umma_commit_pair(&bar); else umma_commit(&bar);
    mbar_wait(&bar, 0, ctl, 1);
    const long long t1 = clock64();
    if (blockIdx.x == 0) { out[0].cyc = t1 - t0; out[0].n = reps * 8; }
  } else if (PAIR && threadIdx.x == 32) {
    mbar_wait(&bar, 0, ctl, 2);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  if (warp == 0) { tc_fence_after_sync(); if (PAIR) tmem_dealloc_pair(tb, 512); else tmem_dealloc(tb, 512); }
}

template <int TS, int N, int NBUF, int PAIR, int BK>
void rate(const char* name) {
  Res* d; cudaMalloc(&d, sizeof(Res));
  auto kern = rate_kernel<TS, N, NBUF, PAIR, BK>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (PAIR) {
    cudaLaunchConfig_t cfg = {}; cfg.gridDim = dim3(148); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = kSmem;
    cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kern, d, 512);
  } else {
    kern<<<148, 128, kSmem>>>(d, 512);
  }
  const cudaError_t e = cudaDeviceSynchronize();
  Res h; cudaMemcpy(&h, d, sizeof h, cudaMemcpyDeviceToHost);
  printf("  %-46s %6.1f cycles per MMA %s\n", name, double(h.cyc) / h.n, e == cudaSuccess ? "" : cudaGetErrorString(e));
  cudaFree(d);
}

// ---------------------------------------------------------------------------------------------- part 2
// LOAD bits: 1 = warps 4..7 loop tcgen05.ld/st on spare columns, 2 = warps 4..11 loop MUFU ex2, 4 = warps 4..11 store
// to shared memory, 8 = warps 4..11 spin on an mbarrier that never completes, 16 = thread 0 streams 32 KB TMA tiles
// into a two-deep ring as fast as it allows.
// SYNC: 0 none, 1 commit after every group, 2 satisfied mbarrier wait + fence before every group (+ commits),
//       3 commit + wait once per iteration.
template <int LOAD, int SYNC>
__global__ void __launch_bounds__(384, 1) pattern_kernel(const __grid_constant__ CUtensorMap tm, Res* out, int reps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar, full[2], grp[2], never, done_bar, open_bar;
  __shared__ uint32_t slot, aflag;
  __shared__ volatile uint32_t done;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 200 * 1024 / 4; i += 384) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) {
    aflag = 0; done = 0;
    mbar_init(&bar, 1); mbar_init(&never, 1); mbar_init(&done_bar, 1); mbar_init(&open_bar, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&full[i], 1); mbar_init(&grp[i], 1); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tb = slot;
  AbortCtl ctl{nullptr, &aflag};
  // shared memory: Q0 at 0, Q1 at 32 K, K at 64 K, V at 96 K (never overwritten); TMA ring at 128 K (2 x 32 KB)
  if (threadIdx.x == 32) {
    const uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false), idesc_pv = make_idesc_bf16(128, 128, false, true);
    const uint64_t qd0 = make_smem_desc(smem_u32(smem), 16, 1024), qd1 = make_smem_desc(smem_u32(smem) + 32768, 16, 1024);
    const uint64_t kd = make_smem_desc(smem_u32(smem) + 65536, 16, 1024);
    const uint64_t vd = make_smem_desc(smem_u32(smem) + 98304, 128 * 128, 1024);
    auto qk = [&](uint32_t d, uint64_t qd) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
        umma_ss(d, desc_advance(qd, off), desc_advance(kd, off), idesc_qk, kk > 0);
      }
    };
    auto pv = [&](uint32_t d, uint32_t pcol) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) umma_ts(d, pcol + kk * 8, desc_advance(vd, kk * 2048), idesc_pv, 1);
    };
    auto before = [&]() { if (SYNC == 2) { mbar_wait(&open_bar, 1, ctl, 7); tc_fence_after_sync(); } };  // parity 1 of a fresh barrier: satisfied
    uint32_t ph = 0;
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
      before(); pv(tb + 256, tb);            // P_0 overlays S_0, as in the kernel
      before(); qk(tb, qd0);
      if (SYNC == 1 || SYNC == 2) umma_commit(&grp[0]);
      before(); pv((LOAD & 1) ? tb + 256 : tb + 384, tb + 128);  // with LOAD bit 1, columns 384..511 belong to the ld/st warps
      before(); qk(tb + 128, qd1);
      if (SYNC == 1 || SYNC == 2) umma_commit(&grp[1]);
      if (SYNC == 3) { umma_commit(&done_bar); mbar_wait(&done_bar, ph, ctl, 8); ph ^= 1; tc_fence_after_sync(); }
    }
    umma_commit(&bar);
    mbar_wait(&bar, 0, ctl, 1);
    const long long t1 = clock64();
    done = 1;
    if (blockIdx.x == 0) { out[0].cyc = t1 - t0; out[0].n = reps; }
  } else if (threadIdx.x == 0 && (LOAD & 16)) {
    int it = 0;
    const long long tstart = clock64();
    while (done == 0 && clock64() - tstart < 400000000ll) {
      const int s = it & 1;
      if (it >= 2) mbar_wait(&full[s], ((it - 2) >> 1) & 1, ctl, 3);  // the previous load into this stage has landed
      mbar_arrive_expect_tx(&full[s], 32768);
      tma_load_4d(smem + 131072 + s * 32768, &tm, &full[s], 0, 0, (it * 128) & 8191, 0);
      tma_load_4d(smem + 131072 + s * 32768 + 16384, &tm, &full[s], 64, 0, (it * 128) & 8191, 0);
      ++it;
    }
    for (int b = 0; b < 2 && it >= 2; ++b) { const int i2 = it - 1 - b; mbar_wait(&full[i2 & 1], (i2 >> 1) & 1, ctl, 4); }
    if (blockIdx.x == 0) out[1].n = it;
  } else if (warp >= 4 && (LOAD & 15)) {
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    float acc = threadIdx.x * 1e-3f;
    const long long tstart = clock64();
    while (done == 0 && clock64() - tstart < 400000000ll) {
      if ((LOAD & 1) && warp < 8) {  // columns 448..511: no MMA touches them in this mode
        uint32_t r[64];
        tmem_ld32(tb + lane_addr + 448, r);
        tmem_ld32(tb + lane_addr + 480, r + 32);
        tmem_wait_ld();
        uint32_t w[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) w[i] = r[2 * i] ^ r[2 * i + 1];
        tmem_st32(tb + lane_addr + 448, w);
        tmem_wait_st();
      }
      if (LOAD & 2) {
#pragma unroll
        for (int i = 0; i < 64; ++i) acc = fast_exp2(acc) * 0.5f;
      }
      if (LOAD & 4) {
        uint4* dst = reinterpret_cast<uint4*>(smem + 196608) + (threadIdx.x - 128);
#pragma unroll
        for (int i = 0; i < 2; ++i) dst[i * 256] = make_uint4(1, 2, 3, 4);
      }
      if (LOAD & 8) (void)mbar_try_wait(&never, 0);
    }
    if (acc == 123.f) out[1].n = -1;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tb, 512); }
}

template <int LOAD, int SYNC>
void pattern(const char* name, const CUtensorMap& tm) {
  Res* d; cudaMalloc(&d, 2 * sizeof(Res)); cudaMemset(d, 0, 2 * sizeof(Res));
  auto kern = pattern_kernel<LOAD, SYNC>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  kern<<<148, 384, kSmem>>>(tm, d, 512);
  const cudaError_t e = cudaDeviceSynchronize();
  Res h[2]; cudaMemcpy(h, d, sizeof h, cudaMemcpyDeviceToHost);
  printf("  %-66s %7.1f cycles per iteration %s\n", name, double(h[0].cyc) / h[0].n, e == cudaSuccess ? "" : cudaGetErrorString(e));
  cudaFree(d);
}

int main() {
  printf("part 1: cycles per MMA, 148 CTAs, 4096 MMAs each\n");
  rate<0, 128, 1, 0, 1>("SS  M=128 N=128  B K-major");
  rate<0, 128, 2, 0, 1>("SS  M=128 N=128  two accumulators");
  rate<0, 128, 1, 0, 0>("SS  M=128 N=128  B MN-major");
  rate<0, 64, 1, 0, 1>("SS  M=128 N=64");
  rate<0, 256, 1, 0, 1>("SS  M=128 N=256");
  rate<1, 128, 1, 0, 0>("TS  M=128 N=128  B MN-major");
  rate<1, 64, 1, 0, 0>("TS  M=128 N=64");
  rate<0, 128, 1, 1, 1>("SS  pair M=256 N=128 (64 per CTA)");
  rate<1, 128, 1, 1, 0>("TS  pair M=256 N=128 (64 per CTA)");
  void* g; cudaMalloc(&g, 8192ull * 4 * 128 * 2); cudaMemset(g, 0x3c, 8192ull * 4 * 128 * 2);
  CUtensorMap tm; int64_t st[3] = {8192ll * 4 * 128, 4 * 128, 128};
  if (make_tensor_map(&tm, g, 2, 1, 8192, 4, 128, st, 64, 128)) { printf("tensor map failed: %s\n", last_error_buffer()); return 1; }
  printf("part 2: forward sequence PV0 QK0 PV1 QK1, ideal 2048 cycles per iteration\n");
  pattern<0, 0>("alone", tm);
  pattern<1, 0>("+ tcgen05.ld/st in 4 warps", tm);
  pattern<2, 0>("+ MUFU in 8 warps", tm);
  pattern<4, 0>("+ shared-memory stores in 8 warps", tm);
  pattern<8, 0>("+ 8 warps spinning on mbarrier.try_wait", tm);
  pattern<16, 0>("+ TMA loads as fast as a two-deep ring allows", tm);
  pattern<31, 0>("+ all of the above", tm);
  pattern<0, 1>("commit after every group", tm);
  pattern<0, 2>("satisfied mbarrier wait + fence before every group, commits", tm);
  pattern<0, 3>("commit + wait (full drain) once per iteration", tm);
  return 0;
}
