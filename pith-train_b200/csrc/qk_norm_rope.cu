// The step in front of the attention operator, fused: per-head RMSNorm of Q and K followed by rotary position
// embedding (rotate-half form), forward and backward, one HBM pass each.
//
//   y = x * rsqrt(mean(x^2) + eps) * w          (per [b][s][h] row of head_dim = 128)
//   z[i]      = y[i]      * cos[i]      - y[i + 64] * sin[i]           i < 64
//   z[i + 64] = y[i + 64] * cos[i + 64] + y[i]      * sin[i + 64]
//
// Sixteen lanes own one row; lane j holds elements [4j, 4j+4) and [64+4j, 64+4j+4), i.e. both members of four
// rotate-half pairs (8-byte accesses, 128 contiguous bytes per half row), so only the two row reductions need
// shuffles (four each). Q rows and K rows go through the same launch. cos/sin are
// shared by all heads of a position, so they come from L1/L2 after the first head. All arithmetic is fp32 with a
// single rounding to bf16 at the end. The backward recomputes the row statistics from x instead of saving them.
#include "../../include/pith_b200.h"
#include "common.cuh"
#include "host_common.h"

namespace pith {

struct QkParams {
  const __nv_bfloat16* x[2];   // q, k
  const __nv_bfloat16* dz[2];  // backward: gradient of the outputs
  __nv_bfloat16* out[2];       // forward: z; backward: dx
  const void* w[2];
  float* dw[2];                // backward: fp32 [128], accumulated into
  const void* cos;
  const void* sin;
  int B, S, Hq, Hkv;
  float eps;
  int64_t xs[2][3], dzs[2][3], os[2][3];  // b, s, h strides (elements)
  int64_t cs[2];                          // b, s strides of cos / sin (elements)
};

// Elements [off, off + 4) and [off + 64, off + 68) of a row: a lane's two halves of the rotate-half pairs.
__device__ __forceinline__ uint4 load_pair_raw(const __nv_bfloat16* p) {
  const uint2 lo = __ldg(reinterpret_cast<const uint2*>(p));
  const uint2 hi = __ldg(reinterpret_cast<const uint2*>(p + 64));
  return make_uint4(lo.x, lo.y, hi.x, hi.y);
}

__device__ __forceinline__ void unpack_pair(const uint4 u, float (&v)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

__device__ __forceinline__ void load_pair_bf16(const __nv_bfloat16* p, float (&v)[8]) { unpack_pair(load_pair_raw(p), v); }

// The same as packed f32x2 pairs: V[0], V[1] = the four elements of the first half, V[2], V[3] = of the second half.
__device__ __forceinline__ void unpack_pair2(const uint4 u, uint64_t (&V)[4]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) V[i] = f2_pack(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
}

template <bool F32>
__device__ __forceinline__ void load_pair_any(const void* base, int64_t off, float (&v)[8]) {
  if constexpr (F32) {
    const float* p = static_cast<const float*>(base) + off;
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p + 64));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    load_pair_bf16(static_cast<const __nv_bfloat16*>(base) + off, v);
  }
}

__device__ __forceinline__ void store_pair_bf16(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
  *reinterpret_cast<uint2*>(p + 64) = make_uint2(pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}

__device__ __forceinline__ float sum16(float v, uint32_t mask) {  // over the 16 lanes that share a row
  v += __shfl_xor_sync(mask, v, 8);
  v += __shfl_xor_sync(mask, v, 4);
  v += __shfl_xor_sync(mask, v, 2);
  v += __shfl_xor_sync(mask, v, 1);
  return v;
}

constexpr int kHeadChunk = 8;  // heads of one position that a half-warp walks through with one cos/sin load

// v[0..4) are elements d0..d0+3 of the row, v[4..8) elements d0+64..d0+67: both members of four rotate-half pairs.
// blockIdx.y is the batch entry; blockIdx.z selects a chunk of kHeadChunk heads, first those of Q, then those of K.
// Each half-warp takes positions s = blockIdx.x * 16 + its index, + 16 * gridDim.x, ...; per position it loads
// cos/sin once and walks through the chunk's heads G rows at a time. The two half-warps of a warp shuffle under
// their own masks, so one may run out of positions before the other.
#ifndef PITH_QK_G_FWD
#define PITH_QK_G_FWD 8
#endif
#ifndef PITH_QK_G_BWD
#define PITH_QK_G_BWD 2
#endif
#ifndef PITH_QK_MINB_FWD
#define PITH_QK_MINB_FWD 3
#endif
#ifndef PITH_QK_MINB_BWD
#define PITH_QK_MINB_BWD 3
#endif

template <bool BWD, bool W_F32, bool CS_F32, int G>
__global__ void __launch_bounds__(256, BWD ? PITH_QK_MINB_BWD : PITH_QK_MINB_FWD) qk_norm_rope_kernel(const QkParams p) {
  __shared__ float dw_s[128];
  const int qchunks = (p.Hq + kHeadChunk - 1) / kHeadChunk;
  const int z = static_cast<int>(blockIdx.z) >= qchunks ? 1 : 0, b = blockIdx.y;
  const int hbeg = (static_cast<int>(blockIdx.z) - (z ? qchunks : 0)) * kHeadChunk;
  const int nh = min(kHeadChunk, (z ? p.Hkv : p.Hq) - hbeg);
  const uint32_t tid = threadIdx.x, lane16 = tid & 15u;
  const uint32_t mask = 0xFFFFu << (tid & 16u);
  const int d0 = static_cast<int>(lane16) * 4;
  const int64_t x_s = p.xs[z][1], x_h = p.xs[z][2], o_s = p.os[z][1], o_h = p.os[z][2];
  const int64_t g_s = p.dzs[z][1], g_h = p.dzs[z][2];
  const __nv_bfloat16* xb = p.x[z] + b * p.xs[z][0] + hbeg * x_h + d0;
  __nv_bfloat16* ob = p.out[z] + b * p.os[z][0] + hbeg * o_h + d0;
  const __nv_bfloat16* gb = BWD ? p.dz[z] + b * p.dzs[z][0] + hbeg * g_h + d0 : nullptr;
  const int64_t cs_b = b * p.cs[0] + d0;

  float w[8], dw[8];
  load_pair_any<W_F32>(p.w[z], d0, w);
  if constexpr (BWD) {
    if (tid < 128u) dw_s[tid] = 0.f;
    __syncthreads();
  }

  // Packed pairs (fma/mul.rn.f32x2): index 0, 1 = the lane's four elements of the first half of the row, 2, 3 = its
  // four elements of the second half; pair q of the first half rotates with pair q + 2.
  uint64_t W[4], DW[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
  for (int q = 0; q < 4; ++q) W[q] = f2_pack(w[2 * q], w[2 * q + 1]);

  for (int s = static_cast<int>(blockIdx.x * 16u + (tid >> 4)); s < p.S; s += static_cast<int>(gridDim.x) * 16) {
    uint64_t C[4], S[4], NS[2];
    {
      float c[8], sn[8];
      const int64_t co = cs_b + s * p.cs[1];
      load_pair_any<CS_F32>(p.cos, co, c);
      load_pair_any<CS_F32>(p.sin, co, sn);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        C[q] = f2_pack(c[2 * q], c[2 * q + 1]);
        S[q] = f2_pack(sn[2 * q], sn[2 * q + 1]);
      }
      NS[0] = f2_pack(-sn[0], -sn[1]);
      NS[1] = f2_pack(-sn[2], -sn[3]);
    }
    const __nv_bfloat16* xp = xb + s * x_s;
    __nv_bfloat16* op = ob + s * o_s;
    const __nv_bfloat16* gp = BWD ? gb + s * g_s : nullptr;
#pragma unroll(BWD ? 1 : 2)  // the backward holds twice the state per row: unrolled it spills
    for (int h = 0; h < nh; h += G) {
      uint4 xr[G], gr[BWD ? G : 1];  // raw bf16 words of G rows: all loads are in flight before the first use
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const int hj = min(h + j, nh - 1);  // a short last group re-reads its last head; only h + j < nh is stored
        xr[j] = load_pair_raw(xp + hj * x_h);
        if constexpr (BWD) gr[j] = load_pair_raw(gp + hj * g_h);
      }
#pragma unroll
      for (int j = 0; j < G; ++j) {
        uint64_t X[4], R4[4];
        unpack_pair2(xr[j], X);
        uint64_t acc = f2_mul(X[0], X[0]);
#pragma unroll
        for (int q = 1; q < 4; ++q) acc = f2_fma(X[q], X[q], acc);
        float s0, s1;
        f2_unpack(acc, s0, s1);
        const float r = rsqrtf(sum16(s0 + s1, mask) * (1.f / 128.f) + p.eps);
        const uint64_t R = f2_pack(r, r);
        if constexpr (!BWD) {
          uint64_t Y[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) Y[q] = f2_mul(X[q], f2_mul(R, W[q]));
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            R4[q] = f2_fma(Y[q], C[q], f2_mul(Y[q + 2], NS[q]));
            R4[q + 2] = f2_fma(Y[q + 2], C[q + 2], f2_mul(Y[q], S[q + 2]));
          }
        } else {
          // dy = dz * cos + rotate_half^T(dz * sin): the pair partner's dz * sin comes back with the opposite sign
          uint64_t Gz[4], dY[4], XH[4];
          unpack_pair2(gr[j], Gz);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            dY[q] = f2_fma(Gz[q], C[q], f2_mul(Gz[q + 2], S[q + 2]));
            dY[q + 2] = f2_fma(Gz[q + 2], C[q + 2], f2_mul(Gz[q], NS[q]));
          }
          const bool counted = h + j < nh;
          uint64_t gacc = 0ull;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            XH[q] = f2_mul(X[q], R);
            if (counted) DW[q] = f2_fma(dY[q], XH[q], DW[q]);
            dY[q] = f2_mul(dY[q], W[q]);
            gacc = f2_fma(dY[q], XH[q], gacc);
          }
          float g0, g1;
          f2_unpack(gacc, g0, g1);
          const float m = sum16(g0 + g1, mask) * (1.f / 128.f);
          const uint64_t NM = f2_pack(-m, -m);
#pragma unroll
          for (int q = 0; q < 4; ++q) R4[q] = f2_mul(f2_fma(XH[q], NM, dY[q]), R);
        }
        if (h + j < nh) {
          float res[8];
#pragma unroll
          for (int q = 0; q < 4; ++q) f2_unpack(R4[q], res[2 * q], res[2 * q + 1]);
          store_pair_bf16(op + (h + j) * o_h, res);
        }
      }
    }
  }

  if constexpr (BWD) {
#pragma unroll
    for (int q = 0; q < 4; ++q) f2_unpack(DW[q], dw[2 * q], dw[2 * q + 1]);
  }
  if constexpr (BWD) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      atomicAdd(&dw_s[d0 + i], dw[i]);
      atomicAdd(&dw_s[d0 + 64 + i], dw[i + 4]);
    }
    __syncthreads();
    if (tid < 128u) atomicAdd(p.dw[z] + tid, dw_s[tid]);
  }
}

static bool rows_ok(const void* p, const int64_t st[3]) {
  return aligned16(p) && st[0] % 8 == 0 && st[1] % 8 == 0 && st[2] % 8 == 0;
}

template <bool BWD>
static int launch(const pith_qk_norm_rope_args* a, void* stream) {
  PITH_REQUIRE(a != nullptr, "null argument struct");
  PITH_REQUIRE(a->B >= 0 && a->S >= 0 && a->Hq >= 0 && a->Hkv >= 0, "negative size");
  PITH_REQUIRE(a->D == 128, "head_dim %d is not supported (128 only)", a->D);
  if (a->B == 0 || a->S == 0 || a->Hq + a->Hkv == 0) return kOk;
  PITH_REQUIRE(a->B <= 65535, "B exceeds 65535");
  PITH_REQUIRE(a->q_weight && a->k_weight && a->cos && a->sin, "null weight or cos/sin pointer");
  PITH_REQUIRE(aligned16(a->q_weight) && aligned16(a->k_weight) && aligned16(a->cos) && aligned16(a->sin),
               "weights and cos/sin must be 16-byte aligned");
  PITH_REQUIRE(a->cs_stride[0] % 8 == 0 && a->cs_stride[1] % 8 == 0, "cos/sin strides must be multiples of 8 elements");
  PITH_REQUIRE((a->weight_dtype == PITH_DTYPE_BF16 || a->weight_dtype == PITH_DTYPE_F32) &&
                   (a->cs_dtype == PITH_DTYPE_BF16 || a->cs_dtype == PITH_DTYPE_F32),
               "weight_dtype and cs_dtype must be PITH_DTYPE_BF16 or PITH_DTYPE_F32");
  if (int rc = require_sm100()) return rc;
  QkParams p = {};
  const void* xin[2] = {a->q, a->k};
  void* xout[2] = {a->q_out, a->k_out};
  const void* gin[2] = {a->dq_out, a->dk_out};
  float* dws[2] = {a->dq_weight, a->dk_weight};
  const int heads[2] = {a->Hq, a->Hkv};
  const int64_t* xs[2] = {a->q_stride, a->k_stride};
  const int64_t* os[2] = {a->q_out_stride, a->k_out_stride};
  const int64_t* gs[2] = {a->dq_out_stride, a->dk_out_stride};
  for (int i = 0; i < 2; ++i) {
    if (heads[i] > 0) {
      PITH_REQUIRE(xin[i] && xout[i], "null input or output pointer");
      PITH_REQUIRE(rows_ok(xin[i], xs[i]) && rows_ok(xout[i], os[i]),
                   "q/k tensors must be 16-byte aligned with strides that are multiples of 8 elements");
      if (BWD) {
        PITH_REQUIRE(gin[i] && rows_ok(gin[i], gs[i]), "output gradients must be 16-byte aligned, strides multiples of 8");
      }
    }
    if (BWD) PITH_REQUIRE(dws[i] != nullptr, "null weight-gradient pointer");
    p.x[i] = static_cast<const __nv_bfloat16*>(xin[i]);
    p.out[i] = static_cast<__nv_bfloat16*>(xout[i]);
    p.dz[i] = static_cast<const __nv_bfloat16*>(gin[i]);
    p.dw[i] = dws[i];
    for (int j = 0; j < 3; ++j) { p.xs[i][j] = xs[i][j]; p.os[i][j] = os[i][j]; p.dzs[i][j] = gs[i][j]; }
  }
  p.w[0] = a->q_weight; p.w[1] = a->k_weight;
  p.cos = a->cos; p.sin = a->sin;
  p.B = a->B; p.S = a->S; p.Hq = a->Hq; p.Hkv = a->Hkv; p.eps = a->eps;
  p.cs[0] = a->cs_stride[0]; p.cs[1] = a->cs_stride[1];
  constexpr int G = BWD ? PITH_QK_G_BWD : PITH_QK_G_FWD;  // rows a thread has in flight
  const int chunks = (a->Hq + kHeadChunk - 1) / kHeadChunk + (a->Hkv + kHeadChunk - 1) / kHeadChunk;
  PITH_REQUIRE(chunks <= 65535, "too many heads");
  int sms = 148;
  {
    int dev = 0;
    PITH_CUDA(cudaGetDevice(&dev));
    PITH_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  // 16 positions per CTA and pass; about 16 CTAs per SM over all batch entries and head chunks, never more than
  // there are groups of 16 positions
  int64_t gx = (static_cast<int64_t>(sms) * 16 + static_cast<int64_t>(a->B) * chunks - 1) /
               (static_cast<int64_t>(a->B) * chunks);
  const int64_t need = (static_cast<int64_t>(a->S) + 15) / 16;
  if (gx > need) gx = need;
  if (gx < 1) gx = 1;
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(a->B), static_cast<unsigned>(chunks));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool wf = a->weight_dtype == PITH_DTYPE_F32, cf = a->cs_dtype == PITH_DTYPE_F32;
  if (wf && cf) qk_norm_rope_kernel<BWD, true, true, G><<<grid, 256, 0, st>>>(p);
  else if (wf) qk_norm_rope_kernel<BWD, true, false, G><<<grid, 256, 0, st>>>(p);
  else if (cf) qk_norm_rope_kernel<BWD, false, true, G><<<grid, 256, 0, st>>>(p);
  else qk_norm_rope_kernel<BWD, false, false, G><<<grid, 256, 0, st>>>(p);
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace pith

extern "C" int pith_qk_norm_rope_fwd(const pith_qk_norm_rope_args* a, void* stream) {
  return pith::launch<false>(a, stream);
}

extern "C" int pith_qk_norm_rope_bwd(const pith_qk_norm_rope_args* a, void* stream) {
  return pith::launch<true>(a, stream);
}
