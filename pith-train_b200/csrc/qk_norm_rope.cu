// The step in front of the attention operator, fused: per-head RMSNorm of Q and K followed by rotary position
// embedding (rotate-half form), forward and backward, one HBM pass each.
//
//   y = x * rsqrt(mean(x^2) + eps) * w          (per [b][s][h] row of head_dim = 128)
//   z[i]      = y[i]      * cos[i]      - y[i + 64] * sin[i]           i < 64
//   z[i + 64] = y[i + 64] * cos[i + 64] + y[i]      * sin[i + 64]
//
// Sixteen lanes own one row (8 consecutive elements each, 16-byte accesses); the rotate-half partner of lane j is
// lane j ^ 8 and the row reductions are four shuffles. Q rows and K rows go through the same launch. cos/sin are
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

__device__ __forceinline__ void load8_bf16(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

template <bool F32>
__device__ __forceinline__ void load8_any(const void* base, int64_t off, float (&v)[8]) {
  if constexpr (F32) {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + off);
    const float4 a = __ldg(p), b = __ldg(p + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    load8_bf16(static_cast<const __nv_bfloat16*>(base) + off, v);
  }
}

__device__ __forceinline__ void store8_bf16(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16(v[0], v[1]); u.y = pack_bf16(v[2], v[3]); u.z = pack_bf16(v[4], v[5]); u.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ float sum16(float v) {  // over the 16 lanes that share a row
  v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
  v += __shfl_xor_sync(0xFFFFFFFFu, v, 4);
  v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
  v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
  return v;
}

template <bool BWD, bool W_F32, bool CS_F32>
__global__ void __launch_bounds__(256) qk_norm_rope_kernel(const QkParams p) {
  __shared__ float dw_s[2][128];
  const uint32_t tid = threadIdx.x, lane16 = tid & 15u;
  const bool upper = lane16 >= 8u;  // this lane owns elements of the second half of the row
  const uint32_t htot = static_cast<uint32_t>(p.Hq + p.Hkv);
  const uint32_t items = static_cast<uint32_t>(p.S) * htot;  // rows of one batch entry
  const uint32_t stride = gridDim.x * 16u;
  const uint32_t first = (blockIdx.x * 256u + tid) >> 4;
  const uint32_t trips = (items + stride - 1u) / stride;  // the same for every lane: the shuffles need whole warps
  const int b = blockIdx.y;
  const int d0 = static_cast<int>(lane16) * 8;

  float w[2][8];
  load8_any<W_F32>(p.w[0], d0, w[0]);
  load8_any<W_F32>(p.w[1], d0, w[1]);
  float dw[2][8] = {};
  if constexpr (BWD) {
    dw_s[tid >> 7][tid & 127u] = 0.f;
    __syncthreads();
  }

  for (uint32_t t = 0; t < trips; ++t) {
    const uint32_t item = first + t * stride;
    const bool valid = item < items;
    const uint32_t s = valid ? item / htot : 0u;
    const uint32_t hh = valid ? item - s * htot : 0u;
    const int which = hh >= static_cast<uint32_t>(p.Hq) ? 1 : 0;
    const int h = static_cast<int>(hh) - (which ? p.Hq : 0);
    float x[8] = {}, c[8] = {}, sn[8] = {}, g[8] = {};
    if (valid) {
      load8_bf16(p.x[which] + b * p.xs[which][0] + s * p.xs[which][1] + h * p.xs[which][2] + d0, x);
      const int64_t co = b * p.cs[0] + s * p.cs[1] + d0;
      load8_any<CS_F32>(p.cos, co, c);
      load8_any<CS_F32>(p.sin, co, sn);
      if constexpr (BWD)
        load8_bf16(p.dz[which] + b * p.dzs[which][0] + s * p.dzs[which][1] + h * p.dzs[which][2] + d0, g);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
    const float r = rsqrtf(sum16(ss) * (1.f / 128.f) + p.eps);
    float res[8], wv[8];  // selects instead of indexing by `which`: keeps the arrays in registers
#pragma unroll
    for (int i = 0; i < 8; ++i) wv[i] = which ? w[1][i] : w[0][i];
    if constexpr (!BWD) {
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = x[i] * r * wv[i];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float partner = __shfl_xor_sync(0xFFFFFFFFu, y[i], 8);
        res[i] = fmaf(y[i], c[i], (upper ? partner : -partner) * sn[i]);
      }
    } else {
      // dy = dz * cos + rotate_half^T(dz * sin): the partner's dz * sin comes back with the opposite sign
      float gx = 0.f, dy[8], xh[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float partner = __shfl_xor_sync(0xFFFFFFFFu, g[i] * sn[i], 8);
        dy[i] = fmaf(g[i], c[i], upper ? -partner : partner);
        xh[i] = x[i] * r;
        const float dwi = dy[i] * xh[i];
        dw[0][i] += which ? 0.f : dwi;
        dw[1][i] += which ? dwi : 0.f;
        dy[i] *= wv[i];
        gx = fmaf(dy[i], xh[i], gx);
      }
      const float m = sum16(gx) * (1.f / 128.f);
#pragma unroll
      for (int i = 0; i < 8; ++i) res[i] = r * (dy[i] - xh[i] * m);
    }
    if (valid)
      store8_bf16(p.out[which] + b * p.os[which][0] + s * p.os[which][1] + h * p.os[which][2] + d0, res);
  }

  if constexpr (BWD) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      atomicAdd(&dw_s[0][d0 + i], dw[0][i]);
      atomicAdd(&dw_s[1][d0 + i], dw[1][i]);
    }
    __syncthreads();
    atomicAdd(p.dw[tid >> 7] + (tid & 127u), dw_s[tid >> 7][tid & 127u]);
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
  PITH_REQUIRE(static_cast<int64_t>(a->S) * (a->Hq + a->Hkv) < (1ll << 31), "S * (Hq + Hkv) exceeds 2^31");
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
  const int64_t items = static_cast<int64_t>(a->S) * (a->Hq + a->Hkv);
  int sms = 148;
  {
    int dev = 0;
    PITH_CUDA(cudaGetDevice(&dev));
    PITH_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  // 8 resident CTAs per SM over all batch entries; never more CTAs than there are 16-row groups
  int64_t gx = (static_cast<int64_t>(sms) * 8 + a->B - 1) / a->B;
  const int64_t need = (items + 15) / 16;
  if (gx > need) gx = need;
  if (gx < 1) gx = 1;
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(a->B));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool wf = a->weight_dtype == PITH_DTYPE_F32, cf = a->cs_dtype == PITH_DTYPE_F32;
  if (wf && cf) qk_norm_rope_kernel<BWD, true, true><<<grid, 256, 0, st>>>(p);
  else if (wf) qk_norm_rope_kernel<BWD, true, false><<<grid, 256, 0, st>>>(p);
  else if (cf) qk_norm_rope_kernel<BWD, false, true><<<grid, 256, 0, st>>>(p);
  else qk_norm_rope_kernel<BWD, false, false><<<grid, 256, 0, st>>>(p);
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
