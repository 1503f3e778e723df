// HBM-bound kernels of the ring-attention path: the online-softmax merge of two partial
// results, of up to 16 partial results in one pass, delta = rowsum(O * dO), and the final fp32 -> bf16 rounding of
// an accumulator.
// Each thread moves 8 consecutive elements of one [b][s][h] row with 16-byte accesses.
// The grid is (blocks per plane, H, B): a block stays inside one (batch, head) plane and walks
// consecutive s, so the row data and the [B][H][S] statistics are read and written in whole
// sectors and all index arithmetic is 32-bit (a 64-bit divide per element would make these
// kernels instruction-bound).
#include "../../include/pith_b200.h"
#include "common.cuh"
#include "host_common.h"

namespace pith {

struct Vec8 {
  float v[8];
};

template <bool F32>
__device__ __forceinline__ Vec8 load8(const void* base, int64_t elem_off) {
  Vec8 r;
  if constexpr (F32) {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem_off);
    float4 a = __ldg(p), b = __ldg(p + 1);
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
    r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
  } else {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + elem_off));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      r.v[2 * i] = __uint_as_float(w[i] << 16);
      r.v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
  return r;
}

struct CombineParams {
  const void* out1;
  const void* out2;
  const float* lse1;
  const float* lse2;
  float* out;
  float* lse;
  int B, S, H, D;
  int64_t o1s[3], o2s[3];
  int64_t l1s[2], l2s[2];
};

template <bool F32A, bool F32B, bool NATURAL>
__global__ void __launch_bounds__(256) combine_kernel(const CombineParams p) {
  const uint32_t chunks = static_cast<uint32_t>(p.D) >> 3;
  const uint32_t plane = static_cast<uint32_t>(p.S) * chunks;  // items of one (b, h) plane
  const int h = blockIdx.y, b = blockIdx.z;
  const char* o1 = static_cast<const char*>(p.out1) + (b * p.o1s[0] + h * p.o1s[2]) * (F32A ? 4 : 2);
  const char* o2 = static_cast<const char*>(p.out2) + (b * p.o2s[0] + h * p.o2s[2]) * (F32B ? 4 : 2);
  const float* l1p = p.lse1 + b * p.l1s[0] + h * p.l1s[1];
  const float* l2p = p.lse2 + b * p.l2s[0] + h * p.l2s[1];
  float* outp = p.out + (static_cast<int64_t>(b) * p.S * p.H + h) * p.D;
  float* lsep = p.lse + (static_cast<int64_t>(b) * p.H + h) * p.S;
  const int64_t out_row = static_cast<int64_t>(p.H) * p.D;
  for (uint32_t item = blockIdx.x * 256u + threadIdx.x; item < plane; item += gridDim.x * 256u) {
    const uint32_t s = item / chunks, d0 = (item - s * chunks) << 3;
    const float l1 = __ldg(l1p + s), l2 = __ldg(l2p + s);
    const Vec8 a = load8<F32A>(o1, s * p.o1s[1] + d0);
    const Vec8 c = load8<F32B>(o2, s * p.o2s[1] + d0);
    const float mx = fmaxf(l1, l2);
    float e1, e2, lse;
    if constexpr (NATURAL) {
      e1 = expf(l1 - mx);
      e2 = expf(l2 - mx);
      lse = mx + logf(e1 + e2);
    } else {
      e1 = exp2f(l1 - mx);
      e2 = exp2f(l2 - mx);
      lse = mx + log2f(e1 + e2);
    }
    const float den = e1 + e2;
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = (e1 * a.v[i] + e2 * c.v[i]) / den;
    float4* dst = reinterpret_cast<float4*>(outp + s * out_row + d0);
    dst[0] = make_float4(o[0], o[1], o[2], o[3]);
    dst[1] = make_float4(o[4], o[5], o[6], o[7]);
    if (d0 == 0) lsep[s] = lse;
  }
}

struct PartialsParams {
  const __nv_bfloat16* o[PITH_MAX_PARTIALS];
  const float* lse[PITH_MAX_PARTIALS];
  int row_begin[PITH_MAX_PARTIALS], rows[PITH_MAX_PARTIALS];
  int64_t os[PITH_MAX_PARTIALS][3];
  int64_t ls[PITH_MAX_PARTIALS][2];
  int n;
  __nv_bfloat16* out;
  float* lse_out;
  int B, S, H, D;
};

// One pass over the output: a thread owns 8 columns of a row. Rows are walked in storage order (s, then h), so every
// partial and the output are streamed linearly (eight input streams: walking one head's rows, 8 KB apart, kept too
// many DRAM pages open); the [B][H][S] LSEs are then read with a stride, but they are 1/64 of the bytes and every
// sector serves eight consecutive rows. The LSEs of all partials are loaded first (one register each), then the rows
// of eight partials at a time, so that up to eight 16-byte loads per thread are in flight; the weighted mean is
// written as bf16. Grid (blocks per batch, 1, B).
__global__ void __launch_bounds__(256) combine_partials_kernel(const __grid_constant__ PartialsParams p) {
  const uint32_t chunks = static_cast<uint32_t>(p.D) >> 3;
  const uint32_t H = static_cast<uint32_t>(p.H);
  const uint32_t plane = static_cast<uint32_t>(p.S) * H * chunks;
  const int b = blockIdx.z;
  __nv_bfloat16* outb = p.out + static_cast<int64_t>(b) * p.S * p.H * p.D;
  float* lseb = p.lse_out + static_cast<int64_t>(b) * p.H * p.S;
  for (uint32_t item = blockIdx.x * 256u + threadIdx.x; item < plane; item += gridDim.x * 256u) {
    const uint32_t row = item / chunks, d0 = (item - row * chunks) << 3;
    const int s = static_cast<int>(row / H), h = static_cast<int>(row - static_cast<uint32_t>(s) * H);
    __nv_bfloat16* outp = outb + static_cast<int64_t>(h) * p.D;
    float* lsep = lseb + static_cast<int64_t>(h) * p.S;
    const int64_t out_row = static_cast<int64_t>(p.H) * p.D;
    float l[PITH_MAX_PARTIALS];
#pragma unroll
    for (int t = 0; t < PITH_MAX_PARTIALS; ++t) {
      const int r = s - p.row_begin[t];
      l[t] = -INFINITY;
      if (t < p.n && r >= 0 && r < p.rows[t]) l[t] = __ldg(p.lse[t] + b * p.ls[t][0] + h * p.ls[t][1] + r);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int t = 0; t < PITH_MAX_PARTIALS; ++t) mx = fmaxf(mx, l[t]);
    float den = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (mx > -INFINITY) {
#pragma unroll
      for (int g = 0; g < PITH_MAX_PARTIALS; g += 8) {
        if (g >= p.n) break;
        uint4 raw[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int t = g + j;
          raw[j] = make_uint4(0u, 0u, 0u, 0u);
          if (l[t] > -INFINITY)  // implies t < n and the row is covered
            raw[j] = __ldg(reinterpret_cast<const uint4*>(
                p.o[t] + b * p.os[t][0] + static_cast<int64_t>(s - p.row_begin[t]) * p.os[t][1] + h * p.os[t][2] + d0));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float w = l[g + j] > -INFINITY ? exp2f(l[g + j] - mx) : 0.f;
          den += w;
          const uint32_t u[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[2 * i] = fmaf(w, __uint_as_float(u[i] << 16), acc[2 * i]);
            acc[2 * i + 1] = fmaf(w, __uint_as_float(u[i] & 0xFFFF0000u), acc[2 * i + 1]);
          }
        }
      }
    }
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    uint4 u;
    u.x = pack_bf16(acc[0] * inv, acc[1] * inv);
    u.y = pack_bf16(acc[2] * inv, acc[3] * inv);
    u.z = pack_bf16(acc[4] * inv, acc[5] * inv);
    u.w = pack_bf16(acc[6] * inv, acc[7] * inv);
    *reinterpret_cast<uint4*>(outp + s * out_row + d0) = u;
    if (d0 == 0) lsep[s] = den > 0.f ? mx + log2f(den) : -INFINITY;
  }
}

struct DeltaParams {
  const void* o;
  const void* dout;
  float* delta;
  int B, S, H, D;
  int64_t os[3], dos[3];
  int64_t ds[2];
};

// `chunks` lanes (a power of two, 16 for D = 128) share one row; partial dot products are folded with shuffles.
__global__ void __launch_bounds__(256) delta_kernel(const DeltaParams p) {
  const uint32_t chunks = static_cast<uint32_t>(p.D) >> 3;  // power of two <= 32 (checked on the host)
  const uint32_t plane = static_cast<uint32_t>(p.S) * chunks;
  const int h = blockIdx.y, b = blockIdx.z;
  const __nv_bfloat16* op = static_cast<const __nv_bfloat16*>(p.o) + b * p.os[0] + h * p.os[2];
  const __nv_bfloat16* dp = static_cast<const __nv_bfloat16*>(p.dout) + b * p.dos[0] + h * p.dos[2];
  float* out = p.delta + b * p.ds[0] + h * p.ds[1];
  const uint32_t stride = gridDim.x * 256u;
  const uint32_t rounds = (plane + stride - 1) / stride;
  uint32_t item = blockIdx.x * 256u + threadIdx.x;
  for (uint32_t it = 0; it < rounds; ++it, item += stride) {
    float acc = 0.f;
    const bool live = item < plane;
    const uint32_t s = item / chunks, d0 = (item - s * chunks) << 3;
    if (live) {
      const Vec8 a = load8<false>(op, s * p.os[1] + d0);
      const Vec8 c = load8<false>(dp, s * p.dos[1] + d0);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf(a.v[i], c.v[i], acc);
    }
    for (uint32_t off = chunks >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    if (live && d0 == 0) out[s] = acc;
  }
}

struct CastParams {
  const float* acc;
  __nv_bfloat16* out;
  int B, S, H, D;
  int64_t as[3], os[3];
  float scale;
};

// Grid (blocks per batch, 1, B); rows are walked in storage order (s, h).
__global__ void __launch_bounds__(256) cast_kernel(const CastParams p) {
  const uint32_t chunks = static_cast<uint32_t>(p.D) >> 3;
  const uint32_t H = static_cast<uint32_t>(p.H);
  const uint32_t plane = static_cast<uint32_t>(p.S) * H * chunks;
  const int b = blockIdx.z;
  const float* src = p.acc + b * p.as[0];
  __nv_bfloat16* dst = p.out + b * p.os[0];
  for (uint32_t item = blockIdx.x * 256u + threadIdx.x; item < plane; item += gridDim.x * 256u) {
    const uint32_t row = item / chunks, d0 = (item - row * chunks) << 3;
    const uint32_t s = row / H, h = row - s * H;
    const Vec8 a = load8<true>(src, s * p.as[1] + h * p.as[2] + d0);
    uint4 u;
    u.x = pack_bf16(a.v[0] * p.scale, a.v[1] * p.scale);
    u.y = pack_bf16(a.v[2] * p.scale, a.v[3] * p.scale);
    u.z = pack_bf16(a.v[4] * p.scale, a.v[5] * p.scale);
    u.w = pack_bf16(a.v[6] * p.scale, a.v[7] * p.scale);
    *reinterpret_cast<uint4*>(dst + s * p.os[1] + h * p.os[2] + d0) = u;
  }
}

// Blocks along x for `planes` planes of `plane_items` items: about 148 SMs x 8 resident blocks in total.
static dim3 grid_for(int64_t plane_items, int planes_y, int planes_z) {
  int64_t need = (plane_items + 255) / 256;
  int64_t planes = static_cast<int64_t>(planes_y) * planes_z;
  int64_t cap = (148 * 8 + planes - 1) / planes;
  if (cap < 1) cap = 1;
  int64_t bx = need < cap ? need : cap;
  if (bx < 1) bx = 1;
  return dim3(static_cast<unsigned>(bx), static_cast<unsigned>(planes_y), static_cast<unsigned>(planes_z));
}

static bool rows_ok(const void* base, const int64_t st[3], int elem_bytes) {
  return aligned16(base) && (st[0] * elem_bytes) % 16 == 0 && (st[1] * elem_bytes) % 16 == 0 &&
         (st[2] * elem_bytes) % 16 == 0;
}

}  // namespace pith

using namespace pith;

extern "C" int pith_combine(const pith_combine_args* a, void* stream) {
  PITH_REQUIRE(a != nullptr, "null args");
  PITH_REQUIRE(a->B >= 0 && a->S >= 0 && a->H >= 0 && a->D > 0 && a->D % 8 == 0, "bad shape %dx%dx%dx%d", a->B, a->S,
               a->H, a->D);
  if (static_cast<int64_t>(a->B) * a->S * a->H == 0) return kOk;  // empty tensors may come with null pointers
  PITH_REQUIRE(a->out1 && a->out2 && a->lse1 && a->lse2 && a->out && a->lse, "null tensor pointer");
  PITH_REQUIRE((a->out1_dtype | 1) == 1 && (a->out2_dtype | 1) == 1, "unknown dtype");
  PITH_REQUIRE(rows_ok(a->out1, a->out1_stride, a->out1_dtype == PITH_DTYPE_F32 ? 4 : 2) &&
                   rows_ok(a->out2, a->out2_stride, a->out2_dtype == PITH_DTYPE_F32 ? 4 : 2) && aligned16(a->out),
               "out tensors must be 16-byte aligned with 16-byte-multiple strides");
  if (static_cast<int64_t>(a->B) * a->S * a->H == 0) return kOk;
  if (int rc = require_sm100()) return rc;
  CombineParams p;
  p.out1 = a->out1; p.out2 = a->out2; p.lse1 = a->lse1; p.lse2 = a->lse2; p.out = a->out; p.lse = a->lse;
  p.B = a->B; p.S = a->S; p.H = a->H; p.D = a->D;
  for (int i = 0; i < 3; ++i) { p.o1s[i] = a->out1_stride[i]; p.o2s[i] = a->out2_stride[i]; }
  for (int i = 0; i < 2; ++i) { p.l1s[i] = a->lse1_stride[i]; p.l2s[i] = a->lse2_stride[i]; }
  const int64_t items = static_cast<int64_t>(a->B) * a->S * a->H * (a->D / 8);
  PITH_REQUIRE(a->H <= 65535 && a->B <= 65535 && items / a->H / a->B < (1ll << 32), "tensor too large for one launch");
  const dim3 grid = grid_for(static_cast<int64_t>(a->S) * (a->D / 8), a->H, a->B);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool nat = (a->flags & PITH_COMBINE_NATURAL) != 0;
  const int sel = (a->out1_dtype == PITH_DTYPE_F32 ? 4 : 0) | (a->out2_dtype == PITH_DTYPE_F32 ? 2 : 0) | (nat ? 1 : 0);
  switch (sel) {
    case 0: combine_kernel<false, false, false><<<grid, 256, 0, st>>>(p); break;
    case 1: combine_kernel<false, false, true><<<grid, 256, 0, st>>>(p); break;
    case 2: combine_kernel<false, true, false><<<grid, 256, 0, st>>>(p); break;
    case 3: combine_kernel<false, true, true><<<grid, 256, 0, st>>>(p); break;
    case 4: combine_kernel<true, false, false><<<grid, 256, 0, st>>>(p); break;
    case 5: combine_kernel<true, false, true><<<grid, 256, 0, st>>>(p); break;
    case 6: combine_kernel<true, true, false><<<grid, 256, 0, st>>>(p); break;
    default: combine_kernel<true, true, true><<<grid, 256, 0, st>>>(p); break;
  }
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

extern "C" int pith_combine_partials(const pith_combine_partials_args* a, void* stream) {
  PITH_REQUIRE(a != nullptr, "null args");
  PITH_REQUIRE(a->n >= 1 && a->n <= PITH_MAX_PARTIALS, "n = %d partials (1 .. %d)", a->n, PITH_MAX_PARTIALS);
  PITH_REQUIRE(a->B >= 0 && a->S >= 0 && a->H >= 0 && a->D > 0 && a->D % 8 == 0, "bad shape %dx%dx%dx%d", a->B, a->S,
               a->H, a->D);
  if (static_cast<int64_t>(a->B) * a->S * a->H == 0) return kOk;
  PITH_REQUIRE(a->out && a->lse && aligned16(a->out), "out must be a 16-byte aligned pointer, lse non-null");
  PartialsParams p = {};
  for (int t = 0; t < a->n; ++t) {
    const pith_partial& q = a->part[t];
    PITH_REQUIRE(q.rows >= 0 && q.row_begin >= 0 && static_cast<int64_t>(q.row_begin) + q.rows <= a->S,
                 "partial %d covers rows [%d, %d + %d) of %d", t, q.row_begin, q.row_begin, q.rows, a->S);
    PITH_REQUIRE(q.rows == 0 || (q.o && q.lse), "partial %d: null tensor pointer", t);
    PITH_REQUIRE(q.rows == 0 || rows_ok(q.o, q.o_stride, 2),
                 "partial %d must be 16-byte aligned with 16-byte-multiple strides", t);
    p.o[t] = static_cast<const __nv_bfloat16*>(q.o);
    p.lse[t] = q.lse;
    p.row_begin[t] = q.row_begin;
    p.rows[t] = q.rows;
    for (int i = 0; i < 3; ++i) p.os[t][i] = q.o_stride[i];
    for (int i = 0; i < 2; ++i) p.ls[t][i] = q.lse_stride[i];
  }
  if (int rc = require_sm100()) return rc;
  p.n = a->n;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse_out = a->lse;
  p.B = a->B; p.S = a->S; p.H = a->H; p.D = a->D;
  const int64_t items = static_cast<int64_t>(a->B) * a->S * a->H * (a->D / 8);
  PITH_REQUIRE(a->B <= 65535 && items / a->B < (1ll << 32), "tensor too large for one launch");
  combine_partials_kernel<<<grid_for(static_cast<int64_t>(a->S) * a->H * (a->D / 8), 1, a->B), 256, 0,
                            static_cast<cudaStream_t>(stream)>>>(p);
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

extern "C" int pith_attn_bwd_preprocess(const pith_bwd_preprocess_args* a, void* stream) {
  PITH_REQUIRE(a != nullptr, "null args");
  PITH_REQUIRE(a->o && a->dout && a->delta, "null tensor pointer");
  const int chunks = a->Dv / 8;
  PITH_REQUIRE(a->Dv > 0 && a->Dv % 8 == 0 && chunks <= 32 && (chunks & (chunks - 1)) == 0,
               "Dv = %d must be 8 * a power of two, at most 256", a->Dv);
  PITH_REQUIRE(a->B >= 0 && a->S >= 0 && a->H >= 0, "bad shape");
  PITH_REQUIRE(rows_ok(a->o, a->o_stride, 2) && rows_ok(a->dout, a->do_stride, 2),
               "o / dout must be 16-byte aligned with 16-byte-multiple strides");
  if (static_cast<int64_t>(a->B) * a->S * a->H == 0) return kOk;
  if (int rc = require_sm100()) return rc;
  DeltaParams p;
  p.o = a->o; p.dout = a->dout; p.delta = a->delta;
  p.B = a->B; p.S = a->S; p.H = a->H; p.D = a->Dv;
  for (int i = 0; i < 3; ++i) { p.os[i] = a->o_stride[i]; p.dos[i] = a->do_stride[i]; }
  p.ds[0] = a->delta_stride[0]; p.ds[1] = a->delta_stride[1];
  const int64_t items = static_cast<int64_t>(a->B) * a->S * a->H * chunks;
  PITH_REQUIRE(a->H <= 65535 && a->B <= 65535 && items / a->H / a->B < (1ll << 32), "tensor too large for one launch");
  delta_kernel<<<grid_for(static_cast<int64_t>(a->S) * chunks, a->H, a->B), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

extern "C" int pith_cast_f32_to_bf16(const float* acc, void* out, int32_t B, int32_t S, int32_t H, int32_t D,
                                     const int64_t acc_stride[3], const int64_t out_stride[3], float scale,
                                     void* stream) {
  PITH_REQUIRE(acc && out && acc_stride && out_stride, "null pointer");
  PITH_REQUIRE(B >= 0 && S >= 0 && H >= 0 && D > 0 && D % 8 == 0, "bad shape %dx%dx%dx%d", B, S, H, D);
  PITH_REQUIRE(rows_ok(acc, acc_stride, 4) && rows_ok(out, out_stride, 2),
               "tensors must be 16-byte aligned with 16-byte-multiple strides");
  if (static_cast<int64_t>(B) * S * H == 0) return kOk;
  if (int rc = require_sm100()) return rc;
  CastParams p;
  p.acc = acc; p.out = static_cast<__nv_bfloat16*>(out);
  p.B = B; p.S = S; p.H = H; p.D = D; p.scale = scale;
  for (int i = 0; i < 3; ++i) { p.as[i] = acc_stride[i]; p.os[i] = out_stride[i]; }
  const int64_t items = static_cast<int64_t>(B) * S * H * (D / 8);
  PITH_REQUIRE(B <= 65535 && items / B < (1ll << 32), "tensor too large for one launch");
  cast_kernel<<<grid_for(static_cast<int64_t>(S) * H * (D / 8), 1, B), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  PITH_CUDA(cudaGetLastError());
  return kOk;
}
