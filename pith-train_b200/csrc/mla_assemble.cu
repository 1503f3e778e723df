// The step in front of the MLA attention operator, fused: rotary embedding of the rope parts of Q and K (DeepSeek
// form: interleaved pairs are de-interleaved, then rotate-half) and the assembly of the operator's inputs
//
//   query[b][s][h] = [ q_nope (128) | rope(q_pe) (64) ]
//   key  [b][s][h] = [ k_nope (128) | rope(k_pe[b][s]) (64, the same for every head) ]
//   value[b][s][h] =   v (128), contiguous
//
// from q = [q_nope | q_pe] (192 per head), kv = [k_nope | v] (256 per head) and k_pe (64 per position), in one pass;
// and the backward of all of it in one pass (dk_pe sums the rope part of dkey over the heads).
//
// With x the 64 rope inputs of one row, the result is  out[j] = x[2j] cos[j] - x[2j+1] sin[j],
// out[32+j] = x[2j+1] cos[32+j] + x[2j] sin[32+j]  (j < 32): both outputs depend on one interleaved input pair, so a
// lane that holds 8 consecutive inputs (4 pairs) produces outputs [4l, 4l+4) and [32+4l, 32+4l+4) on its own.
//
// One warp per position walks through the heads (the forward through a chunk of four; blockIdx.z picks the chunk):
// lanes 0-15 move the 128 "nope" elements of Q (and dQ), lanes 16-23 rotate the 64 rope elements; all 32 lanes move
// the 256-element kv row; the rotated k_pe is computed once per position and chunk (lanes 24-31) and stored for
// every head.
#include "../../include/pith_b200.h"
#include "common.cuh"
#include "host_common.h"

namespace pith {

struct MlaAsmParams {
  // forward inputs / backward outputs
  __nv_bfloat16* q;     // [B][S][H][192]
  __nv_bfloat16* kv;    // [B][S][H][256]
  __nv_bfloat16* k_pe;  // [B][S][64]
  // forward outputs / backward inputs
  __nv_bfloat16* query;  // [B][S][H][192]
  __nv_bfloat16* key;    // [B][S][H][192]
  __nv_bfloat16* value;  // [B][S][H][128]
  const void* cos;
  const void* sin;
  int B, S, H;
  int64_t qs[3], kvs[3], qys[3], kys[3], vs[3];  // b, s, h strides (elements)
  int64_t kps[2], cs[2];                         // b, s strides
};

__device__ __forceinline__ void unpack8(const uint4 u, float (&v)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

template <bool F32>
__device__ __forceinline__ void load4(const void* base, int64_t off, float (&v)[4]) {
  if constexpr (F32) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(base) + off));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  } else {
    const uint2 u = __ldg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(base) + off));
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xFFFF0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xFFFF0000u);
  }
}

// Forward rotation of 4 interleaved pairs x[0..8) -> lo[4] (outputs 4l..4l+3), hi[4] (outputs 32+4l..).
__device__ __forceinline__ void rope_fwd(const float (&x)[8], const float (&cl)[4], const float (&sl)[4],
                                         const float (&ch)[4], const float (&sh)[4], float (&lo)[4], float (&hi)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo[i] = fmaf(x[2 * i], cl[i], -x[2 * i + 1] * sl[i]);
    hi[i] = fmaf(x[2 * i + 1], ch[i], x[2 * i] * sh[i]);
  }
}

// Transpose of the above: gradients lo[4], hi[4] of the outputs -> gradient of the 4 interleaved input pairs.
__device__ __forceinline__ void rope_bwd(const float (&lo)[4], const float (&hi)[4], const float (&cl)[4],
                                         const float (&sl)[4], const float (&ch)[4], const float (&sh)[4],
                                         float (&dx)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    dx[2 * i] = fmaf(lo[i], cl[i], hi[i] * sh[i]);
    dx[2 * i + 1] = fmaf(hi[i], ch[i], -lo[i] * sl[i]);
  }
}

__device__ __forceinline__ uint2 pack4(const float (&v)[4]) {
  return make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
}

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}

constexpr int kFwdHeads = 4;  // heads per work item (blockIdx.z picks the chunk)

template <bool BWD, bool CS_F32>
__global__ void __launch_bounds__(256) mla_assemble_kernel(const MlaAsmParams p) {
  const uint32_t lane = threadIdx.x & 31u;
  const int b = blockIdx.y;
  const bool rope_q = lane >= 16u && lane < 24u, rope_k = lane >= 24u;
  const int l8 = static_cast<int>(lane & 7u);  // which 4 pairs of the rope part this lane owns (lanes 16-31)
  for (int s = static_cast<int>(blockIdx.x * 8u + (threadIdx.x >> 5)); s < p.S; s += static_cast<int>(gridDim.x) * 8) {
    float cl[4] = {}, sl[4] = {}, ch[4] = {}, sh[4] = {};
    if (lane >= 16u) {
      const int64_t co = b * p.cs[0] + s * p.cs[1] + 4 * l8;
      load4<CS_F32>(p.cos, co, cl);
      load4<CS_F32>(p.sin, co, sl);
      load4<CS_F32>(p.cos, co + 32, ch);
      load4<CS_F32>(p.sin, co + 32, sh);
    }
    __nv_bfloat16* qrow = p.q + b * p.qs[0] + s * p.qs[1];
    __nv_bfloat16* kvrow = p.kv + b * p.kvs[0] + s * p.kvs[1];
    __nv_bfloat16* qyrow = p.query + b * p.qys[0] + s * p.qys[1];
    __nv_bfloat16* kyrow = p.key + b * p.kys[0] + s * p.kys[1];
    __nv_bfloat16* vrow = p.value + b * p.vs[0] + s * p.vs[1];
    __nv_bfloat16* kpe = p.k_pe + b * p.kps[0] + s * p.kps[1] + 8 * l8;
    if constexpr (!BWD) {
      uint2 klo = make_uint2(0u, 0u), khi = make_uint2(0u, 0u);  // rotated k_pe of this position (lanes 24-31)
      if (rope_k) {
        float x[8], lo[4], hi[4];
        unpack8(__ldg(reinterpret_cast<const uint4*>(kpe)), x);
        rope_fwd(x, cl, sl, ch, sh, lo, hi);
        klo = pack4(lo);
        khi = pack4(hi);
      }
      // the forward splits the heads over blockIdx.z in chunks of kFwdHeads; all loads of a chunk are issued first
      const int hbeg = static_cast<int>(blockIdx.z) * kFwdHeads;
      uint4 kvv[kFwdHeads], qv[kFwdHeads];
#pragma unroll
      for (int j = 0; j < kFwdHeads; ++j) {
        const int h = min(hbeg + j, p.H - 1);
        kvv[j] = __ldg(reinterpret_cast<const uint4*>(kvrow + h * p.kvs[2]) + lane);
        qv[j] = lane < 24u ? __ldg(reinterpret_cast<const uint4*>(qrow + h * p.qs[2]) + lane) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < kFwdHeads; ++j) {
        const int h = hbeg + j;
        if (h >= p.H) break;
        __nv_bfloat16* qy = qyrow + h * p.qys[2];
        __nv_bfloat16* ky = kyrow + h * p.kys[2];
        if (lane < 16u) {
          *(reinterpret_cast<uint4*>(qy) + lane) = qv[j];
          *(reinterpret_cast<uint4*>(ky) + lane) = kvv[j];
        } else {
          *(reinterpret_cast<uint4*>(vrow + h * p.vs[2]) + (lane - 16u)) = kvv[j];
          if (rope_q) {
            float x[8], lo[4], hi[4];
            unpack8(qv[j], x);
            rope_fwd(x, cl, sl, ch, sh, lo, hi);
            *reinterpret_cast<uint2*>(qy + 128 + 4 * l8) = pack4(lo);
            *reinterpret_cast<uint2*>(qy + 160 + 4 * l8) = pack4(hi);
          } else {
            *reinterpret_cast<uint2*>(ky + 128 + 4 * l8) = klo;
            *reinterpret_cast<uint2*>(ky + 160 + 4 * l8) = khi;
          }
        }
      }
    } else {
      // Like the forward: a chunk of kFwdHeads heads per blockIdx.z, loads first. The rope part of dkey is summed
      // over ALL heads by lanes 24-31 of chunk 0 only (16 x 128 bytes per position), which then write dk_pe.
      const int hbeg = static_cast<int>(blockIdx.z) * kFwdHeads;
      uint4 a[kFwdHeads], c[kFwdHeads];  // lanes 0-15: dquery nope, dkey nope; lanes 16-31: rope source, dvalue
#pragma unroll
      for (int j = 0; j < kFwdHeads; ++j) {
        const int h = min(hbeg + j, p.H - 1);
        const __nv_bfloat16* qy = qyrow + h * p.qys[2];
        const __nv_bfloat16* ky = kyrow + h * p.kys[2];
        if (lane < 16u) {
          a[j] = __ldg(reinterpret_cast<const uint4*>(qy) + lane);
          c[j] = __ldg(reinterpret_cast<const uint4*>(ky) + lane);
        } else {
          const uint2 lo = __ldg(reinterpret_cast<const uint2*>(qy + 128 + 4 * l8));
          const uint2 hi = __ldg(reinterpret_cast<const uint2*>(qy + 160 + 4 * l8));
          a[j] = make_uint4(lo.x, lo.y, hi.x, hi.y);
          c[j] = __ldg(reinterpret_cast<const uint4*>(vrow + h * p.vs[2]) + (lane - 16u));
        }
      }
#pragma unroll
      for (int j = 0; j < kFwdHeads; ++j) {
        const int h = hbeg + j;
        if (h >= p.H) break;
        __nv_bfloat16* qh = qrow + h * p.qs[2];     // dq (output)
        __nv_bfloat16* kvh = kvrow + h * p.kvs[2];  // dkv (output)
        *(reinterpret_cast<uint4*>(kvh) + lane) = c[j];
        if (lane < 16u) {
          *(reinterpret_cast<uint4*>(qh) + lane) = a[j];
        } else if (rope_q) {
          float g[8], lo[4], hi[4], dx[8];
          unpack8(a[j], g);  // g[0..4) = gradient of outputs 4l..4l+3, g[4..8) = of outputs 32+4l..
#pragma unroll
          for (int i = 0; i < 4; ++i) { lo[i] = g[i]; hi[i] = g[4 + i]; }
          rope_bwd(lo, hi, cl, sl, ch, sh, dx);
          *(reinterpret_cast<uint4*>(qh) + lane) = pack8(dx);
        }
      }
      if (rope_k && blockIdx.z == 0) {
        float klo[4] = {}, khi[4] = {};
#pragma unroll 4
        for (int h = 0; h < p.H; ++h) {
          float lo[4], hi[4];
          load4<false>(kyrow + h * p.kys[2], 128 + 4 * l8, lo);
          load4<false>(kyrow + h * p.kys[2], 160 + 4 * l8, hi);
#pragma unroll
          for (int i = 0; i < 4; ++i) { klo[i] += lo[i]; khi[i] += hi[i]; }
        }
        float dx[8];
        rope_bwd(klo, khi, cl, sl, ch, sh, dx);
        *reinterpret_cast<uint4*>(kpe) = pack8(dx);
      }
    }
  }
}

static bool ok3(const void* p, const int64_t st[3]) {
  return p != nullptr && aligned16(p) && st[0] % 8 == 0 && st[1] % 8 == 0 && st[2] % 8 == 0;
}

template <bool BWD>
static int launch_mla_assemble(const pith_mla_assemble_args* a, void* stream) {
  PITH_REQUIRE(a != nullptr, "null argument struct");
  PITH_REQUIRE(a->B >= 0 && a->S >= 0 && a->H >= 0, "negative size");
  PITH_REQUIRE(a->Dnope == 128 && a->Drope == 64 && a->Dv == 128,
               "only qk_nope_head_dim 128, qk_rope_head_dim 64, v_head_dim 128 are supported (got %d, %d, %d)",
               a->Dnope, a->Drope, a->Dv);
  if (a->B == 0 || a->S == 0 || a->H == 0) return kOk;
  PITH_REQUIRE(a->B <= 65535, "B exceeds 65535");
  PITH_REQUIRE(a->cs_dtype == PITH_DTYPE_BF16 || a->cs_dtype == PITH_DTYPE_F32, "cs_dtype must be PITH_DTYPE_*");
  void* q = BWD ? a->dq : const_cast<void*>(a->q);
  void* kv = BWD ? a->dkv : const_cast<void*>(a->kv);
  void* kpe = BWD ? a->dk_pe : const_cast<void*>(a->k_pe);
  void* query = BWD ? const_cast<void*>(a->dquery) : a->query;
  void* key = BWD ? const_cast<void*>(a->dkey) : a->key;
  void* value = BWD ? const_cast<void*>(a->dvalue) : a->value;
  PITH_REQUIRE(ok3(q, a->q_stride) && ok3(kv, a->kv_stride) && ok3(query, a->query_stride) && ok3(key, a->key_stride) &&
                   ok3(value, a->value_stride),
               "tensors must be non-null, 16-byte aligned, with strides that are multiples of 8 elements");
  PITH_REQUIRE(kpe != nullptr && aligned16(kpe) && a->k_pe_stride[0] % 8 == 0 && a->k_pe_stride[1] % 8 == 0,
               "k_pe must be 16-byte aligned with strides that are multiples of 8 elements");
  PITH_REQUIRE(a->cos && a->sin && aligned16(a->cos) && aligned16(a->sin) && a->cs_stride[0] % 4 == 0 &&
                   a->cs_stride[1] % 4 == 0,
               "cos/sin must be 16-byte aligned with strides that are multiples of 4 elements");
  if (int rc = require_sm100()) return rc;
  MlaAsmParams p = {};
  p.q = static_cast<__nv_bfloat16*>(q); p.kv = static_cast<__nv_bfloat16*>(kv); p.k_pe = static_cast<__nv_bfloat16*>(kpe);
  p.query = static_cast<__nv_bfloat16*>(query); p.key = static_cast<__nv_bfloat16*>(key);
  p.value = static_cast<__nv_bfloat16*>(value);
  p.cos = a->cos; p.sin = a->sin;
  p.B = a->B; p.S = a->S; p.H = a->H;
  for (int i = 0; i < 3; ++i) {
    p.qs[i] = a->q_stride[i]; p.kvs[i] = a->kv_stride[i]; p.qys[i] = a->query_stride[i];
    p.kys[i] = a->key_stride[i]; p.vs[i] = a->value_stride[i];
  }
  for (int i = 0; i < 2; ++i) { p.kps[i] = a->k_pe_stride[i]; p.cs[i] = a->cs_stride[i]; }
  int sms = 148;
  {
    int dev = 0;
    PITH_CUDA(cudaGetDevice(&dev));
    PITH_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  // 8 positions per CTA and pass; about 16 CTAs per SM over all batch entries and head chunks
  const int chunks = (a->H + kFwdHeads - 1) / kFwdHeads;
  PITH_REQUIRE(chunks <= 65535, "too many heads");
  int64_t gx = (static_cast<int64_t>(sms) * 16 + static_cast<int64_t>(a->B) * chunks - 1) /
               (static_cast<int64_t>(a->B) * chunks);
  const int64_t need = (static_cast<int64_t>(a->S) + 7) / 8;
  if (gx > need) gx = need;
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(a->B), static_cast<unsigned>(chunks));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->cs_dtype == PITH_DTYPE_F32) mla_assemble_kernel<BWD, true><<<grid, 256, 0, st>>>(p);
  else mla_assemble_kernel<BWD, false><<<grid, 256, 0, st>>>(p);
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

}  // namespace pith

extern "C" int pith_mla_assemble_fwd(const pith_mla_assemble_args* a, void* stream) {
  return pith::launch_mla_assemble<false>(a, stream);
}

extern "C" int pith_mla_assemble_bwd(const pith_mla_assemble_args* a, void* stream) {
  return pith::launch_mla_assemble<true>(a, stream);
}
