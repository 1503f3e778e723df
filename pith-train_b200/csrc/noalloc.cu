// Attention backward for callers that must not allocate device memory.
//
// pith_attn_bwd (attn_bwd.cu) adds its results into fp32 accumulators, and a complete backward also
// needs delta = rowsum(O * dO); a caller normally allocates those buffers with cudaMalloc or a framework
// allocator. Some callers cannot: a host that froze its device memory pool after start-up, a plugin living
// inside another runtime that owns every device allocation, a latency-critical loop that cannot afford the
// device-wide synchronisation cudaMalloc and cudaFree imply. For them this file keeps one fixed scratch area
// inside the library's own image (a file-scope __device__ array) and carves delta and the three
// accumulators out of it.
//
// The first call on a device looks the area's address up (cudaGetSymbolAddress, with that device current)
// and remembers it; make that first call before any stream capture begins. The remembered address belongs to
// the device's current context: a process that calls cudaDeviceReset must not use this entry point afterwards.
//
// Consequences of the shared, static scratch area:
//  - every GPU that loads the library holds kScratchBytes of device memory until the process exits;
//  - problems whose scratch need exceeds kScratchBytes are rejected with an error, never truncated;
//  - the area keeps the previous call's contents, so each call re-zeroes the accumulators it uses;
//  - two calls whose GPU work overlaps (different streams, or different host threads) race on it:
//    issue them on one stream, or order them with events.
#include <mutex>

#include "../../include/pith_b200.h"
#include "host_common.h"

namespace pith {

constexpr size_t kScratchBytes = PITH_NOALLOC_SCRATCH_BYTES;

// In host code this name is only a handle for the runtime's symbol table, not a device address:
// the address used by the kernels comes from cudaGetSymbolAddress (scratch_base below).
static __device__ __align__(256) unsigned char g_bwd_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_scratch_mutex;
static void* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch area on the CURRENT device; resolved once per device.
static int scratch_base(unsigned char** out) {
  int dev = -1;
  PITH_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(kErrUnsupported, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    PITH_CUDA(cudaGetSymbolAddress(&p, g_bwd_scratch));
    g_scratch_ptr[dev] = p;
  }
  *out = static_cast<unsigned char*>(g_scratch_ptr[dev]);
  return kOk;
}

static size_t round256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

// sizeof(float) * a * b * c * d rounded up to 256, or SIZE_MAX if that does not fit (so that a huge shape can
// never wrap around into a small byte count).
static size_t f32_bytes(int64_t a, int64_t b, int64_t c, int64_t d) {
  if (a <= 0 || b <= 0 || c <= 0 || d <= 0) return SIZE_MAX;
  unsigned long long n = sizeof(float);
  for (int64_t f : {a, b, c, d})
    if (__builtin_mul_overflow(n, static_cast<unsigned long long>(f), &n)) return SIZE_MAX;
  if (n > SIZE_MAX - 256) return SIZE_MAX;
  return round256(static_cast<size_t>(n));
}

}  // namespace pith

using namespace pith;

extern "C" size_t pith_attn_bwd_noalloc_scratch_bytes(int32_t B, int32_t Sq, int32_t Sk, int32_t Hq, int32_t Hkv,
                                                      int32_t Dqk, int32_t Dv) {
  size_t total = 0;
  for (size_t part : {f32_bytes(B, Hq, Sq, 1), f32_bytes(B, Sq, Hq, Dqk), f32_bytes(B, Sk, Hkv, Dqk),
                      f32_bytes(B, Sk, Hkv, Dv)}) {
    if (part == SIZE_MAX || total > SIZE_MAX - part) return SIZE_MAX;  // invalid or absurdly large: never fits
    total += part;
  }
  return total;
}

extern "C" int pith_attn_bwd_noalloc(const pith_attn_bwd_noalloc_args* a, void* stream) {
  PITH_REQUIRE(a != nullptr, "null args");
  PITH_REQUIRE(a->q && a->k && a->v && a->o && a->dout && a->lse && a->dq && a->dk && a->dv, "null tensor pointer");
  PITH_REQUIRE(a->B > 0 && a->Sq > 0 && a->Sk > 0 && a->Hq > 0 && a->Hkv > 0 && a->Dqk > 0 && a->Dv > 0,
               "bad shape B=%d Sq=%d Sk=%d Hq=%d Hkv=%d Dqk=%d Dv=%d", a->B, a->Sq, a->Sk, a->Hq, a->Hkv, a->Dqk, a->Dv);
  // the checks pith_attn_bwd would make, made here before anything is enqueued or the shared area is touched
  PITH_REQUIRE(a->Hq % a->Hkv == 0, "Hq=%d is not a multiple of Hkv=%d", a->Hq, a->Hkv);
  PITH_REQUIRE(a->Dv == 128 && (a->Dqk == 128 || a->Dqk == 192),
               "unsupported head dims Dqk=%d Dv=%d (supported: 128/128 and 192/128)", a->Dqk, a->Dv);
  PITH_REQUIRE(a->softmax_scale > 0.f, "softmax_scale must be positive");
  PITH_REQUIRE(a->Hq <= 65535 && a->B <= 65535, "Hq and B must fit a grid dimension");
  for (const void* ptr : {a->q, a->k, a->v, a->o, a->dout, static_cast<const void*>(a->dq),
                          static_cast<const void*>(a->dk), static_cast<const void*>(a->dv)})
    PITH_REQUIRE(aligned16(ptr), "tensor base %p is not 16-byte aligned", ptr);
  auto strides_ok = [&](const int64_t* st3, int heads) {  // bf16: 8 elements = 16 bytes
    return st3[1] % 8 == 0 && (heads == 1 || st3[2] % 8 == 0) && (a->B == 1 || st3[0] % 8 == 0);
  };
  PITH_REQUIRE(strides_ok(a->q_stride, a->Hq) && strides_ok(a->o_stride, a->Hq) && strides_ok(a->do_stride, a->Hq) &&
                   strides_ok(a->dq_stride, a->Hq) && strides_ok(a->k_stride, a->Hkv) &&
                   strides_ok(a->v_stride, a->Hkv) && strides_ok(a->dk_stride, a->Hkv) &&
                   strides_ok(a->dv_stride, a->Hkv),
               "strides must be multiples of 16 bytes");
  const size_t need = pith_attn_bwd_noalloc_scratch_bytes(a->B, a->Sq, a->Sk, a->Hq, a->Hkv, a->Dqk, a->Dv);
  if (need > kScratchBytes)
    return fail(kErrInvalidArg,
                "pith_attn_bwd_noalloc needs %zu bytes of scratch for this problem but the built-in area holds %zu; "
                "use pith_attn_bwd with caller-allocated accumulators",
                need, kScratchBytes);
  if (int rc = require_sm100()) return rc;
  unsigned char* base = nullptr;
  if (int rc = scratch_base(&base)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const size_t n_delta = round256(sizeof(float) * static_cast<size_t>(a->B) * a->Hq * a->Sq);
  const size_t n_dq = round256(sizeof(float) * static_cast<size_t>(a->B) * a->Sq * a->Hq * a->Dqk);
  const size_t n_dk = round256(sizeof(float) * static_cast<size_t>(a->B) * a->Sk * a->Hkv * a->Dqk);
  float* delta = reinterpret_cast<float*>(base);
  float* dq_acc = reinterpret_cast<float*>(base + n_delta);
  float* dk_acc = reinterpret_cast<float*>(base + n_delta + n_dq);
  float* dv_acc = reinterpret_cast<float*>(base + n_delta + n_dq + n_dk);
  // the accumulators are added into, and the area still holds the previous call's values
  PITH_CUDA(cudaMemsetAsync(base + n_delta, 0, need - n_delta, st));

  pith_bwd_preprocess_args pre = {};
  pre.o = a->o; pre.dout = a->dout; pre.delta = delta;
  pre.B = a->B; pre.S = a->Sq; pre.H = a->Hq; pre.Dv = a->Dv;
  for (int i = 0; i < 3; ++i) { pre.o_stride[i] = a->o_stride[i]; pre.do_stride[i] = a->do_stride[i]; }
  pre.delta_stride[0] = static_cast<int64_t>(a->Hq) * a->Sq;
  pre.delta_stride[1] = a->Sq;
  if (int rc = pith_attn_bwd_preprocess(&pre, stream)) return rc;

  pith_attn_bwd_args b = {};
  b.q = a->q; b.k = a->k; b.v = a->v; b.dout = a->dout; b.lse = a->lse; b.delta = delta;
  b.dq_acc = dq_acc; b.dk_acc = dk_acc; b.dv_acc = dv_acc; b.status = a->status;
  b.B = a->B; b.Sq = a->Sq; b.Sk = a->Sk; b.Hq = a->Hq; b.Hkv = a->Hkv; b.Dqk = a->Dqk; b.Dv = a->Dv;
  b.causal = a->causal; b.causal_offset = a->causal_offset; b.softmax_scale = a->softmax_scale;
  b.flags = PITH_BWD_SERIAL;  // one stream, no side stream or events
  const int64_t dq_st[3] = {static_cast<int64_t>(a->Sq) * a->Hq * a->Dqk, static_cast<int64_t>(a->Hq) * a->Dqk, a->Dqk};
  const int64_t dk_st[3] = {static_cast<int64_t>(a->Sk) * a->Hkv * a->Dqk, static_cast<int64_t>(a->Hkv) * a->Dqk, a->Dqk};
  const int64_t dv_st[3] = {static_cast<int64_t>(a->Sk) * a->Hkv * a->Dv, static_cast<int64_t>(a->Hkv) * a->Dv, a->Dv};
  for (int i = 0; i < 3; ++i) {
    b.q_stride[i] = a->q_stride[i]; b.k_stride[i] = a->k_stride[i]; b.v_stride[i] = a->v_stride[i];
    b.do_stride[i] = a->do_stride[i];
    b.dq_stride[i] = dq_st[i]; b.dk_stride[i] = dk_st[i]; b.dv_stride[i] = dv_st[i];
  }
  b.lse_stride[0] = a->lse_stride[0]; b.lse_stride[1] = a->lse_stride[1];
  b.delta_stride[0] = pre.delta_stride[0]; b.delta_stride[1] = pre.delta_stride[1];
  if (int rc = pith_attn_bwd(&b, stream)) return rc;

  if (int rc = pith_cast_f32_to_bf16(dq_acc, a->dq, a->B, a->Sq, a->Hq, a->Dqk, dq_st, a->dq_stride, 1.0f, stream)) return rc;
  if (int rc = pith_cast_f32_to_bf16(dk_acc, a->dk, a->B, a->Sk, a->Hkv, a->Dqk, dk_st, a->dk_stride, 1.0f, stream)) return rc;
  return pith_cast_f32_to_bf16(dv_acc, a->dv, a->B, a->Sk, a->Hkv, a->Dv, dv_st, a->dv_stride, 1.0f, stream);
}
