#include "host_common.h"

#include <string.h>

#include "../../include/pith_b200.h"
#include "common.cuh"

namespace pith {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int require_sm100() {
  int dev = 0;
  PITH_CUDA(cudaGetDevice(&dev));
  int major = 0;
  PITH_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10)
    return fail(kErrUnsupported, "pith_b200 kernels are built for sm_100a only; device %d has compute capability %d.x",
                dev, major);
  return kOk;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int make_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, int64_t B, int64_t S, int64_t H, int64_t D,
                    const int64_t st[3], int box_d, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(kErrNoDriver, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  PITH_REQUIRE(aligned16(base), "tensor base %p is not 16-byte aligned", base);
  PITH_REQUIRE(B > 0 && S > 0 && H > 0 && D > 0, "empty tensor %lldx%lldx%lldx%lld", (long long)B, (long long)S,
               (long long)H, (long long)D);
  int64_t sb = st[0], ss = st[1], sh = st[2];
  if (B == 1 && (sb * elem_bytes) % 16 != 0) sb = ss * S;
  if (H == 1 && (sh * elem_bytes) % 16 != 0) sh = D;
  PITH_REQUIRE((sb * elem_bytes) % 16 == 0 && (ss * elem_bytes) % 16 == 0 && (sh * elem_bytes) % 16 == 0,
               "strides (%lld, %lld, %lld elements) must be multiples of 16 bytes", (long long)sb, (long long)ss,
               (long long)sh);
  PITH_REQUIRE(sb > 0 && ss > 0 && sh > 0, "strides must be positive");
  PITH_REQUIRE(box_d * elem_bytes <= 128 && box_rows <= 256, "box %dx%d does not fit the 128-byte swizzle", box_d,
               box_rows);
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)(sh * elem_bytes), (cuuint64_t)(ss * elem_bytes),
                           (cuuint64_t)(sb * elem_bytes)};
  cuuint32_t box[4] = {(cuuint32_t)box_d, 1u, (cuuint32_t)box_rows, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kErrCuda, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return kOk;
}

}  // namespace pith

extern "C" {

const char* pith_last_error(void) { return pith::last_error_buffer(); }

const char* pith_status_string(uint32_t status) {
  static thread_local char buf[128];
  uint32_t code = status >> 24, detail = status & 0xFFFFFFu;
  if (status == 0)
    snprintf(buf, sizeof buf, "ok");
  else if (code == pith::kErrWaitTimeout)
    snprintf(buf, sizeof buf, "device wait timed out (barrier tag 0x%06x)", detail);
  else if (code == 3u)
    snprintf(buf, sizeof buf, "wait for a ring neighbour timed out (sequence number 0x%06x)", detail);
  else if (code == pith::kErrTmemAlloc)
    snprintf(buf, sizeof buf, "unexpected TMEM allocation (0x%06x)", detail);
  else if (code == pith::kErrSmemAlign)
    snprintf(buf, sizeof buf, "shared-memory window not 1024-byte aligned (offset 0x%06x)", detail);
  else
    snprintf(buf, sizeof buf, "unknown device status 0x%08x", status);
  return buf;
}

int pith_abi_version(void) { return PITH_B200_ABI_VERSION; }
}
