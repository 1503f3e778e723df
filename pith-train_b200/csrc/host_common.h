// Host-side helpers shared by the C-ABI entry points: error text, argument checks and
// TMA descriptor creation. The driver's tensor-map encoder is looked up at run time
// through the CUDA runtime so the library has no link-time dependency on libcuda and
// can be loaded (for symbol checks) on a machine without a GPU driver.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

namespace pith {

enum : int {
  kOk = 0,
  kErrInvalidArg = -1,
  kErrUnsupported = -2,
  kErrCuda = -3,
  kErrNoDriver = -4,
};

char* last_error_buffer();  // thread-local, 512 bytes

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define PITH_REQUIRE(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) return ::pith::fail(::pith::kErrInvalidArg, __VA_ARGS__); \
  } while (0)

#define PITH_CUDA(call)                                                                       \
  do {                                                                                        \
    cudaError_t e__ = (call);                                                                 \
    if (e__ != cudaSuccess)                                                                   \
      return ::pith::fail(::pith::kErrCuda, "%s failed: %s", #call, cudaGetErrorString(e__)); \
  } while (0)

// Checks that the current device is compute capability 10.x; the kernels hold sm_100a code only.
int require_sm100();

// Builds a 4-D tiled tensor map over a [B][S][H][D] tensor (dims given innermost first:
// D, H, S, B) with a {box_d, 1, box_rows, 1} box and the 128-byte shared-memory swizzle.
// strides_elems = {b, s, h}. elem_bytes = 2 (bf16) or 4 (fp32).
int make_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, int64_t B, int64_t S, int64_t H, int64_t D,
                    const int64_t strides_elems[3], int box_d, int box_rows);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace pith
