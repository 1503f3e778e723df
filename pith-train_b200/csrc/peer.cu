// Stream-ordered flags in peer-visible memory: the hand-off between ring neighbours when K/V and dK/dV blocks
// are moved by the copy engines (cudaMemcpyAsync between peer-mapped buffers) instead of NCCL send/recv kernels,
// which would take SMs away from the attention kernels.
//
//   pith_flag_signal  one thread advances a sequence counter in THIS GPU's memory, publishes everything written so
//                     far (system-scope fence) and stores the new sequence number into a flag that may live in
//                     another GPU's memory.
//   pith_flag_wait    one thread advances its own sequence counter and polls a flag in THIS GPU's memory until it
//                     reaches that number. The wait is bounded: after `max_cycles` it records an error in the
//                     status word and returns, so a late or dead neighbour stalls a stream for a bounded time and
//                     never hangs the GPU.
// The sequence numbers live on the device, so the same launches can be replayed from a CUDA graph. Flags only grow;
// comparisons are wrap-safe.
#include <string.h>

#include "../../include/pith_b200.h"
#include "common.cuh"
#include "host_common.h"

namespace pith {

constexpr uint32_t kErrPeerWait = 3u;

__global__ void flag_signal_kernel(uint32_t* flag, uint32_t* counter) {
  const uint32_t value = *counter + 1u;
  *counter = value;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

__global__ void flag_wait_kernel(const uint32_t* flag, uint32_t* counter, long long max_cycles, uint32_t* status) {
  const uint32_t value = *counter + 1u;
  *counter = value;
  // Once any wait on this GPU has run out the ring is lost anyway: later waits return at once, so that the stream
  // drains in milliseconds and the host sees the status word at its next check.
  if (status != nullptr && *reinterpret_cast<volatile uint32_t*>(status) != 0u) return;
  const long long t0 = clock64();
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - value) >= 0) break;
    if (clock64() - t0 > max_cycles) {
      if (status != nullptr) atomicCAS(status, 0u, (kErrPeerWait << 24) | (value & 0xFFFFFFu));
      break;
    }
    __nanosleep(200);
  }
  __threadfence_system();
}

}  // namespace pith

using namespace pith;

extern "C" int pith_flag_signal(uint32_t* flag, uint32_t* counter, void* stream) {
  PITH_REQUIRE(flag != nullptr && counter != nullptr, "null flag or counter");
  flag_signal_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(flag, counter);
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

extern "C" int pith_flag_wait(const uint32_t* flag, uint32_t* counter, double max_seconds, uint32_t* status,
                              void* stream) {
  PITH_REQUIRE(flag != nullptr && counter != nullptr, "null flag or counter");
  PITH_REQUIRE(max_seconds > 0.0 && max_seconds <= 120.0, "max_seconds must be in (0, 120]");
  const long long cycles = static_cast<long long>(max_seconds * 2.0e9);
  flag_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(flag, counter, cycles, status);
  PITH_CUDA(cudaGetLastError());
  return kOk;
}

typedef CUresult (*AddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

static AddressRangeFn address_range_fn() {
  static AddressRangeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<AddressRangeFn>(p);
  }
  return fn;
}

static_assert(sizeof(cudaIpcMemHandle_t) == PITH_IPC_HANDLE_BYTES, "IPC handle size");

extern "C" int pith_ipc_export(const void* ptr, void* handle64, uint64_t* offset) {
  PITH_REQUIRE(ptr != nullptr && handle64 != nullptr && offset != nullptr, "null argument");
  AddressRangeFn fn = address_range_fn();
  if (fn == nullptr) return fail(kErrNoDriver, "cuMemGetAddressRange is not available from the CUDA driver");
  CUdeviceptr base = 0;
  size_t size = 0;
  CUresult r = fn(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  if (r != CUDA_SUCCESS) return fail(kErrCuda, "cuMemGetAddressRange failed with CUresult %d", (int)r);
  cudaIpcMemHandle_t h;
  PITH_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(handle64, &h, sizeof h);
  *offset = static_cast<uint64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return kOk;
}

extern "C" int pith_ipc_open(const void* handle64, void** base) {
  PITH_REQUIRE(handle64 != nullptr && base != nullptr, "null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof h);
  PITH_CUDA(cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess));
  return kOk;
}

extern "C" int pith_ipc_close(void* base) {
  PITH_REQUIRE(base != nullptr, "null argument");
  PITH_CUDA(cudaIpcCloseMemHandle(base));
  return kOk;
}

extern "C" int pith_peer_copy(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return kOk;
  PITH_REQUIRE(dst != nullptr && src != nullptr, "null argument");
  PITH_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
  return kOk;
}

extern "C" int pith_enable_peer_access(int32_t peer_device) {
  int dev = 0;
  PITH_CUDA(cudaGetDevice(&dev));
  if (peer_device == dev) return kOk;
  int can = 0;
  PITH_CUDA(cudaDeviceCanAccessPeer(&can, dev, peer_device));
  if (!can) return fail(kErrUnsupported, "device %d cannot access device %d directly", dev, peer_device);
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return kOk;
  }
  if (e != cudaSuccess) return fail(kErrCuda, "cudaDeviceEnablePeerAccess(%d) failed: %s", peer_device, cudaGetErrorString(e));
  return kOk;
}
