// Shared host-side helpers of libbaretile_b200: status codes, the per-thread error text, launch counting.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include "../../include/baretile_b200.h"

namespace bt {

extern thread_local char g_error[512];
extern std::atomic<uint64_t> g_launches;
extern std::atomic<uint64_t> g_calls;   // entry-point calls that selected a device: a cheap "has anything else been queued since" stamp

inline int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return code;
}

inline int cuda_status(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return BT_OK;
  int code = e == cudaErrorMemoryAllocation ? BT_NO_MEMORY : e == cudaErrorInvalidValue ? BT_BAD_ARGUMENT : BT_DEVICE;
  return fail(code, "%s: %s", what, cudaGetErrorString(e));
}

#define BT_CUDA(call)                                          \
  do {                                                         \
    int bt_status_ = ::bt::cuda_status((call), #call);         \
    if (bt_status_ != BT_OK) return bt_status_;                \
  } while (0)

#define BT_REQUIRE(cond, ...)                                  \
  do {                                                         \
    if (!(cond)) return ::bt::fail(BT_BAD_ARGUMENT, __VA_ARGS__); \
  } while (0)

// Select the device for the calling thread; every entry point starts with it.
inline int use_device(int device) {
  int n = 0;
  BT_CUDA(cudaGetDeviceCount(&n));
  if (device < 0 || device >= n) return fail(BT_BAD_ARGUMENT, "device %d: there are %d CUDA devices", device, n);
  BT_CUDA(cudaSetDevice(device));
  g_calls.fetch_add(1, std::memory_order_relaxed);
  return BT_OK;
}

// After a kernel launch: count it and surface launch errors.
inline int launched(const char *name) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cuda_status(cudaGetLastError(), name);
}

inline cudaStream_t as_stream(uint64_t s) { return reinterpret_cast<cudaStream_t>(s); }
template <class T> inline T *as_ptr(uint64_t p) { return reinterpret_cast<T *>(p); }

__host__ __device__ constexpr int tile_bytes(int fmt) { return fmt == BT_BFP8 ? 1088 : fmt == BT_BFP4 ? 576 : fmt == BT_BF16 ? 2048 : 4096; }

}  // namespace bt
