// Device, memory, stream and event entry points: the CUDA stand-in for the reference's device and launch
// layer (baretile/pci.py, baretile/chip.py, baretile/runtime.py). Everything here is thin plumbing over the
// CUDA runtime; the kernels live in layout.cu, gemv.cu and gemm.cu.
#include "common.cuh"
#include <chrono>
#include <cstring>
#include <thread>

namespace bt {
thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_calls{0};
}  // namespace bt

using namespace bt;

extern "C" {

const char *bt_last_error(void) { return g_error; }

int bt_launch_count(uint64_t *count) {
  BT_REQUIRE(count, "bt_launch_count: null result");
  *count = g_launches.load();
  return BT_OK;
}

int bt_device_count(int *count) {
  BT_REQUIRE(count, "bt_device_count: null result");
  cudaError_t e = cudaGetDeviceCount(count);
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) { *count = 0; cudaGetLastError(); return BT_OK; }
  return cuda_status(e, "cudaGetDeviceCount");
}

int bt_device_info_get(int device, bt_device_info *out) {
  BT_REQUIRE(out, "bt_device_info_get: null result");
  if (int s = use_device(device)) return s;
  cudaDeviceProp p;
  BT_CUDA(cudaGetDeviceProperties(&p, device));
  memset(out, 0, sizeof *out);
  strncpy(out->name, p.name, sizeof out->name - 1);
  out->sm_count = p.multiProcessorCount;
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->l2_bytes = p.l2CacheSize;
  out->memory_bytes = p.totalGlobalMem;
  out->max_shared_bytes = (int)p.sharedMemPerBlockOptin;
  int khz = 0;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device);
  out->clock_khz = khz;
  return BT_OK;
}

int bt_malloc(int device, size_t bytes, uint64_t *ptr) {
  BT_REQUIRE(ptr && bytes, "bt_malloc: needs a result pointer and a nonzero size");
  if (int s = use_device(device)) return s;
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) { cudaGetLastError(); return fail(BT_NO_MEMORY, "no %zu bytes free in device memory: %s", bytes, cudaGetErrorString(e)); }
  *ptr = reinterpret_cast<uint64_t>(p);
  return BT_OK;
}

int bt_free(int device, uint64_t ptr) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaFree(as_ptr<void>(ptr)));
  return BT_OK;
}

int bt_host_alloc(size_t bytes, void **ptr) {
  BT_REQUIRE(ptr && bytes, "bt_host_alloc: needs a result pointer and a nonzero size");
  cudaError_t e = cudaMallocHost(ptr, bytes);
  if (e != cudaSuccess) { cudaGetLastError(); return fail(BT_NO_MEMORY, "no %zu bytes of pinned host memory: %s", bytes, cudaGetErrorString(e)); }
  return BT_OK;
}

int bt_host_free(void *ptr) {
  BT_CUDA(cudaFreeHost(ptr));
  return BT_OK;
}

int bt_stream_create(int device, uint64_t *stream) {
  BT_REQUIRE(stream, "bt_stream_create: null result");
  if (int s = use_device(device)) return s;
  cudaStream_t st;
  BT_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  *stream = reinterpret_cast<uint64_t>(st);
  return BT_OK;
}

int bt_stream_destroy(int device, uint64_t stream) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaStreamDestroy(as_stream(stream)));
  return BT_OK;
}

int bt_stream_query(int device, uint64_t stream, int *done) {
  BT_REQUIRE(done, "bt_stream_query: null result");
  if (int s = use_device(device)) return s;
  cudaError_t e = cudaStreamQuery(as_stream(stream));
  if (e == cudaErrorNotReady) { *done = 0; cudaGetLastError(); return BT_OK; }
  *done = 1;
  return cuda_status(e, "cudaStreamQuery");
}

// Poll rather than block, so that a launch that never finishes becomes a TimeoutError on the host while the
// context stays usable (Runtime.wait polls the status word the same way, baretile/runtime.py:849-880).
int bt_stream_sync(int device, uint64_t stream, int timeout_ms) {
  if (int s = use_device(device)) return s;
  if (timeout_ms < 0) { BT_CUDA(cudaStreamSynchronize(as_stream(stream))); return BT_OK; }
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (unsigned spins = 0;; spins++) {
    cudaError_t e = cudaStreamQuery(as_stream(stream));
    if (e == cudaSuccess) return BT_OK;
    if (e != cudaErrorNotReady) return cuda_status(e, "cudaStreamQuery");
    cudaGetLastError();
    if (std::chrono::steady_clock::now() > deadline) return fail(BT_TIMEOUT, "the stream did not finish its queued work within %d ms", timeout_ms);
    if (spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

int bt_h2d(int device, uint64_t dst, const void *src, size_t bytes, uint64_t stream) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaMemcpyAsync(as_ptr<void>(dst), src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
  return BT_OK;
}

int bt_d2h(int device, void *dst, uint64_t src, size_t bytes, uint64_t stream) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaMemcpyAsync(dst, as_ptr<void>(src), bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
  return BT_OK;
}

int bt_d2d(int device, uint64_t dst, uint64_t src, size_t bytes, uint64_t stream) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaMemcpyAsync(as_ptr<void>(dst), as_ptr<void>(src), bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
  return BT_OK;
}

int bt_memset(int device, uint64_t dst, int value, size_t bytes, uint64_t stream) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaMemsetAsync(as_ptr<void>(dst), value, bytes, as_stream(stream)));
  return BT_OK;
}

int bt_event_create(int device, uint64_t *event) {
  BT_REQUIRE(event, "bt_event_create: null result");
  if (int s = use_device(device)) return s;
  cudaEvent_t e;
  BT_CUDA(cudaEventCreate(&e));
  *event = reinterpret_cast<uint64_t>(e);
  return BT_OK;
}

int bt_event_destroy(int device, uint64_t event) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
  return BT_OK;
}

int bt_event_record(int device, uint64_t event, uint64_t stream) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), as_stream(stream)));
  return BT_OK;
}

int bt_stream_wait_event(int device, uint64_t stream, uint64_t event) {
  BT_REQUIRE(event, "bt_stream_wait_event: null event");
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaStreamWaitEvent(as_stream(stream), reinterpret_cast<cudaEvent_t>(event), 0));
  return BT_OK;
}

int bt_event_elapsed_ms(int device, uint64_t start, uint64_t end, float *ms) {
  BT_REQUIRE(ms, "bt_event_elapsed_ms: null result");
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(end)));
  BT_CUDA(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start), reinterpret_cast<cudaEvent_t>(end)));
  return BT_OK;
}

// ---- replay: record the launches queued on a stream once, then replay them with one call ----

int bt_graph_begin(int device, uint64_t stream) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaStreamBeginCapture(as_stream(stream), cudaStreamCaptureModeThreadLocal));
  return BT_OK;
}

int bt_graph_end(int device, uint64_t stream, uint64_t *graph) {
  BT_REQUIRE(graph, "bt_graph_end: null result");
  if (int s = use_device(device)) return s;
  cudaGraph_t g = nullptr;
  BT_CUDA(cudaStreamEndCapture(as_stream(stream), &g));
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
  cudaGraphDestroy(g);
  BT_CUDA(e);
  *graph = reinterpret_cast<uint64_t>(exec);
  return BT_OK;
}

int bt_graph_launch(int device, uint64_t graph, uint64_t stream) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(graph), as_stream(stream)));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return BT_OK;
}

int bt_graph_destroy(int device, uint64_t graph) {
  if (int s = use_device(device)) return s;
  BT_CUDA(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(graph)));
  return BT_OK;
}

}  // extern "C"
