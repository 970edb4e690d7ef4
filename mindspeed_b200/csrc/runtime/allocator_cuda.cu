// Device build of the caching allocator (msb_caching_allocator.hpp over cudaMalloc / cudaFree) with the entry points
// torch.cuda.memory.CUDAPluggableAllocator expects, plus the controls the memory features use: a soft limit, a
// pressure callback (swap-out / drop-recomputable hook run before an out-of-memory error is raised), allocation
// tracing with step/phase tags, statistics, and a pinned-host swap pool with asynchronous copies on a dedicated stream.
//
//   void* msb_torch_malloc(ssize_t size, int device, cudaStream_t stream)
//   void  msb_torch_free(void* ptr, ssize_t size, int device, cudaStream_t stream)
//
// One allocator instance per device, created on first use.  Stream-ordered reuse: a freed block returns to the pool
// of the stream it was allocated on, so reuse on that stream is ordered by the stream itself; cross-stream use is
// the caller's responsibility (torch calls record_stream, which the pluggable interface does not forward here, so
// the framework keeps side-stream tensors alive until their events complete - see memory/swap_attention.py).
// reference behaviour: mindspeed/ops/csrc/pluggable_allocator/smart_swap/{PluggableAllocator,DeviceCachingAllocator,
// NPUSwapManager}.cpp and adaptive_recomputing/NpuCachingCustomAllocator.cpp.
#include "msb_common.cuh"
#include "msb_caching_allocator.hpp"

namespace {
constexpr int kMaxDevices = 16;
msb::alloc::CachingAllocator* g_alloc[kMaxDevices] = {nullptr};
std::mutex g_create_mu;

void* cuda_raw_malloc(size_t bytes, int device) {
  int cur = -1;
  cudaGetDevice(&cur);
  if (cur != device) cudaSetDevice(device);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (cur != device && cur >= 0) cudaSetDevice(cur);
  if (e != cudaSuccess) { cudaGetLastError(); return nullptr; }   // clear the sticky-free OOM error; the caller retries
  return p;
}
int cuda_raw_free(void* p, int device) {
  int cur = -1;
  cudaGetDevice(&cur);
  if (cur != device) cudaSetDevice(device);
  cudaError_t e = cudaFree(p);
  if (cur != device && cur >= 0) cudaSetDevice(cur);
  return e == cudaSuccess ? 0 : 1;
}
msb::alloc::CachingAllocator* get(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  if (!g_alloc[device]) {
    std::lock_guard<std::mutex> g(g_create_mu);
    if (!g_alloc[device]) g_alloc[device] = new msb::alloc::CachingAllocator(cuda_raw_malloc, cuda_raw_free, device);
  }
  return g_alloc[device];
}
}  // namespace

MSB_API void* msb_torch_malloc(ssize_t size, int device, cudaStream_t stream) {
  msb::alloc::CachingAllocator* a = get(device);
  if (!a || size < 0) return nullptr;
  return a->malloc((size_t)size, (uint64_t)reinterpret_cast<uintptr_t>(stream));
}
MSB_API void msb_torch_free(void* ptr, ssize_t, int device, cudaStream_t) {
  msb::alloc::CachingAllocator* a = get(device);
  if (a) a->free(ptr);
}
MSB_API unsigned long long msb_dalloc_empty_cache(int device) { auto* a = get(device); return a ? a->empty_cache() : 0; }
MSB_API void msb_dalloc_set_limit(int device, unsigned long long bytes) { if (auto* a = get(device)) a->set_limit(bytes); }
MSB_API void msb_dalloc_set_tags(int device, int step, int phase) { if (auto* a = get(device)) a->set_tags(step, phase); }
MSB_API void msb_dalloc_set_pressure_callback(int device, msb::alloc::PressureCallback cb, void* user) { if (auto* a = get(device)) a->set_pressure_callback(cb, user); }
MSB_API void msb_dalloc_enable_trace(int device, unsigned long long capacity) { if (auto* a = get(device)) a->enable_trace((size_t)capacity); }
MSB_API unsigned long long msb_dalloc_read_trace(int device, msb::alloc::TraceEvent* out, unsigned long long max_events, int clear) {
  auto* a = get(device);
  return a ? a->read_trace(out, (size_t)max_events, clear != 0) : 0;
}
MSB_API void msb_dalloc_stats(int device, msb::alloc::Stats* out) { if (auto* a = get(device)) *out = a->stats(); }
MSB_API void msb_dalloc_reset_peaks(int device) { if (auto* a = get(device)) a->reset_peaks(); }

// ---- pinned-host swap pool: asynchronous device <-> host moves on a dedicated stream ----------------------------------
namespace {
struct SwapSlot { void* host; size_t bytes; cudaEvent_t done; bool busy; };
std::vector<SwapSlot> g_slots;
std::mutex g_swap_mu;
cudaStream_t g_swap_stream = nullptr;
}  // namespace

// Copy `bytes` from device memory to a pinned host buffer on the swap stream, after `after_stream` has reached this
// point.  Returns a slot id (>= 0) or -1.  The device memory may be released once msb_swap_wait(slot) has returned or
// the caller has made its stream wait for the slot's event (msb_swap_stream_wait).
MSB_API int msb_swap_out(const void* dev_ptr, unsigned long long bytes, cudaStream_t after_stream) {
  std::lock_guard<std::mutex> g(g_swap_mu);
  if (!g_swap_stream && cudaStreamCreateWithFlags(&g_swap_stream, cudaStreamNonBlocking) != cudaSuccess) { msb_set_error("swap: cannot create stream"); return -1; }
  int id = -1;
  for (size_t i = 0; i < g_slots.size(); ++i) if (!g_slots[i].busy && g_slots[i].bytes >= bytes) { id = (int)i; break; }
  if (id < 0) {
    SwapSlot s{nullptr, (size_t)bytes, nullptr, false};
    if (cudaMallocHost(&s.host, bytes) != cudaSuccess) { cudaGetLastError(); msb_set_error("swap: pinned allocation of %llu bytes failed", bytes); return -1; }
    cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming);
    g_slots.push_back(s);
    id = (int)g_slots.size() - 1;
  }
  SwapSlot& s = g_slots[id];
  s.busy = true;
  cudaEvent_t ready;
  cudaEventCreateWithFlags(&ready, cudaEventDisableTiming);
  cudaEventRecord(ready, after_stream);
  cudaStreamWaitEvent(g_swap_stream, ready, 0);
  cudaEventDestroy(ready);
  if (cudaMemcpyAsync(s.host, dev_ptr, bytes, cudaMemcpyDeviceToHost, g_swap_stream) != cudaSuccess) { msb_set_error("swap: D2H copy failed"); s.busy = false; return -1; }
  cudaEventRecord(s.done, g_swap_stream);
  return id;
}
// Copy a slot back into device memory on the swap stream; `consumer_stream` is made to wait for the copy.
MSB_API int msb_swap_in(int slot, void* dev_ptr, unsigned long long bytes, cudaStream_t consumer_stream, int release_slot) {
  std::lock_guard<std::mutex> g(g_swap_mu);
  if (slot < 0 || slot >= (int)g_slots.size() || !g_slots[slot].busy || g_slots[slot].bytes < bytes) { msb_set_error("swap: bad slot %d", slot); return 1; }
  SwapSlot& s = g_slots[slot];
  if (cudaMemcpyAsync(dev_ptr, s.host, bytes, cudaMemcpyHostToDevice, g_swap_stream) != cudaSuccess) { msb_set_error("swap: H2D copy failed"); return 1; }
  cudaEventRecord(s.done, g_swap_stream);
  cudaStreamWaitEvent(consumer_stream, s.done, 0);
  if (release_slot) {
    // the host buffer may be reused only after the copy has left it: later users of the slot queue on the same stream
    s.busy = false;
  }
  return 0;
}
MSB_API int msb_swap_stream_wait(int slot, cudaStream_t stream) {
  std::lock_guard<std::mutex> g(g_swap_mu);
  if (slot < 0 || slot >= (int)g_slots.size()) return 1;
  return cudaStreamWaitEvent(stream, g_slots[slot].done, 0) == cudaSuccess ? 0 : 1;
}
MSB_API int msb_swap_wait(int slot) {
  cudaEvent_t e;
  {
    std::lock_guard<std::mutex> g(g_swap_mu);
    if (slot < 0 || slot >= (int)g_slots.size()) return 1;
    e = g_slots[slot].done;
  }
  return cudaEventSynchronize(e) == cudaSuccess ? 0 : 1;
}
MSB_API unsigned long long msb_swap_pinned_bytes() {
  std::lock_guard<std::mutex> g(g_swap_mu);
  unsigned long long t = 0;
  for (auto& s : g_slots) t += s.bytes;
  return t;
}
