// Host build of the caching allocator: C ABI over msb_caching_allocator.hpp with a malloc/free (or fake, size-limited)
// backend.  It exists so that the allocator logic - splitting, merging, the pressure path, tracing - is exercised by
// CPU tests; the device build in csrc/runtime/allocator_cuda.cu instantiates the same class over cudaMalloc.
#include <stdlib.h>
#include <string.h>

#include "msb_caching_allocator.hpp"

#define MSB_HOST_API extern "C" __attribute__((visibility("default")))

namespace {
uint64_t g_backend_capacity = 0;   // 0 = unlimited; otherwise the fake device runs out of memory at this many bytes
uint64_t g_backend_in_use = 0;
std::unordered_map<void*, size_t> g_backend_sizes;
std::mutex g_backend_mu;

void* host_raw_malloc(size_t bytes, int) {
  std::lock_guard<std::mutex> g(g_backend_mu);
  if (g_backend_capacity && g_backend_in_use + bytes > g_backend_capacity) return nullptr;
  void* p = nullptr;
  if (posix_memalign(&p, 512, bytes) != 0) return nullptr;
  g_backend_in_use += bytes;
  g_backend_sizes[p] = bytes;
  return p;
}
int host_raw_free(void* p, int) {
  std::lock_guard<std::mutex> g(g_backend_mu);
  auto it = g_backend_sizes.find(p);
  if (it == g_backend_sizes.end()) return 1;
  g_backend_in_use -= it->second;
  g_backend_sizes.erase(it);
  free(p);
  return 0;
}
}  // namespace

MSB_HOST_API void* msb_halloc_create(unsigned long long backend_capacity_bytes) {
  g_backend_capacity = backend_capacity_bytes;
  return new msb::alloc::CachingAllocator(host_raw_malloc, host_raw_free, 0);
}
MSB_HOST_API void msb_halloc_destroy(void* h) { delete static_cast<msb::alloc::CachingAllocator*>(h); }
MSB_HOST_API void* msb_halloc_malloc(void* h, unsigned long long bytes, unsigned long long stream) {
  return static_cast<msb::alloc::CachingAllocator*>(h)->malloc((size_t)bytes, stream);
}
MSB_HOST_API int msb_halloc_free(void* h, void* p) { return static_cast<msb::alloc::CachingAllocator*>(h)->free(p); }
MSB_HOST_API unsigned long long msb_halloc_empty_cache(void* h) { return static_cast<msb::alloc::CachingAllocator*>(h)->empty_cache(); }
MSB_HOST_API void msb_halloc_set_limit(void* h, unsigned long long bytes) { static_cast<msb::alloc::CachingAllocator*>(h)->set_limit(bytes); }
MSB_HOST_API void msb_halloc_set_tags(void* h, int step, int phase) { static_cast<msb::alloc::CachingAllocator*>(h)->set_tags(step, phase); }
MSB_HOST_API void msb_halloc_set_pressure_callback(void* h, msb::alloc::PressureCallback cb, void* user) {
  static_cast<msb::alloc::CachingAllocator*>(h)->set_pressure_callback(cb, user);
}
MSB_HOST_API void msb_halloc_enable_trace(void* h, unsigned long long capacity) { static_cast<msb::alloc::CachingAllocator*>(h)->enable_trace((size_t)capacity); }
MSB_HOST_API unsigned long long msb_halloc_read_trace(void* h, msb::alloc::TraceEvent* out, unsigned long long max_events, int clear) {
  return static_cast<msb::alloc::CachingAllocator*>(h)->read_trace(out, (size_t)max_events, clear != 0);
}
MSB_HOST_API void msb_halloc_stats(void* h, msb::alloc::Stats* out) { *out = static_cast<msb::alloc::CachingAllocator*>(h)->stats(); }
MSB_HOST_API unsigned long long msb_halloc_block_size(void* h, void* p) { return static_cast<msb::alloc::CachingAllocator*>(h)->block_size(p); }
MSB_HOST_API unsigned long long msb_halloc_backend_in_use() { return g_backend_in_use; }
