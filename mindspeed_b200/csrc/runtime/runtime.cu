// Launch bookkeeping and error text for the kernel library.
#include "msb_common.cuh"
#include <atomic>
#include <mutex>
#include <stdarg.h>
#include <string.h>

static std::atomic<unsigned long long> g_launches{0};
static char g_err[512] = {0};
static std::mutex g_err_mu;

extern "C" void msb_count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
MSB_API unsigned long long msb_launch_count() { return g_launches.load(); }
MSB_API void msb_reset_launch_count() { g_launches.store(0); }

extern "C" void msb_set_error(const char* fmt, ...) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
MSB_API const char* msb_last_error() { return g_err; }

MSB_API int msb_device_info(int* sms, int* cc_major, int* cc_minor, size_t* smem_optin) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 1;
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) return 1;
  *sms = p.multiProcessorCount; *cc_major = p.major; *cc_minor = p.minor; *smem_optin = p.sharedMemPerBlockOptin;
  return 0;
}

// Write `bytes` of a scratch buffer: used by benchmarks to flush the 126 MB L2 between timed iterations.
__global__ void msb_flush_kernel(uint4* p, size_t n, unsigned v) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) p[i] = make_uint4(v, v, v, v);
}
MSB_API int msb_l2_flush(void* buf, size_t bytes, cudaStream_t s) {
  size_t n = bytes / 16;
  msb_flush_kernel<<<msb::num_sms() * 4, 512, 0, s>>>((uint4*)buf, n, 0u);
  MSB_CHECK_LAUNCH("l2_flush");
  return 0;
}
