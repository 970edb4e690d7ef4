// MoE token permutation: row gather and (optionally weighted) row scatter-add with fp32 accumulation.
// reference semantics: npu_moe_token_permute / npu_moe_token_unpermute
// (mindspeed/ops/csrc/cann/npu_moe_token_permute.cpp, npu_moe_token_unpermute.cpp).
#include "msb_common.cuh"
using namespace msb;

namespace {
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const long long* __restrict__ idx, T* __restrict__ out,
                                   long long n, int cols) {
  const int vec = (cols % 8 == 0) ? cols / 8 : 0;
  for (long long r = blockIdx.x; r < n; r += gridDim.x) {
    const T* src = x + idx[r] * (long long)cols;
    T* dst = out + r * (long long)cols;
    if (vec) {
      for (int v = threadIdx.x; v < vec; v += blockDim.x) { Vec8<T> t; t.load(src + v * 8); t.store(dst + v * 8); }
    } else {
      for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = src[c];
    }
  }
}
template <typename T>
__global__ void scatter_add_rows_kernel(const T* __restrict__ src, const long long* __restrict__ idx,
                                        const float* __restrict__ weight, float* __restrict__ out, long long n, int cols) {
  for (long long r = blockIdx.x; r < n; r += gridDim.x) {
    const T* s = src + r * (long long)cols;
    float* d = out + idx[r] * (long long)cols;
    const float w = weight ? weight[r] : 1.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) atomicAdd(d + c, to_f(s[c]) * w);
  }
}
}  // namespace

MSB_API int msb_gather_rows(const void* x, const long long* idx, void* out, long long n, int cols, int dtype, cudaStream_t s) {
  if (n == 0) return 0;
  int grid = (int)(n < (long long)msb::num_sms() * 16 ? n : (long long)msb::num_sms() * 16);
  MSB_DISPATCH_FLOAT(dtype, T, gather_rows_kernel<T><<<grid, 256, 0, s>>>((const T*)x, idx, (T*)out, n, cols));
  MSB_CHECK_LAUNCH("gather_rows");
  return 0;
}
MSB_API int msb_scatter_add_rows(const void* src, const long long* idx, const float* weight, float* out, long long n, int cols,
                                 int dtype, cudaStream_t s) {
  if (n == 0) return 0;
  int grid = (int)(n < (long long)msb::num_sms() * 16 ? n : (long long)msb::num_sms() * 16);
  MSB_DISPATCH_FLOAT(dtype, T, scatter_add_rows_kernel<T><<<grid, 256, 0, s>>>((const T*)src, idx, weight, out, n, cols));
  MSB_CHECK_LAUNCH("scatter_add_rows");
  return 0;
}
