// Smaller fused ops of the reference's op layer.
//   scaled_masked_softmax   softmax(scale * x masked) over the last dim, fwd / bwd (non-flash attention path;
//                           reference: mindspeed/core/fusions/fused_softmax.py:6-52)
//   ring_attention_update   online-softmax merge of two partial attention results (out, max, sum)
//                           (reference: mindspeed/ops/csrc/cann/npu_ring_attention_update.cpp:45, math
//                           mindspeed/core/context_parallel/utils.py:77-119)
//   add_rmsnorm             residual add fused with RMSNorm: h = x + residual; y = rmsnorm(h) (returns both)
//                           (reference family: npu_dropout_add_layer_norm / npu_mm_all_reduce_add_rms_norm)
//   quant_1x128             per-row, per-128-column fp8 e4m3 quantisation with fp32 scales (blockwise recipe)
#include "msb_common.cuh"
#include <cuda_fp8.h>
using namespace msb;

namespace {
// mask: uint8 [rows_mask, cols] broadcast over (rows / rows_mask) leading groups; mode 1 = causal (upper triangular) instead
template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, const uint8_t* __restrict__ mask, T* __restrict__ y, long long rows,
                                   int cols, float scale, int sq, int causal, long long mask_rows) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * cols;
  T* yr = y + row * cols;
  const int qi = (int)(row % sq);
  const uint8_t* mr = mask ? mask + (row % mask_rows) * cols : nullptr;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    bool masked = (mr && mr[c]) || (causal && c > qi + (cols - sq));
    float v = masked ? -INFINITY : to_f(xr[c]) * scale;
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    bool masked = (mr && mr[c]) || (causal && c > qi + (cols - sq));
    sum += masked ? 0.f : __expf(to_f(xr[c]) * scale - mx);
  }
  sum = block_sum(sum, red);
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    bool masked = (mr && mr[c]) || (causal && c > qi + (cols - sq));
    yr[c] = from_f<T>(masked ? 0.f : __expf(to_f(xr[c]) * scale - mx) * inv);
  }
}
template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int cols, float scale) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* dyr = dy + row * cols; const T* yr = y + row * cols; T* dxr = dx + row * cols;
  float dot = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dot += to_f(dyr[c]) * to_f(yr[c]);
  dot = block_sum(dot, red);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dxr[c] = from_f<T>(scale * to_f(yr[c]) * (to_f(dyr[c]) - dot));
}

// out[r, :] over rows r = (b, n, s) flattened; max/sum fp32 per row
template <typename T>
__global__ void ring_update_kernel(const T* __restrict__ prev_out, const float* __restrict__ prev_max, const float* __restrict__ prev_sum,
                                   const T* __restrict__ cur_out, const float* __restrict__ cur_max, const float* __restrict__ cur_sum,
                                   T* __restrict__ out, float* __restrict__ out_max, float* __restrict__ out_sum, long long rows, int d) {
  for (long long r = (long long)blockIdx.x * blockDim.y + threadIdx.y; r < rows; r += (long long)gridDim.x * blockDim.y) {
    const float m1 = prev_max[r], m2 = cur_max[r], l1 = prev_sum[r], l2 = cur_sum[r];
    const float m = fmaxf(m1, m2);
    const float a = (m1 == -INFINITY) ? 0.f : l1 * __expf(m1 - m), b = (m2 == -INFINITY) ? 0.f : l2 * __expf(m2 - m);
    const float l = a + b;
    const float wa = l > 0.f ? a / l : 0.f, wb = l > 0.f ? b / l : 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x)
      out[r * d + c] = from_f<T>(to_f(prev_out[r * d + c]) * wa + to_f(cur_out[r * d + c]) * wb);
    if (threadIdx.x == 0) { out_max[r] = m; out_sum[r] = l; }
  }
}

template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ gamma, T* __restrict__ h,
                                   T* __restrict__ y, float* __restrict__ rstd, int cols, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = to_f(x[row * cols + c]) + to_f(res[row * cols + c]);
    T hv = from_f<T>(v);
    h[row * cols + c] = hv;
    float vr = to_f(hv);
    ss += vr * vr;
  }
  ss = block_sum(ss, red);
  const float rs = rsqrtf(ss / cols + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = rs;
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    y[row * cols + c] = from_f<T>(to_f(h[row * cols + c]) * rs * to_f(gamma[c]));
}

template <typename T>
__global__ void quant_1x128_kernel(const T* __restrict__ x, __nv_fp8_e4m3* __restrict__ q, float* __restrict__ scale, long long rows,
                                   int cols, int pow2) {
  // one warp per (row, 128-column block); lane holds 4 values
  const long long blocks_per_row = cols / 128;
  const long long total = rows * blocks_per_row;
  const int lane = threadIdx.x & 31;
  for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total; w += (long long)gridDim.x * (blockDim.x >> 5)) {
    const long long r = w / blocks_per_row, b = w % blocks_per_row;
    const T* src = x + r * cols + b * 128 + lane * 4;
    float v[4]; float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[i] = to_f(src[i]); amax = fmaxf(amax, fabsf(v[i])); }
    amax = warp_max(amax);
    float s = fmaxf(amax, 1e-30f) / 448.f;
    if (pow2) s = exp2f(ceilf(log2f(s)));
    const float inv = 1.f / s;
    __nv_fp8_e4m3* dst = q + r * cols + b * 128 + lane * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = __nv_fp8_e4m3(fminf(fmaxf(v[i] * inv, -448.f), 448.f));
    if (lane == 0) scale[r * blocks_per_row + b] = s;
  }
}
}  // namespace

MSB_API int msb_scaled_masked_softmax_fwd(const void* x, const void* mask, void* y, long long rows, int cols, float scale, int sq,
                                          int causal, long long mask_rows, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  MSB_DISPATCH_FLOAT(dtype, T, softmax_fwd_kernel<T><<<(unsigned)rows, 256, 0, s>>>((const T*)x, (const uint8_t*)mask, (T*)y, rows, cols, scale, sq, causal, mask_rows > 0 ? mask_rows : 1));
  MSB_CHECK_LAUNCH("scaled_masked_softmax_fwd");
  return 0;
}
MSB_API int msb_scaled_masked_softmax_bwd(const void* dy, const void* y, void* dx, long long rows, int cols, float scale, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  MSB_DISPATCH_FLOAT(dtype, T, softmax_bwd_kernel<T><<<(unsigned)rows, 256, 0, s>>>((const T*)dy, (const T*)y, (T*)dx, cols, scale));
  MSB_CHECK_LAUNCH("scaled_masked_softmax_bwd");
  return 0;
}
MSB_API int msb_ring_attention_update(const void* prev_out, const float* prev_max, const float* prev_sum, const void* cur_out,
                                      const float* cur_max, const float* cur_sum, void* out, float* out_max, float* out_sum,
                                      long long rows, int d, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  dim3 block(32, 8);
  long long g = (rows + 7) / 8;
  int grid = (int)(g > (long long)msb::num_sms() * 16 ? (long long)msb::num_sms() * 16 : g);
  MSB_DISPATCH_FLOAT(dtype, T, ring_update_kernel<T><<<grid, block, 0, s>>>((const T*)prev_out, prev_max, prev_sum, (const T*)cur_out, cur_max, cur_sum, (T*)out, out_max, out_sum, rows, d));
  MSB_CHECK_LAUNCH("ring_attention_update");
  return 0;
}
MSB_API int msb_add_rmsnorm(const void* x, const void* res, const void* gamma, void* h, void* y, float* rstd, long long rows, int cols,
                            float eps, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  MSB_DISPATCH_FLOAT(dtype, T, add_rmsnorm_kernel<T><<<(unsigned)rows, 256, 0, s>>>((const T*)x, (const T*)res, (const T*)gamma, (T*)h, (T*)y, rstd, cols, eps));
  MSB_CHECK_LAUNCH("add_rmsnorm");
  return 0;
}
MSB_API int msb_quant_1x128(const void* x, void* q, float* scale, long long rows, int cols, int pow2, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  MSB_REQUIRE(cols % 128 == 0, "quant_1x128: cols=%d must be a multiple of 128", cols);
  long long warps = rows * (cols / 128);
  int grid = (int)((warps + 7) / 8); if (grid > msb::num_sms() * 32) grid = msb::num_sms() * 32;
  MSB_DISPATCH_FLOAT(dtype, T, quant_1x128_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (__nv_fp8_e4m3*)q, scale, rows, cols, pow2));
  MSB_CHECK_LAUNCH("quant_1x128");
  return 0;
}
