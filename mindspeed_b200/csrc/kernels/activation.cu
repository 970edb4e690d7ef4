// SwiGLU forward / backward (optionally weighted by per-row router probabilities for MoE).
//   x = [rows, 2F], y[r, j] = silu(x[r, j]) * x[r, F + j]            (chunk(2, dim=-1) convention)
// reference semantics: torch_npu.npu_swiglu(x, dim=-1) used by mindspeed/core/fusions/fused_bias_swiglu.py:4-17,
// weighted form mindspeed/te/pytorch/module/grouped_linear.py:402.
#include "msb_common.cuh"
using namespace msb;

namespace {
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ row_scale,
                                  size_t rows, int F) {
  const int fv = F >> 3;
  const size_t total = rows * (size_t)fv;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / fv;
    int c = (int)(i - r * fv) * 8;
    const T* xr = x + r * (size_t)(2 * F);
    Vec8<T> a, b; a.load(xr + c); b.load(xr + F + c);
    float af[8], bf[8], o[8]; a.to_float(af); b.to_float(bf);
    const float sc = row_scale ? row_scale[r] : 1.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { float sg = 1.f / (1.f + __expf(-af[j])); o[j] = af[j] * sg * bf[j] * sc; }
    Vec8<T> out; out.from_float(o); out.store(y + r * (size_t)F + c);
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx,
                                  const float* __restrict__ row_scale, float* __restrict__ dscale, size_t rows, int F) {
  // dscale (optional): per-row gradient of the scale, accumulated with one atomic per vector
  const int fv = F >> 3;
  const size_t total = rows * (size_t)fv;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / fv;
    int c = (int)(i - r * fv) * 8;
    const T* xr = x + r * (size_t)(2 * F);
    T* dxr = dx + r * (size_t)(2 * F);
    Vec8<T> a, b, g; a.load(xr + c); b.load(xr + F + c); g.load(dy + r * (size_t)F + c);
    float af[8], bf[8], gf[8], da[8], db[8]; a.to_float(af); b.to_float(bf); g.to_float(gf);
    const float sc = row_scale ? row_scale[r] : 1.f;
    float ds = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float sg = 1.f / (1.f + __expf(-af[j]));
      float silu = af[j] * sg;
      ds += gf[j] * silu * bf[j];
      float gs = gf[j] * sc;
      da[j] = gs * bf[j] * sg * (1.f + af[j] * (1.f - sg));
      db[j] = gs * silu;
    }
    Vec8<T> oa, ob; oa.from_float(da); ob.from_float(db);
    oa.store(dxr + c); ob.store(dxr + F + c);
    if (dscale) atomicAdd(dscale + r, ds);
  }
}

template <typename T>
__global__ void gelu_fwd_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ y, size_t n, int cols) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = to_f(x[i]) + (bias ? to_f(bias[i % cols]) : 0.f);
    y[i] = from_f<T>(0.5f * v * (1.f + tanhf(0.79788456f * v * (1.f + 0.044715f * v * v))));
  }
}
}  // namespace

MSB_API int msb_swiglu_fwd(const void* x, void* y, const float* row_scale, long long rows, int F, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  MSB_REQUIRE(F % 8 == 0, "swiglu: F=%d must be a multiple of 8", F);
  size_t total = (size_t)rows * (F / 8);
  int grid = (int)((total + 255) / 256); if (grid > msb::num_sms() * 16) grid = msb::num_sms() * 16;
  MSB_DISPATCH_FLOAT(dtype, T, swiglu_fwd_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (T*)y, row_scale, (size_t)rows, F));
  MSB_CHECK_LAUNCH("swiglu_fwd");
  return 0;
}

MSB_API int msb_swiglu_bwd(const void* dy, const void* x, void* dx, const float* row_scale, float* dscale, long long rows,
                           int F, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  MSB_REQUIRE(F % 8 == 0, "swiglu: F=%d must be a multiple of 8", F);
  size_t total = (size_t)rows * (F / 8);
  int grid = (int)((total + 255) / 256); if (grid > msb::num_sms() * 16) grid = msb::num_sms() * 16;
  MSB_DISPATCH_FLOAT(dtype, T, swiglu_bwd_kernel<T><<<grid, 256, 0, s>>>((const T*)dy, (const T*)x, (T*)dx, row_scale, dscale, (size_t)rows, F));
  MSB_CHECK_LAUNCH("swiglu_bwd");
  return 0;
}

MSB_API int msb_bias_gelu_fwd(const void* x, const void* bias, void* y, long long n, int cols, int dtype, cudaStream_t s) {
  if (n == 0) return 0;
  int grid = (int)((n + 255) / 256); if (grid > msb::num_sms() * 16) grid = msb::num_sms() * 16;
  MSB_DISPATCH_FLOAT(dtype, T, gelu_fwd_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (const T*)bias, (T*)y, (size_t)n, cols));
  MSB_CHECK_LAUNCH("bias_gelu_fwd");
  return 0;
}
