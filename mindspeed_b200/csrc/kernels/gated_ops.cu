// Gated RMSNorm and Sinkhorn normalisation (the small fused ops the reference keeps as Triton kernels:
// mindspeed/lite/ops/triton/fused_norm_gate.py:31-325 and mindspeed/lite/ops/triton/sinkhorn.py:11-363).
//
//   gated RMSNorm   y = rmsnorm(x) * w * silu(g)          one warp per row, bf16/fp32 I/O, fp32 math
//                   backward gives dx, dg and per-CTA partial dw (summed by the caller)
//   Sinkhorn        P = exp(logits); repeat `iters` times: rows /= row sums, columns /= column sums
//                   n x n matrices with n <= 8 (hyper-connection mixing weights), one thread per matrix;
//                   the backward recomputes the forward, keeps only the row / column sums of every iteration and walks
//                   the iterations in reverse, rebuilding the iterates by multiplying the sums back in.
#include "msb_common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float silu(float z) { return z / (1.f + __expf(-z)); }
__device__ __forceinline__ float dsilu(float z) { const float s = 1.f / (1.f + __expf(-z)); return s * (1.f + z * (1.f - s)); }

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_gated_fwd_kernel(const T* __restrict__ x, const T* __restrict__ g, const T* __restrict__ w,
                                                                 T* __restrict__ y, float* __restrict__ rstd, long long rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const long long base = row * cols;
  float ss = 0.f;
  for (int c = lane; c < cols; c += 32) { const float v = ldf(x, base + c); ss += v * v; }
  ss = msb::warp_sum(ss);
  const float r = rsqrtf(ss / cols + eps);
  if (lane == 0) rstd[row] = r;
  for (int c = lane; c < cols; c += 32)
    stf(y, base + c, ldf(x, base + c) * r * ldf(w, c) * silu(ldf(g, base + c)));
}

// dw_partial: [gridDim.x, cols] fp32, each CTA accumulates its rows (8 warps) through shared memory
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_gated_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ g,
                                                                 const T* __restrict__ w, const float* __restrict__ rstd, T* __restrict__ dx,
                                                                 T* __restrict__ dg, float* __restrict__ dw_partial, long long rows, int cols,
                                                                 int rows_per_cta) {
  extern __shared__ float s_dw[];       // [cols]
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s_dw[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const long long row0 = (long long)blockIdx.x * rows_per_cta;
  for (long long row = row0 + warp; row < row0 + rows_per_cta && row < rows; row += nw) {
    const long long base = row * cols;
    const float r = rstd[row];
    // t_c = dy_c * silu(g_c) * w_c ; dx_c = r * (t_c - xhat_c * mean(t * xhat))
    float dot = 0.f;
    for (int c = lane; c < cols; c += 32) {
      const float xh = ldf(x, base + c) * r;
      dot += ldf(dy, base + c) * silu(ldf(g, base + c)) * ldf(w, c) * xh;
    }
    dot = msb::warp_sum(dot) / cols;
    for (int c = lane; c < cols; c += 32) {
      const float xv = ldf(x, base + c), gv = ldf(g, base + c), dyv = ldf(dy, base + c), wv = ldf(w, c);
      const float xh = xv * r, sg = silu(gv);
      stf(dx, base + c, r * (dyv * sg * wv - xh * dot));
      stf(dg, base + c, dyv * xh * wv * dsilu(gv));
      atomicAdd(&s_dw[c], dyv * sg * xh);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dw_partial[(long long)blockIdx.x * cols + c] = s_dw[c];
}

constexpr int SK_MAX_N = 8;
constexpr int SK_MAX_ITERS = 32;

__global__ void __launch_bounds__(128) sinkhorn_fwd_kernel(const float* __restrict__ logits, float* __restrict__ out, long long count, int n,
                                                           int iters, float eps) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float m[SK_MAX_N * SK_MAX_N];
  const float* src = logits + i * n * n;
  float mx = -3.0e38f;
  for (int k = 0; k < n * n; ++k) mx = fmaxf(mx, src[k]);
  for (int k = 0; k < n * n; ++k) m[k] = __expf(src[k] - mx);
  for (int it = 0; it < iters; ++it) {
    for (int r = 0; r < n; ++r) {
      float s = eps;
      for (int c = 0; c < n; ++c) s += m[r * n + c];
      const float inv = 1.f / s;
      for (int c = 0; c < n; ++c) m[r * n + c] *= inv;
    }
    for (int c = 0; c < n; ++c) {
      float s = eps;
      for (int r = 0; r < n; ++r) s += m[r * n + c];
      const float inv = 1.f / s;
      for (int r = 0; r < n; ++r) m[r * n + c] *= inv;
    }
  }
  for (int k = 0; k < n * n; ++k) out[i * n * n + k] = m[k];
}

__global__ void __launch_bounds__(128) sinkhorn_bwd_kernel(const float* __restrict__ logits, const float* __restrict__ dout,
                                                           float* __restrict__ dlogits, long long count, int n, int iters, float eps) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float m[SK_MAX_N * SK_MAX_N], d[SK_MAX_N * SK_MAX_N];
  float rs[SK_MAX_ITERS][SK_MAX_N], cs[SK_MAX_ITERS][SK_MAX_N];
  const float* src = logits + i * n * n;
  float mx = -3.0e38f;
  for (int k = 0; k < n * n; ++k) mx = fmaxf(mx, src[k]);
  for (int k = 0; k < n * n; ++k) m[k] = __expf(src[k] - mx);
  for (int it = 0; it < iters; ++it) {
    for (int r = 0; r < n; ++r) {
      float s = eps;
      for (int c = 0; c < n; ++c) s += m[r * n + c];
      rs[it][r] = s;
      for (int c = 0; c < n; ++c) m[r * n + c] /= s;
    }
    for (int c = 0; c < n; ++c) {
      float s = eps;
      for (int r = 0; r < n; ++r) s += m[r * n + c];
      cs[it][c] = s;
      for (int r = 0; r < n; ++r) m[r * n + c] /= s;
    }
  }
  for (int k = 0; k < n * n; ++k) d[k] = dout[i * n * n + k];
  // reverse: Y = X / s(X)  =>  dX = (dY - sum(dY * Y)) / s   along the normalised axis
  for (int it = iters - 1; it >= 0; --it) {
    for (int c = 0; c < n; ++c) {
      float dot = 0.f;
      for (int r = 0; r < n; ++r) dot += d[r * n + c] * m[r * n + c];
      for (int r = 0; r < n; ++r) { d[r * n + c] = (d[r * n + c] - dot) / cs[it][c]; m[r * n + c] *= cs[it][c]; }
    }
    for (int r = 0; r < n; ++r) {
      float dot = 0.f;
      for (int c = 0; c < n; ++c) dot += d[r * n + c] * m[r * n + c];
      for (int c = 0; c < n; ++c) { d[r * n + c] = (d[r * n + c] - dot) / rs[it][r]; m[r * n + c] *= rs[it][r]; }
    }
  }
  for (int k = 0; k < n * n; ++k) dlogits[i * n * n + k] = d[k] * m[k];     // through exp: m is exp(logit - max) again
}

}  // namespace

MSB_API int msb_rmsnorm_gated_fwd(const void* x, const void* g, const void* w, void* y, float* rstd, long long rows, int cols, float eps,
                                  int dtype, cudaStream_t s) {
  MSB_REQUIRE(rows > 0 && cols > 0, "rmsnorm_gated_fwd: empty input");
  const int grid = (int)((rows + 7) / 8);
  if (dtype == MSB_BF16)
    rmsnorm_gated_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)g, (const __nv_bfloat16*)w,
                                                                 (__nv_bfloat16*)y, rstd, rows, cols, eps);
  else if (dtype == MSB_F32)
    rmsnorm_gated_fwd_kernel<float><<<grid, 256, 0, s>>>((const float*)x, (const float*)g, (const float*)w, (float*)y, rstd, rows, cols, eps);
  else { msb_set_error("rmsnorm_gated_fwd: unsupported dtype %d", dtype); return 2; }
  MSB_CHECK_LAUNCH("rmsnorm_gated_fwd");
  return 0;
}

MSB_API int msb_rmsnorm_gated_bwd_ctas(long long rows) {
  long long g = (rows + 63) / 64;
  return (int)(g > 1184 ? 1184 : (g < 1 ? 1 : g));
}

// dw_partial must hold msb_rmsnorm_gated_bwd_ctas(rows) * cols floats; the caller sums it over the first dimension.
MSB_API int msb_rmsnorm_gated_bwd(const void* dy, const void* x, const void* g, const void* w, const float* rstd, void* dx, void* dg,
                                  float* dw_partial, long long rows, int cols, int dtype, cudaStream_t s) {
  MSB_REQUIRE(rows > 0 && cols > 0 && cols <= 12288, "rmsnorm_gated_bwd: cols=%d out of range", cols);
  const int grid = msb_rmsnorm_gated_bwd_ctas(rows);
  const int rpc = (int)((rows + grid - 1) / grid);
  const size_t smem = sizeof(float) * (size_t)cols;
  if (dtype == MSB_BF16)
    rmsnorm_gated_bwd_kernel<__nv_bfloat16><<<grid, 256, smem, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)g,
                                                                    (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, (__nv_bfloat16*)dg,
                                                                    dw_partial, rows, cols, rpc);
  else if (dtype == MSB_F32)
    rmsnorm_gated_bwd_kernel<float><<<grid, 256, smem, s>>>((const float*)dy, (const float*)x, (const float*)g, (const float*)w, rstd,
                                                            (float*)dx, (float*)dg, dw_partial, rows, cols, rpc);
  else { msb_set_error("rmsnorm_gated_bwd: unsupported dtype %d", dtype); return 2; }
  MSB_CHECK_LAUNCH("rmsnorm_gated_bwd");
  return 0;
}

MSB_API int msb_sinkhorn_fwd(const float* logits, float* out, long long count, int n, int iters, float eps, cudaStream_t s) {
  MSB_REQUIRE(n >= 1 && n <= SK_MAX_N && iters >= 0 && iters <= SK_MAX_ITERS, "sinkhorn: n=%d (max %d), iters=%d (max %d)", n, SK_MAX_N, iters, SK_MAX_ITERS);
  if (count == 0) return 0;
  sinkhorn_fwd_kernel<<<(int)((count + 127) / 128), 128, 0, s>>>(logits, out, count, n, iters, eps);
  MSB_CHECK_LAUNCH("sinkhorn_fwd");
  return 0;
}
MSB_API int msb_sinkhorn_bwd(const float* logits, const float* dout, float* dlogits, long long count, int n, int iters, float eps, cudaStream_t s) {
  MSB_REQUIRE(n >= 1 && n <= SK_MAX_N && iters >= 0 && iters <= SK_MAX_ITERS, "sinkhorn: n=%d (max %d), iters=%d (max %d)", n, SK_MAX_N, iters, SK_MAX_ITERS);
  if (count == 0) return 0;
  sinkhorn_bwd_kernel<<<(int)((count + 127) / 128), 128, 0, s>>>(logits, dout, dlogits, count, n, iters, eps);
  MSB_CHECK_LAUNCH("sinkhorn_bwd");
  return 0;
}
