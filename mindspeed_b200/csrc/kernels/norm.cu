// RMSNorm / LayerNorm forward and backward, bandwidth-bound.
//
// Forward: one thread block per row, the row is held in registers (up to
// MAX_VEC 16-byte vectors per thread) so x is read from HBM exactly once.
// Backward: a persistent grid walks rows; dgamma partial sums stay in registers
// per column slot and are written once per block to a [grid, cols] fp32 scratch,
// then reduced by a second kernel (fixed order => run-to-run deterministic).
//
// Math (reference semantics: torch_npu.npu_rms_norm used by
// mindspeed/core/fusions/fused_rms_norm.py:36-42):
//   rstd = rsqrt(mean(x^2) + eps);  y = x * rstd * gamma
//   dx   = rstd * (dy*gamma - xhat * mean(dy*gamma*xhat)),  dgamma = sum_rows(dy * xhat)
#include "msb_common.cuh"
using namespace msb;

namespace {
constexpr int MAX_VEC = 4;  // vectors of 8 elements per thread kept in registers

template <typename T, bool ZERO_CENTERED>
__global__ void __launch_bounds__(1024) rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                           T* __restrict__ y, float* __restrict__ rstd_out, int rows,
                                                           int cols, float eps) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nvec = cols >> 3;
  const T* xr = x + (size_t)row * cols;
  T* yr = y + (size_t)row * cols;
  float vals[MAX_VEC][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAX_VEC; ++k) {
    int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) {
      Vec8<T> t; t.load(xr + v * 8); t.to_float(vals[k]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[k][j] * vals[k][j];
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)cols + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int k = 0; k < MAX_VEC; ++k) {
    int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) {
      Vec8<T> g; g.load(gamma + v * 8);
      float gf[8]; g.to_float(gf);
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[k][j] * rstd * (ZERO_CENTERED ? gf[j] + 1.f : gf[j]);
      Vec8<T> out; out.from_float(o); out.store(yr + v * 8);
    }
  }
}

// scalar fallback for rows that are not a multiple of 8 or exceed the register budget
template <typename T, bool ZERO_CENTERED>
__global__ void rmsnorm_fwd_generic(const T* __restrict__ x, const T* __restrict__ gamma, T* __restrict__ y,
                                    float* __restrict__ rstd_out, int rows, int cols, float eps) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const T* xr = x + (size_t)row * cols;
  T* yr = y + (size_t)row * cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) { float v = to_f(xr[c]); ss += v * v; }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)cols + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float g = to_f(gamma[c]);
    yr[c] = from_f<T>(to_f(xr[c]) * rstd * (ZERO_CENTERED ? g + 1.f : g));
  }
}

template <typename T, bool ZERO_CENTERED>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                           const T* __restrict__ gamma, const float* __restrict__ rstd,
                                                           T* __restrict__ dx, float* __restrict__ dgamma_partial,
                                                           int rows, int cols) {
  __shared__ float red[32];
  const int nvec = cols >> 3;
  float gf[MAX_VEC][8];
  float dg[MAX_VEC][8];
#pragma unroll
  for (int k = 0; k < MAX_VEC; ++k) {
    int v = threadIdx.x + k * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dg[k][j] = 0.f; gf[k][j] = 0.f; }
    if (v < nvec) {
      Vec8<T> g; g.load(gamma + v * 8); g.to_float(gf[k]);
      if (ZERO_CENTERED) {
#pragma unroll
        for (int j = 0; j < 8; ++j) gf[k][j] += 1.f;
      }
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + (size_t)row * cols;
    const T* dyr = dy + (size_t)row * cols;
    T* dxr = dx + (size_t)row * cols;
    const float rs = rstd[row];
    float xh[MAX_VEC][8], wdy[MAX_VEC][8];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < MAX_VEC; ++k) {
      int v = threadIdx.x + k * blockDim.x;
      if (v < nvec) {
        Vec8<T> a, b; a.load(xr + v * 8); b.load(dyr + v * 8);
        float xf[8], df[8]; a.to_float(xf); b.to_float(df);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[k][j] = xf[j] * rs;
          wdy[k][j] = df[j] * gf[k][j];
          dot += wdy[k][j] * xh[k][j];
          dg[k][j] += df[j] * xh[k][j];
        }
      }
    }
    dot = block_sum(dot, red) / (float)cols;
#pragma unroll
    for (int k = 0; k < MAX_VEC; ++k) {
      int v = threadIdx.x + k * blockDim.x;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (wdy[k][j] - xh[k][j] * dot);
        Vec8<T> out; out.from_float(o); out.store(dxr + v * 8);
      }
    }
  }
  float* part = dgamma_partial + (size_t)blockIdx.x * cols;
#pragma unroll
  for (int k = 0; k < MAX_VEC; ++k) {
    int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) {
      Vec8<float> o; o.from_float(dg[k]); o.store(part + v * 8);
    }
  }
}

// generic backward: one block per row, scalar accesses, dgamma through fp32 atomics into scratch[cols]
template <typename T, bool ZERO_CENTERED>
__global__ void rmsnorm_bwd_generic(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                                    const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dgamma_acc,
                                    int rows, int cols) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const T* xr = x + (size_t)row * cols;
  const T* dyr = dy + (size_t)row * cols;
  T* dxr = dx + (size_t)row * cols;
  const float rs = rstd[row];
  float dot = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float g = to_f(gamma[c]); if (ZERO_CENTERED) g += 1.f;
    dot += to_f(dyr[c]) * g * to_f(xr[c]) * rs;
  }
  dot = block_sum(dot, red) / (float)cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float g = to_f(gamma[c]); if (ZERO_CENTERED) g += 1.f;
    float xh = to_f(xr[c]) * rs, d = to_f(dyr[c]);
    dxr[c] = from_f<T>(rs * (d * g - xh * dot));
    atomicAdd(dgamma_acc + c, d * xh);
  }
}

template <typename T>
__global__ void colsum_partials_kernel(const float* __restrict__ partial, T* __restrict__ out, int nparts, int cols,
                                       int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[(size_t)p * cols + c];
  if (accumulate) s += to_f(out[c]);
  out[c] = from_f<T>(s);
}

inline int pick_threads(int nvec, int cap = 1024) {
  int t = (nvec + MAX_VEC - 1) / MAX_VEC;
  t = ((t + 31) / 32) * 32;
  if (t < 32) t = 32;
  if (t > cap) t = cap;
  return t;
}
constexpr int BWD_MAX_COLS = 256 * MAX_VEC * 8;
}  // namespace

MSB_API int msb_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, int rows, int cols, float eps,
                            int zero_centered, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  const bool fast = (cols % 8 == 0) && (cols / 8 <= MAX_VEC * 1024);
  MSB_DISPATCH_FLOAT(dtype, T, {
    if (fast) {
      int th = pick_threads(cols / 8);
      if (zero_centered) rmsnorm_fwd_kernel<T, true><<<rows, th, 0, s>>>((const T*)x, (const T*)gamma, (T*)y, rstd, rows, cols, eps);
      else rmsnorm_fwd_kernel<T, false><<<rows, th, 0, s>>>((const T*)x, (const T*)gamma, (T*)y, rstd, rows, cols, eps);
    } else {
      if (zero_centered) rmsnorm_fwd_generic<T, true><<<rows, 256, 0, s>>>((const T*)x, (const T*)gamma, (T*)y, rstd, rows, cols, eps);
      else rmsnorm_fwd_generic<T, false><<<rows, 256, 0, s>>>((const T*)x, (const T*)gamma, (T*)y, rstd, rows, cols, eps);
    }
  });
  MSB_CHECK_LAUNCH("rmsnorm_fwd");
  return 0;
}

// Number of fp32 scratch elements msb_rmsnorm_bwd needs for a given problem.
MSB_API size_t msb_rmsnorm_bwd_scratch_elems(int rows, int cols) {
  if (cols % 8 != 0 || cols > BWD_MAX_COLS) return (size_t)cols;
  int grid = msb::num_sms() * 2;
  if (grid > rows) grid = rows;
  if (grid < 1) grid = 1;
  return (size_t)grid * cols;
}

MSB_API int msb_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx, void* dgamma,
                            float* scratch, int rows, int cols, int zero_centered, int accumulate_dgamma, int dtype,
                            cudaStream_t s) {
  if (rows == 0) return 0;
  const bool fast = (cols % 8 == 0) && cols <= BWD_MAX_COLS;
  int grid = msb::num_sms() * 2;
  if (grid > rows) grid = rows;
  MSB_DISPATCH_FLOAT(dtype, T, {
    if (fast) {
      int th = pick_threads(cols / 8, 256);
      if (zero_centered) rmsnorm_bwd_kernel<T, true><<<grid, th, 0, s>>>((const T*)dy, (const T*)x, (const T*)gamma, rstd, (T*)dx, scratch, rows, cols);
      else rmsnorm_bwd_kernel<T, false><<<grid, th, 0, s>>>((const T*)dy, (const T*)x, (const T*)gamma, rstd, (T*)dx, scratch, rows, cols);
      MSB_CHECK_LAUNCH("rmsnorm_bwd");
    } else {
      grid = 1;
      if (cudaMemsetAsync(scratch, 0, sizeof(float) * (size_t)cols, s) != cudaSuccess) { msb_set_error("rmsnorm_bwd: memset failed"); return 1; }
      if (zero_centered) rmsnorm_bwd_generic<T, true><<<rows, 256, 0, s>>>((const T*)dy, (const T*)x, (const T*)gamma, rstd, (T*)dx, scratch, rows, cols);
      else rmsnorm_bwd_generic<T, false><<<rows, 256, 0, s>>>((const T*)dy, (const T*)x, (const T*)gamma, rstd, (T*)dx, scratch, rows, cols);
      MSB_CHECK_LAUNCH("rmsnorm_bwd_generic");
    }
    colsum_partials_kernel<T><<<(cols + 255) / 256, 256, 0, s>>>(scratch, (T*)dgamma, grid, cols, accumulate_dgamma);
    MSB_CHECK_LAUNCH("rmsnorm_bwd_reduce");
  });
  return 0;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate (declared in include/msb_noalloc.h).
//
// Same math and kernels as msb_rmsnorm_bwd, but the fp32 partial-sum scratch is a fixed array that
// lives inside this library instead of a buffer the caller provides.
// ---------------------------------------------------------------------------------------------
#define MSB_NOALLOC_SCRATCH_FLOATS (512 * 1024)  // 2 MiB per GPU that loads the library
static __device__ __align__(256) float g_noalloc_scratch[MSB_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};

// Device address of the scratch array for the current device. In host code the array's name is only a
// stand-in symbol, not something a kernel can dereference, so it is translated once per device.
int noalloc_scratch(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
    msb_set_error("rmsnorm_bwd_noalloc: cannot identify the current device");
    return 1;
  }
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      msb_set_error("rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return 1;
    }
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

MSB_API size_t msb_rmsnorm_bwd_noalloc_max_cols() { return (size_t)BWD_MAX_COLS; }

MSB_API int msb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx,
                                    void* dgamma, int rows, int cols, int zero_centered, int accumulate_dgamma,
                                    int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  MSB_REQUIRE(rows > 0 && cols > 0, "rmsnorm_bwd_noalloc: rows=%d cols=%d must be positive", rows, cols);
  MSB_REQUIRE(cols % 8 == 0 && cols <= BWD_MAX_COLS,
              "rmsnorm_bwd_noalloc: cols=%d is not supported (multiple of 8, at most %d); use msb_rmsnorm_bwd with "
              "caller-provided scratch instead", cols, BWD_MAX_COLS);
  float* scratch = nullptr;
  if (noalloc_scratch(&scratch) != 0) return 1;
  int grid = msb::num_sms() * 2;
  if (grid > rows) grid = rows;
  const int fit = MSB_NOALLOC_SCRATCH_FLOATS / cols;  // >= 64 because cols <= 8192
  if (grid > fit) grid = fit;
  // every one of the grid*cols partial sums is overwritten by the first kernel before the second reads it,
  // so nothing left over from an earlier call needs clearing
  MSB_DISPATCH_FLOAT(dtype, T, {
    int th = pick_threads(cols / 8, 256);
    if (zero_centered) rmsnorm_bwd_kernel<T, true><<<grid, th, 0, s>>>((const T*)dy, (const T*)x, (const T*)gamma, rstd, (T*)dx, scratch, rows, cols);
    else rmsnorm_bwd_kernel<T, false><<<grid, th, 0, s>>>((const T*)dy, (const T*)x, (const T*)gamma, rstd, (T*)dx, scratch, rows, cols);
    MSB_CHECK_LAUNCH("rmsnorm_bwd_noalloc");
    colsum_partials_kernel<T><<<(cols + 255) / 256, 256, 0, s>>>(scratch, (T*)dgamma, grid, cols, accumulate_dgamma);
    MSB_CHECK_LAUNCH("rmsnorm_bwd_noalloc_reduce");
  });
  return 0;
}
