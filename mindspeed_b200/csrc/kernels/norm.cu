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
// ---------------------------------------------------------------------------------------------------------------
// Fast path layout (both directions): a row is covered by one GROUP of TPR threads, each thread owning VPT vectors of
// 8 elements (vector v = tid + k * TPR).  A block holds G groups, every group walks its own rows of a persistent grid
// and loads the NEXT row's vectors before it reduces the current one, so each thread always has 2 * VPT 16-byte loads
// per input tensor in flight and the block-level reduction of one row overlaps the memory latency of the next.
// Groups synchronise among themselves with a named barrier (id 1 + group), never with the whole block.
// ---------------------------------------------------------------------------------------------------------------
constexpr int MAX_VPT = 4;             // vectors of 8 elements per thread
constexpr int MAX_TPR = 512;           // threads per row
constexpr int FAST_MAX_COLS = MAX_TPR * MAX_VPT * 8;   // 16384

__device__ __forceinline__ void group_bar(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Sum over the TPR threads of a group.  ``red`` holds [2][16] floats for this group; ``parity`` alternates per row so
// that a fast warp writing the next row's partial never overwrites one that a slow warp still has to read.
__device__ __forceinline__ float group_sum(float v, float* red, int parity, int gtid, int tpr, int bar_id) {
  v = warp_sum(v);
  const int nw = tpr >> 5;
  if (nw == 1) return v;
  float* r = red + parity * 16;
  if ((gtid & 31) == 0) r[gtid >> 5] = v;
  group_bar(bar_id, tpr);
  float t = ((gtid & 31) < nw) ? r[gtid & 31] : 0.f;
  return warp_sum(t);
}

struct RowPlan { int vpt, tpr, groups; };
inline RowPlan plan_row(int cols, int max_block, bool prefer2 = false) {
  const int nvec = cols >> 3;
  int vpt = 1;
  while (vpt < MAX_VPT && (nvec + vpt - 1) / vpt > MAX_TPR) vpt <<= 1;
  // forward only: two vectors per thread once a row has enough of them (fewer, fatter threads reduce faster); the
  // backward kernel keeps one, its dgamma accumulators would not fit 64 registers otherwise
  if (prefer2 && vpt == 1 && nvec >= 512) vpt = 2;
  int tpr = (nvec + vpt - 1) / vpt;
  tpr = ((tpr + 31) / 32) * 32;
  int groups = max_block / tpr;
  if (groups < 1) groups = 1;
  if (groups > 8) groups = 8;
  return {vpt, tpr, groups};
}

template <typename T, bool ZERO_CENTERED, int VPT>
__global__ void __launch_bounds__(1024) rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                           T* __restrict__ y, float* __restrict__ rstd_out, int rows,
                                                           int cols, float eps, int tpr, const T* __restrict__ res,
                                                           T* __restrict__ h_out) {
  // res != nullptr: the row that is normalised is h = x + res, rounded to T and also written to h_out
  __shared__ float red_all[8 * 32];
  const int g = threadIdx.x / tpr, gtid = threadIdx.x - g * tpr, groups = blockDim.x / tpr;
  float* red = red_all + g * 32;
  const int nvec = cols >> 3;
  Vec8<T> gam[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = gtid + k * tpr;
    if (v < nvec) gam[k].load(gamma + v * 8);
  }
  Vec8<T> cur[VPT], nxt[VPT], rcur[VPT], rnxt[VPT];
  int row = blockIdx.x * groups + g;
  const int stride = gridDim.x * groups;
  if (row < rows) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = gtid + k * tpr;
      if (v < nvec) {
        cur[k].load(x + (size_t)row * cols + v * 8);
        if (res) rcur[k].load(res + (size_t)row * cols + v * 8);
      }
    }
  }
  int parity = 0;
  for (; row < rows; row += stride, parity ^= 1) {
    const int nrow = row + stride;
    if (nrow < rows) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = gtid + k * tpr;
        if (v < nvec) {
          nxt[k].load(x + (size_t)nrow * cols + v * 8);
          if (res) rnxt[k].load(res + (size_t)nrow * cols + v * 8);
        }
      }
    }
    if (res) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = gtid + k * tpr;
        if (v < nvec) {
          float a[8], b[8];
          cur[k].to_float(a); rcur[k].to_float(b);
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] += b[j];
          cur[k].from_float(a);                         // rounded: the norm sees exactly what h_out holds
          cur[k].store(h_out + (size_t)row * cols + v * 8);
        }
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      if (gtid + k * tpr < nvec) {
        float f[8]; cur[k].to_float(f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
      }
    }
    ss = group_sum(ss, red, parity, gtid, tpr, 1 + g);
    const float rstd = rsqrtf(ss / (float)cols + eps);
    if (gtid == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = gtid + k * tpr;
      if (v < nvec) {
        float f[8], gf[8], o[8];
        cur[k].to_float(f); gam[k].to_float(gf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = f[j] * rstd * (ZERO_CENTERED ? gf[j] + 1.f : gf[j]);
        Vec8<T> out; out.from_float(o); out.store(y + (size_t)row * cols + v * 8);
      }
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) { cur[k] = nxt[k]; if (res) rcur[k] = rnxt[k]; }
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

// Backward.  dgamma partial sums stay in registers per thread for all the rows of its group; at the end the groups of
// a block add theirs in a fixed order through shared memory and the block writes ONE fp32 row of partials.
template <typename T, bool ZERO_CENTERED, int VPT>
__global__ void __launch_bounds__(1024) rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                            const T* __restrict__ gamma, const float* __restrict__ rstd,
                                                            T* __restrict__ dx, float* __restrict__ dgamma_partial,
                                                            int rows, int cols, int tpr, const T* __restrict__ addend) {
  // addend != nullptr: dx = (gradient through the norm) + addend, the gradient that reaches the same tensor directly
  extern __shared__ float dg_smem[];          // [cols] when the block has more than one group
  __shared__ float red_all[8 * 32];
  const int g = threadIdx.x / tpr, gtid = threadIdx.x - g * tpr, groups = blockDim.x / tpr;
  float* red = red_all + g * 32;
  const int nvec = cols >> 3;
  Vec8<T> gam[VPT];
  float dg[VPT][8];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = gtid + k * tpr;
#pragma unroll
    for (int j = 0; j < 8; ++j) dg[k][j] = 0.f;
    if (v < nvec) gam[k].load(gamma + v * 8);
  }
  Vec8<T> cx[VPT], cd[VPT], nx[VPT], nd[VPT];
  int row = blockIdx.x * groups + g;
  const int stride = gridDim.x * groups;
  float rs = 0.f, nrs = 0.f;
  if (row < rows) {
    rs = rstd[row];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = gtid + k * tpr;
      if (v < nvec) { cx[k].load(x + (size_t)row * cols + v * 8); cd[k].load(dy + (size_t)row * cols + v * 8); }
    }
  }
  int parity = 0;
  for (; row < rows; row += stride, parity ^= 1) {
    const int nrow = row + stride;
    if (nrow < rows) {
      nrs = rstd[nrow];
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = gtid + k * tpr;
        if (v < nvec) { nx[k].load(x + (size_t)nrow * cols + v * 8); nd[k].load(dy + (size_t)nrow * cols + v * 8); }
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      if (gtid + k * tpr < nvec) {
        float xf[8], df[8], gf[8];
        cx[k].to_float(xf); cd[k].to_float(df); gam[k].to_float(gf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = xf[j] * rs;
          dot += df[j] * (ZERO_CENTERED ? gf[j] + 1.f : gf[j]) * xh;
          dg[k][j] += df[j] * xh;
        }
      }
    }
    dot = group_sum(dot, red, parity, gtid, tpr, 1 + g) / (float)cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = gtid + k * tpr;
      if (v < nvec) {
        float xf[8], df[8], gf[8], o[8];
        cx[k].to_float(xf); cd[k].to_float(df); gam[k].to_float(gf);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          o[j] = rs * (df[j] * (ZERO_CENTERED ? gf[j] + 1.f : gf[j]) - xf[j] * rs * dot);
        if (addend) {
          Vec8<T> ad; ad.load(addend + (size_t)row * cols + v * 8);
          float af[8]; ad.to_float(af);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += af[j];
        }
        Vec8<T> out; out.from_float(o); out.store(dx + (size_t)row * cols + v * 8);
      }
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) { cx[k] = nx[k]; cd[k] = nd[k]; }
    rs = nrs;
  }
  float* part = dgamma_partial + (size_t)blockIdx.x * cols;
  if (groups == 1) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = gtid + k * tpr;
      if (v < nvec) { Vec8<float> o; o.from_float(dg[k]); o.store(part + v * 8); }
    }
    return;
  }
  // groups add into shared memory one after the other (fixed order: run-to-run identical sums)
  for (int turn = 0; turn < groups; ++turn) {
    if (g == turn) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = gtid + k * tpr;
        if (v < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) dg_smem[v * 8 + j] = (turn == 0 ? 0.f : dg_smem[v * 8 + j]) + dg[k][j];
        }
      }
    }
    __syncthreads();
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) part[c] = dg_smem[c];
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

constexpr int BWD_MAX_COLS = 8192;      // limit of the allocation-free entry point's built-in scratch

// several groups per block share a [cols] fp32 array in shared memory for the final dgamma sum; rows too wide for the
// default 48 KB get one group per block, which needs none
inline RowPlan plan_bwd(int cols) {
  RowPlan rp = plan_row(cols, 1024);
  if (rp.groups > 1 && sizeof(float) * (size_t)cols > 40 * 1024) rp.groups = 1;
  return rp;
}

inline int bwd_grid(int rows, const RowPlan& rp) {
  // persistent: as many blocks as are resident at once (the kernel needs up to 64 registers per thread)
  int grid = msb::num_sms() * (1024 / (rp.tpr * rp.groups) > 0 ? 1024 / (rp.tpr * rp.groups) : 1);
  const int need = (rows + rp.groups - 1) / rp.groups;
  if (grid > need) grid = need;
  return grid < 1 ? 1 : grid;
}

template <typename T>
void launch_fwd(const void* x, const void* gamma, void* y, float* rstd, int rows, int cols, float eps, int zc, cudaStream_t s,
                const void* res = nullptr, void* h_out = nullptr) {
  const RowPlan rp = plan_row(cols, 512, true);
  int grid = msb::num_sms() * 4;
  const int need = (rows + rp.groups - 1) / rp.groups;
  if (grid > need) grid = need;
  const int th = rp.tpr * rp.groups;
#define MSB_FWD(V)                                                                                                             \
  if (zc) rmsnorm_fwd_kernel<T, true, V><<<grid, th, 0, s>>>((const T*)x, (const T*)gamma, (T*)y, rstd, rows, cols, eps, rp.tpr, (const T*)res, (T*)h_out); \
  else rmsnorm_fwd_kernel<T, false, V><<<grid, th, 0, s>>>((const T*)x, (const T*)gamma, (T*)y, rstd, rows, cols, eps, rp.tpr, (const T*)res, (T*)h_out);
  if (rp.vpt == 1) { MSB_FWD(1) } else if (rp.vpt == 2) { MSB_FWD(2) } else { MSB_FWD(4) }
#undef MSB_FWD
}

// returns the number of partial rows written to ``scratch`` (= grid)
template <typename T>
int launch_bwd(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx, float* scratch, int rows, int cols,
               int zc, int max_grid, cudaStream_t s, const void* addend = nullptr) {
  const RowPlan rp = plan_bwd(cols);
  int grid = bwd_grid(rows, rp);
  if (max_grid > 0 && grid > max_grid) grid = max_grid;
  const int th = rp.tpr * rp.groups;
  const size_t smem = rp.groups > 1 ? sizeof(float) * (size_t)cols : 0;
#define MSB_BWD(V)                                                                                                                        \
  if (zc) rmsnorm_bwd_kernel<T, true, V><<<grid, th, smem, s>>>((const T*)dy, (const T*)x, (const T*)gamma, rstd, (T*)dx, scratch, rows, cols, rp.tpr, (const T*)addend); \
  else rmsnorm_bwd_kernel<T, false, V><<<grid, th, smem, s>>>((const T*)dy, (const T*)x, (const T*)gamma, rstd, (T*)dx, scratch, rows, cols, rp.tpr, (const T*)addend);
  if (rp.vpt == 1) { MSB_BWD(1) } else if (rp.vpt == 2) { MSB_BWD(2) } else { MSB_BWD(4) }
#undef MSB_BWD
  return grid;
}
}  // namespace

MSB_API int msb_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, int rows, int cols, float eps,
                            int zero_centered, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  const bool fast = (cols % 8 == 0) && cols <= FAST_MAX_COLS;
  MSB_DISPATCH_FLOAT(dtype, T, {
    if (fast) {
      launch_fwd<T>(x, gamma, y, rstd, rows, cols, eps, zero_centered, s);
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
  if (cols % 8 != 0 || cols > FAST_MAX_COLS) return (size_t)cols;
  return (size_t)bwd_grid(rows, plan_bwd(cols)) * cols;
}

// 1 when (cols) takes the vector kernels, which is what the fused residual forms below need
MSB_API int msb_rmsnorm_fast_path(int cols) { return (cols % 8 == 0) && cols <= FAST_MAX_COLS; }

// h = x + res (rounded to the tensor type, written to h);  y = rmsnorm(h) * gamma;  rstd per row
MSB_API int msb_add_rmsnorm_fwd(const void* x, const void* res, const void* gamma, void* h, void* y, float* rstd, int rows, int cols,
                                float eps, int zero_centered, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  MSB_REQUIRE(msb_rmsnorm_fast_path(cols), "add_rmsnorm_fwd: cols=%d must be a multiple of 8 and at most %d", cols, FAST_MAX_COLS);
  MSB_DISPATCH_FLOAT(dtype, T, launch_fwd<T>(x, gamma, y, rstd, rows, cols, eps, zero_centered, s, res, h));
  MSB_CHECK_LAUNCH("add_rmsnorm_fwd");
  return 0;
}

MSB_API int msb_rmsnorm_bwd_add(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx, void* dgamma,
                                float* scratch, int rows, int cols, int zero_centered, int accumulate_dgamma, int dtype,
                                const void* addend, cudaStream_t s);

MSB_API int msb_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx, void* dgamma,
                            float* scratch, int rows, int cols, int zero_centered, int accumulate_dgamma, int dtype,
                            cudaStream_t s) {
  return msb_rmsnorm_bwd_add(dy, x, gamma, rstd, dx, dgamma, scratch, rows, cols, zero_centered, accumulate_dgamma, dtype, nullptr, s);
}

// dx = d(rmsnorm)/dx applied to dy, plus ``addend`` when given (the gradient that reaches x without passing the norm)
MSB_API int msb_rmsnorm_bwd_add(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx, void* dgamma,
                                float* scratch, int rows, int cols, int zero_centered, int accumulate_dgamma, int dtype,
                                const void* addend, cudaStream_t s) {
  if (rows == 0) return 0;
  const bool fast = (cols % 8 == 0) && cols <= FAST_MAX_COLS;
  MSB_REQUIRE(fast || addend == nullptr, "rmsnorm_bwd_add: an addend needs cols=%d to be a multiple of 8 and at most %d", cols, FAST_MAX_COLS);
  int grid = 1;
  MSB_DISPATCH_FLOAT(dtype, T, {
    if (fast) {
      grid = launch_bwd<T>(dy, x, gamma, rstd, dx, scratch, rows, cols, zero_centered, 0, s, addend);
      MSB_CHECK_LAUNCH("rmsnorm_bwd");
    } else {
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
  const int fit = MSB_NOALLOC_SCRATCH_FLOATS / cols;  // >= 64 because cols <= 8192
  // every one of the grid*cols partial sums is overwritten by the first kernel before the second reads it,
  // so nothing left over from an earlier call needs clearing
  MSB_DISPATCH_FLOAT(dtype, T, {
    const int grid = launch_bwd<T>(dy, x, gamma, rstd, dx, scratch, rows, cols, zero_centered, fit, s);
    MSB_CHECK_LAUNCH("rmsnorm_bwd_noalloc");
    colsum_partials_kernel<T><<<(cols + 255) / 256, 256, 0, s>>>(scratch, (T*)dgamma, grid, cols, accumulate_dgamma);
    MSB_CHECK_LAUNCH("rmsnorm_bwd_noalloc_reduce");
  });
  return 0;
}
