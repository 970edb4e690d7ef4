// Vocabulary-parallel cross entropy, local pieces.
//
// phase 1 (msb_ce_stats): per row of the local vocabulary slice, one pass with an online
//   (max, sum-exp) pair per thread: writes local max, sum exp(x - local max) and the target logit
//   (0 when the target is outside this rank's slice).
// between the phases the host all-reduces max (MAX) and rescales / all-reduces the sums
//   (reference: mindspeed/core/tensor_parallel/cross_entropy.py:6-38 — three small reductions).
// phase 2 (msb_ce_grad): dlogits = (exp(x - gmax)/gsum - onehot(target)) * g[row], written
//   IN PLACE over the logits in their own dtype, so no fp32 copy of the [tokens, vocab] matrix exists.
#include "msb_common.cuh"
using namespace msb;

namespace {
template <typename T>
__global__ void __launch_bounds__(512) ce_stats_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
                                                       float* __restrict__ row_max, float* __restrict__ row_sum,
                                                       float* __restrict__ picked, int vocab_local, long long vocab_start,
                                                       long long ignore_index) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const T* lr = logits + row * (size_t)vocab_local;
  float mx = -INFINITY, sm = 0.f;
  const bool vec_ok = (vocab_local % 8 == 0) && ((reinterpret_cast<uintptr_t>(lr) & 15) == 0);
  if (vec_ok) {
    const int nv = vocab_local >> 3;
    for (int v = threadIdx.x; v < nv; v += blockDim.x) {
      Vec8<T> t; t.load(lr + v * 8);
      float f[8]; t.to_float(f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      if (lm > mx) { sm *= __expf(mx - lm); mx = lm; }
#pragma unroll
      for (int j = 0; j < 8; ++j) sm += __expf(f[j] - mx);
    }
  } else {
    for (int c = threadIdx.x; c < vocab_local; c += blockDim.x) {
      float f = to_f(lr[c]);
      if (f > mx) { sm *= __expf(mx - f); mx = f; }
      sm += __expf(f - mx);
    }
  }
  const float gmx = block_max(mx, red);
  const float scaled = (mx == -INFINITY) ? 0.f : sm * __expf(mx - gmx);
  const float tot = block_sum(scaled, red);
  if (threadIdx.x == 0) {
    row_max[row] = gmx;
    row_sum[row] = tot;
    long long t = target[row] - vocab_start;
    float pk = 0.f;
    if (target[row] != ignore_index && t >= 0 && t < vocab_local) pk = to_f(lr[t]);
    picked[row] = pk;
  }
}

template <typename T>
__global__ void __launch_bounds__(512) ce_grad_kernel(T* __restrict__ logits, const long long* __restrict__ target,
                                                      const float* __restrict__ gmax, const float* __restrict__ gsum,
                                                      const float* __restrict__ gout, int vocab_local,
                                                      long long vocab_start, long long ignore_index) {
  const size_t row = blockIdx.x;
  T* lr = logits + row * (size_t)vocab_local;
  const float mx = gmax[row], inv = 1.f / gsum[row];
  const long long tg = target[row];
  const float g = (tg == ignore_index) ? 0.f : gout[row];
  const long long t = tg - vocab_start;
  const bool vec_ok = (vocab_local % 8 == 0) && ((reinterpret_cast<uintptr_t>(lr) & 15) == 0);
  if (vec_ok) {
    const int nv = vocab_local >> 3;
    for (int v = threadIdx.x; v < nv; v += blockDim.x) {
      Vec8<T> x; x.load(lr + v * 8);
      float f[8]; x.to_float(f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float pr = __expf(f[j] - mx) * inv;
        if ((long long)(v * 8 + j) == t) pr -= 1.f;
        f[j] = pr * g;
      }
      x.from_float(f); x.store(lr + v * 8);
    }
  } else {
    for (int c = threadIdx.x; c < vocab_local; c += blockDim.x) {
      float pr = __expf(to_f(lr[c]) - mx) * inv;
      if ((long long)c == t) pr -= 1.f;
      lr[c] = from_f<T>(pr * g);
    }
  }
}

// loss[row] = log(gsum) + gmax - picked  (0 for ignored rows)
__global__ void ce_loss_kernel(const float* gmax, const float* gsum, const float* picked, const long long* target,
                               float* loss, long long rows, long long ignore_index) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows) loss[i] = (target[i] == ignore_index) ? 0.f : __logf(gsum[i]) + gmax[i] - picked[i];
}
// sum[row] *= exp(local_max - global_max)
__global__ void ce_rescale_kernel(float* sum, const float* local_max, const float* global_max, long long rows) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows) sum[i] *= __expf(local_max[i] - global_max[i]);
}
}  // namespace

MSB_API int msb_ce_stats(const void* logits, const long long* target, float* row_max, float* row_sum, float* picked,
                         long long rows, int vocab_local, long long vocab_start, long long ignore_index, int dtype,
                         cudaStream_t s) {
  if (rows == 0) return 0;
  MSB_DISPATCH_FLOAT(dtype, T, ce_stats_kernel<T><<<(unsigned)rows, 512, 0, s>>>((const T*)logits, target, row_max, row_sum, picked,
                                                                              vocab_local, vocab_start, ignore_index));
  MSB_CHECK_LAUNCH("ce_stats");
  return 0;
}
MSB_API int msb_ce_rescale(float* sum, const float* local_max, const float* global_max, long long rows, cudaStream_t s) {
  if (rows == 0) return 0;
  ce_rescale_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, s>>>(sum, local_max, global_max, rows);
  MSB_CHECK_LAUNCH("ce_rescale");
  return 0;
}
MSB_API int msb_ce_loss(const float* gmax, const float* gsum, const float* picked, const long long* target, float* loss,
                        long long rows, long long ignore_index, cudaStream_t s) {
  if (rows == 0) return 0;
  ce_loss_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, s>>>(gmax, gsum, picked, target, loss, rows, ignore_index);
  MSB_CHECK_LAUNCH("ce_loss");
  return 0;
}
MSB_API int msb_ce_grad(void* logits, const long long* target, const float* gmax, const float* gsum, const float* gout,
                        long long rows, int vocab_local, long long vocab_start, long long ignore_index, int dtype,
                        cudaStream_t s) {
  if (rows == 0) return 0;
  MSB_DISPATCH_FLOAT(dtype, T, ce_grad_kernel<T><<<(unsigned)rows, 512, 0, s>>>((T*)logits, target, gmax, gsum, gout, vocab_local,
                                                                             vocab_start, ignore_index));
  MSB_CHECK_LAUNCH("ce_grad");
  return 0;
}
