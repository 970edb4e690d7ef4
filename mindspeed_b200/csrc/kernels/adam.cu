// Fused optimizer kernels on flat fp32 shards (the distributed optimizer owns contiguous slices).
//
// msb_adam_flat: grad unscale (x grad_scale: inverse loss scale times clip coefficient) + AdamW
//   (decoupled weight decay, bias correction) on fp32 master/m/v + cast of the new master to the
//   bf16/fp16 model parameter shard, one pass: reads g,p,m,v and writes p,m,v,param16.
//   Optional EMA of the master weights in the same pass (fused_ema_adamw).
// reference semantics: torch._fused_adamw_ driven by mindspeed/core/optimizer/adamw.py:23-62,96-189;
//   EMA variant mindspeed/ops/csrc/cann/npu_apply_fused_ema_adamw.cpp:49.
// msb_l2norm_sq: sum of squares of a flat buffer (for gradient clipping), deterministic two-stage.
#include "msb_common.cuh"
using namespace msb;

namespace {
template <typename G, typename P16>
__global__ void adam_flat_kernel(float* __restrict__ p, const G* __restrict__ g, float* __restrict__ m,
                                 float* __restrict__ v, P16* __restrict__ p16, float* __restrict__ ema, size_t n,
                                 float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2_sqrt,
                                 float grad_scale, float ema_decay, int adam_w_mode, int maximize,
                                 const float* __restrict__ found_inf, const float* __restrict__ grad_scale_dev) {
  if (found_inf && *found_inf != 0.f) return;
  if (grad_scale_dev) grad_scale *= *grad_scale_dev;
  const size_t nv = n >> 2;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  auto upd = [&](float& pf, float gf, float& mf, float& vf) {
    gf *= grad_scale;
    if (maximize) gf = -gf;
    if (!adam_w_mode) gf += wd * pf;
    mf = beta1 * mf + (1.f - beta1) * gf;
    vf = beta2 * vf + (1.f - beta2) * gf * gf;
    float denom = sqrtf(vf) / bc2_sqrt + eps;
    float step = (mf / bc1) / denom;
    if (adam_w_mode) pf = pf * (1.f - lr * wd) - lr * step; else pf = pf - lr * step;
  };
  for (size_t i = tid; i < nv; i += stride) {
    float4 pf = reinterpret_cast<float4*>(p)[i];
    float4 mf = reinterpret_cast<float4*>(m)[i];
    float4 vf = reinterpret_cast<float4*>(v)[i];
    float gf[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) gf[j] = to_f(g[i * 4 + j]);
    upd(pf.x, gf[0], mf.x, vf.x); upd(pf.y, gf[1], mf.y, vf.y); upd(pf.z, gf[2], mf.z, vf.z); upd(pf.w, gf[3], mf.w, vf.w);
    reinterpret_cast<float4*>(p)[i] = pf;
    reinterpret_cast<float4*>(m)[i] = mf;
    reinterpret_cast<float4*>(v)[i] = vf;
    if (p16) {
      p16[i * 4 + 0] = from_f<P16>(pf.x); p16[i * 4 + 1] = from_f<P16>(pf.y);
      p16[i * 4 + 2] = from_f<P16>(pf.z); p16[i * 4 + 3] = from_f<P16>(pf.w);
    }
    if (ema) {
      float4 e = reinterpret_cast<float4*>(ema)[i];
      e.x = ema_decay * e.x + (1.f - ema_decay) * pf.x; e.y = ema_decay * e.y + (1.f - ema_decay) * pf.y;
      e.z = ema_decay * e.z + (1.f - ema_decay) * pf.z; e.w = ema_decay * e.w + (1.f - ema_decay) * pf.w;
      reinterpret_cast<float4*>(ema)[i] = e;
    }
  }
  for (size_t i = (nv << 2) + tid; i < n; i += stride) {
    float pf = p[i], mf = m[i], vf = v[i];
    upd(pf, to_f(g[i]), mf, vf);
    p[i] = pf; m[i] = mf; v[i] = vf;
    if (p16) p16[i] = from_f<P16>(pf);
    if (ema) ema[i] = ema_decay * ema[i] + (1.f - ema_decay) * pf;
  }
}

// AdamW on a master weight stored as (bf16 model parameter, 16-bit residual): the fp32 master never exists in memory.
//   stored = bits(fp32) + 0x8000 (as integers);  hi = stored >> 16 is the bf16 parameter the model uses (round-half-up of
//   the master), lo = stored & 0xffff is the residual;  bits(fp32) = ((hi << 16) | lo) - 0x8000 recovers the master exactly.
// reference: mindspeed/optimizer/optimizer.py:249-280 (reuse-fp32-param: int32 add/sub of 32768 and a split in halves).
template <typename G>
__global__ void adam_flat_reuse_kernel(__nv_bfloat16* __restrict__ hi, unsigned short* __restrict__ lo, const G* __restrict__ g,
                                       float* __restrict__ m, float* __restrict__ v, size_t n, float lr, float beta1, float beta2,
                                       float eps, float wd, float bc1, float bc2_sqrt, float grad_scale, int adam_w_mode,
                                       const float* __restrict__ found_inf, const float* __restrict__ grad_scale_dev) {
  if (found_inf && *found_inf != 0.f) return;
  if (grad_scale_dev) grad_scale *= *grad_scale_dev;
  const unsigned short* hi_bits = reinterpret_cast<const unsigned short*>(hi);
  unsigned short* hi_out = reinterpret_cast<unsigned short*>(hi);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const unsigned int stored = ((unsigned int)hi_bits[i] << 16) | (unsigned int)lo[i];
    float pf = __uint_as_float(stored - 0x8000u);
    float gf = to_f(g[i]) * grad_scale;
    if (!adam_w_mode) gf += wd * pf;
    float mf = beta1 * m[i] + (1.f - beta1) * gf;
    float vf = beta2 * v[i] + (1.f - beta2) * gf * gf;
    const float step = (mf / bc1) / (sqrtf(vf) / bc2_sqrt + eps);
    pf = adam_w_mode ? pf * (1.f - lr * wd) - lr * step : pf - lr * step;
    m[i] = mf; v[i] = vf;
    const unsigned int out = __float_as_uint(pf) + 0x8000u;
    hi_out[i] = (unsigned short)(out >> 16);
    lo[i] = (unsigned short)(out & 0xffffu);
  }
}

template <typename G>
__global__ void l2norm_sq_partial(const G* __restrict__ g, size_t n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = to_f(g[i]); s += v * v;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void l2norm_sq_final(const float* __restrict__ partial, int n, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) *out = accumulate ? *out + s : s;
}

template <typename T>
__global__ void scale_kernel(T* __restrict__ x, size_t n, float scale, const float* __restrict__ scale_dev) {
  if (scale_dev) scale *= *scale_dev;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = from_f<T>(to_f(x[i]) * scale);
}

// clip coefficient on device: coef = min(1, max_norm / (sqrt(norm_sq) + 1e-6)); found_inf set if not finite
__global__ void clip_coef_kernel(const float* norm_sq, float max_norm, float* coef, float* found_inf, float* norm_out) {
  float nrm = sqrtf(*norm_sq);
  if (norm_out) *norm_out = nrm;
  bool bad = !(nrm == nrm) || isinf(nrm);
  if (found_inf) *found_inf = bad ? 1.f : 0.f;
  float c = max_norm > 0.f ? max_norm / (nrm + 1e-6f) : 1.f;
  *coef = c < 1.f ? c : 1.f;
}
}  // namespace

MSB_API int msb_adam_flat(float* p, const void* g, float* m, float* v, void* p16, float* ema, long long n, float lr,
                          float beta1, float beta2, float eps, float wd, int step, float grad_scale, float ema_decay,
                          int adam_w_mode, int maximize, int bias_correction, const float* found_inf,
                          const float* grad_scale_dev, int grad_dtype, int p16_dtype, cudaStream_t s) {
  if (n == 0) return 0;
  float bc1 = 1.f, bc2s = 1.f;
  if (bias_correction) { bc1 = 1.f - powf(beta1, (float)step); bc2s = sqrtf(1.f - powf(beta2, (float)step)); }
  int grid = (int)(((size_t)n / 4 + 255) / 256); if (grid < 1) grid = 1;
  if (grid > msb::num_sms() * 8) grid = msb::num_sms() * 8;
#define LAUNCH(G, P)                                                                                                   \
  adam_flat_kernel<G, P><<<grid, 256, 0, s>>>(p, (const G*)g, m, v, (P*)p16, ema, (size_t)n, lr, beta1, beta2, eps, wd, \
                                              bc1, bc2s, grad_scale, ema_decay, adam_w_mode, maximize, found_inf, grad_scale_dev)
  if (grad_dtype == MSB_F32) {
    if (p16_dtype == MSB_F16) LAUNCH(float, __half); else LAUNCH(float, __nv_bfloat16);
  } else if (grad_dtype == MSB_BF16) {
    if (p16_dtype == MSB_F16) LAUNCH(__nv_bfloat16, __half); else LAUNCH(__nv_bfloat16, __nv_bfloat16);
  } else {
    if (p16_dtype == MSB_F16) LAUNCH(__half, __half); else LAUNCH(__half, __nv_bfloat16);
  }
#undef LAUNCH
  MSB_CHECK_LAUNCH("adam_flat");
  return 0;
}

MSB_API int msb_l2norm_sq_scratch_elems() { return msb::num_sms() * 4; }

MSB_API int msb_l2norm_sq(const void* g, long long n, float* scratch, float* out, int accumulate, int dtype, cudaStream_t s) {
  int grid = msb::num_sms() * 4;
  MSB_DISPATCH_FLOAT(dtype, T, l2norm_sq_partial<T><<<grid, 512, 0, s>>>((const T*)g, (size_t)n, scratch));
  MSB_CHECK_LAUNCH("l2norm_sq_partial");
  l2norm_sq_final<<<1, 256, 0, s>>>(scratch, grid, out, accumulate);
  MSB_CHECK_LAUNCH("l2norm_sq_final");
  return 0;
}

MSB_API int msb_scale(void* x, long long n, float scale, const float* scale_dev, int dtype, cudaStream_t s) {
  if (n == 0) return 0;
  int grid = (int)(((size_t)n + 255) / 256); if (grid > msb::num_sms() * 8) grid = msb::num_sms() * 8;
  MSB_DISPATCH_FLOAT(dtype, T, scale_kernel<T><<<grid, 256, 0, s>>>((T*)x, (size_t)n, scale, scale_dev));
  MSB_CHECK_LAUNCH("scale");
  return 0;
}

MSB_API int msb_clip_coef(const float* norm_sq, float max_norm, float* coef, float* found_inf, float* norm_out, cudaStream_t s) {
  clip_coef_kernel<<<1, 1, 0, s>>>(norm_sq, max_norm, coef, found_inf, norm_out);
  MSB_CHECK_LAUNCH("clip_coef");
  return 0;
}

MSB_API int msb_adam_flat_reuse(void* hi, void* lo, const void* g, float* m, float* v, long long n, float lr, float beta1,
                                float beta2, float eps, float wd, int step, float grad_scale, int adam_w_mode, int bias_correction,
                                const float* found_inf, const float* grad_scale_dev, int grad_dtype, cudaStream_t s) {
  if (n == 0) return 0;
  float bc1 = 1.f, bc2s = 1.f;
  if (bias_correction) { bc1 = 1.f - powf(beta1, (float)step); bc2s = sqrtf(1.f - powf(beta2, (float)step)); }
  int grid = (int)(((size_t)n + 255) / 256); if (grid > msb::num_sms() * 16) grid = msb::num_sms() * 16;
  MSB_DISPATCH_FLOAT(grad_dtype, G, adam_flat_reuse_kernel<G><<<grid, 256, 0, s>>>((__nv_bfloat16*)hi, (unsigned short*)lo, (const G*)g, m, v,
      (size_t)n, lr, beta1, beta2, eps, wd, bc1, bc2s, grad_scale, adam_w_mode, found_inf, grad_scale_dev));
  MSB_CHECK_LAUNCH("adam_flat_reuse");
  return 0;
}
