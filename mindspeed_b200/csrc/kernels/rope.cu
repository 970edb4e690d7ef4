// Rotary position embedding, forward and backward, in place or out of place, on strided heads.
//
// Tensor view: tokens x heads x head_dim, where token t starts at x + t*token_stride and
// head h at + h*head_stride.  Heads are grouped: of every `group_heads` consecutive heads only the
// first `rope_heads` are rotated (packed QKV layout [groups][q..q k v]: rotate q and k, skip v).
// cos/sin: fp32 [positions, rot_dim]; token t uses row (t / tokens_per_pos) (tokens of one sequence
// position are the batch entries in the [s, b, ...] layout).
//   mode 0 (half):        out[j] = x[j]*cos[j] - x[j+h]*sin[j];  out[j+h] = x[j+h]*cos[j+h] + x[j]*sin[j+h]
//   mode 1 (interleaved): pairs (2j, 2j+1)
// backward = same rotation with sin negated.
// reference semantics: npu_rotary_position_embedding(x, cos, sin, mode) (mindspeed/ops/csrc/cann/npu_rotary_position_embedding.cpp:113-143,
// mindspeed/core/fusions/fused_rope.py:28-74).
#include "msb_common.cuh"
using namespace msb;

namespace {
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ cosv,
                            const float* __restrict__ sinv, long long tokens, int heads, int head_dim, int rot_dim,
                            long long token_stride_in, long long head_stride_in, long long token_stride_out,
                            long long head_stride_out, int tokens_per_pos, int group_heads, int rope_heads, int mode,
                            float sin_sign) {
  const int half = rot_dim >> 1;
  const long long work = tokens * heads;
  for (long long w = (long long)blockIdx.x * blockDim.y + threadIdx.y; w < work; w += (long long)gridDim.x * blockDim.y) {
    long long t = w / heads;
    int h = (int)(w - t * heads);
    const bool rotate = (h % group_heads) < rope_heads;
    const T* xi = x + t * token_stride_in + (long long)h * head_stride_in;
    T* yo = y + t * token_stride_out + (long long)h * head_stride_out;
    if (!rotate) {
      if (xi != yo) for (int j = threadIdx.x; j < head_dim; j += blockDim.x) yo[j] = xi[j];
      continue;
    }
    const float* c = cosv + (t / tokens_per_pos) * rot_dim;
    const float* sn = sinv + (t / tokens_per_pos) * rot_dim;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      int i0 = mode == 0 ? j : 2 * j;
      int i1 = mode == 0 ? j + half : 2 * j + 1;
      float a = to_f(xi[i0]), b = to_f(xi[i1]);
      float o0 = a * c[i0] - b * sn[i0] * sin_sign;
      float o1 = b * c[i1] + a * sn[i1] * sin_sign;
      yo[i0] = from_f<T>(o0);
      yo[i1] = from_f<T>(o1);
    }
    if (xi != yo) for (int j = rot_dim + threadIdx.x; j < head_dim; j += blockDim.x) yo[j] = xi[j];
  }
}
// Vector path: bf16, half-split layout (mode 0), the whole head rotated.  One thread handles 8 consecutive elements of
// the first half of a head and their 8 partners in the second half (two 16-byte loads, two 16-byte stores).
__global__ void __launch_bounds__(256) rope_bf16_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                             const float* __restrict__ cosv, const float* __restrict__ sinv, long long tokens,
                                                             int heads, int head_dim, long long token_stride_in, long long head_stride_in,
                                                             long long token_stride_out, long long head_stride_out, int tokens_per_pos,
                                                             int group_heads, int rope_heads, float sin_sign) {
  const int half = head_dim >> 1;
  const int vec_per_head = half >> 3;
  const long long total = tokens * heads * vec_per_head;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(idx % vec_per_head) << 3;
    const long long th = idx / vec_per_head;
    const int h = (int)(th % heads);
    const long long t = th / heads;
    const __nv_bfloat16* xi = x + t * token_stride_in + (long long)h * head_stride_in;
    __nv_bfloat16* yo = y + t * token_stride_out + (long long)h * head_stride_out;
    const uint4 va = *reinterpret_cast<const uint4*>(xi + j);
    const uint4 vb = *reinterpret_cast<const uint4*>(xi + j + half);
    if ((h % group_heads) >= rope_heads) {
      if (xi != yo) { *reinterpret_cast<uint4*>(yo + j) = va; *reinterpret_cast<uint4*>(yo + j + half) = vb; }
      continue;
    }
    const float* c = cosv + (t / tokens_per_pos) * head_dim;
    const float* sn = sinv + (t / tokens_per_pos) * head_dim;
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&va);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&vb);
    uint4 oa, ob;
    __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
    __nv_bfloat162* qb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 a = __bfloat1622float2(pa[q]), b = __bfloat1622float2(pb[q]);
      const float2 c0 = *reinterpret_cast<const float2*>(c + j + 2 * q), s0 = *reinterpret_cast<const float2*>(sn + j + 2 * q);
      const float2 c1 = *reinterpret_cast<const float2*>(c + j + half + 2 * q), s1 = *reinterpret_cast<const float2*>(sn + j + half + 2 * q);
      qa[q] = __floats2bfloat162_rn(a.x * c0.x - b.x * s0.x * sin_sign, a.y * c0.y - b.y * s0.y * sin_sign);
      qb[q] = __floats2bfloat162_rn(b.x * c1.x + a.x * s1.x * sin_sign, b.y * c1.y + a.y * s1.y * sin_sign);
    }
    *reinterpret_cast<uint4*>(yo + j) = oa;
    *reinterpret_cast<uint4*>(yo + j + half) = ob;
  }
}

// Token-major vector path (head_dim / 16 a power of two): a block walks tokens, a thread owns one (head, 8-element slot)
// of the token, so the per-element index arithmetic is a shift and a mask, the position row is found once per token,
// and TOK tokens are loaded before any of them is rotated (2 * TOK 16-byte loads in flight per thread).
template <int TOK>
__global__ void __launch_bounds__(512, 2) rope_bf16_token_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, const float* __restrict__ cosv,
                                                               const float* __restrict__ sinv, long long tokens, int heads, int head_dim,
                                                               long long token_stride_in, long long head_stride_in,
                                                               long long token_stride_out, long long head_stride_out, int tokens_per_pos,
                                                               int group_heads, int rope_heads, float sin_sign, int vec_shift) {
  const int half = head_dim >> 1;
  const int per_token = heads << vec_shift;
  const bool in_place = (x == y) && token_stride_in == token_stride_out && head_stride_in == head_stride_out;
  for (long long t0 = (long long)blockIdx.x * TOK; t0 < tokens; t0 += (long long)gridDim.x * TOK) {
    for (int i = threadIdx.x; i < per_token; i += blockDim.x) {
      const int h = i >> vec_shift;
      const int j = (i & ((1 << vec_shift) - 1)) << 3;
      const bool rotate = (h % group_heads) < rope_heads;
      if (!rotate && in_place) continue;
      uint4 va[TOK], vb[TOK];
#pragma unroll
      for (int u = 0; u < TOK; ++u) {
        if (t0 + u < tokens) {
          const __nv_bfloat16* xi = x + (t0 + u) * token_stride_in + (long long)h * head_stride_in;
          va[u] = *reinterpret_cast<const uint4*>(xi + j);
          vb[u] = *reinterpret_cast<const uint4*>(xi + j + half);
        }
      }
#pragma unroll
      for (int u = 0; u < TOK; ++u) {
        if (t0 + u >= tokens) break;
        __nv_bfloat16* yo = y + (t0 + u) * token_stride_out + (long long)h * head_stride_out;
        if (!rotate) {
          *reinterpret_cast<uint4*>(yo + j) = va[u];
          *reinterpret_cast<uint4*>(yo + j + half) = vb[u];
          continue;
        }
        const long long pos = (t0 + u) / tokens_per_pos;
        const float4* c0 = reinterpret_cast<const float4*>(cosv + pos * head_dim + j);
        const float4* s0 = reinterpret_cast<const float4*>(sinv + pos * head_dim + j);
        const float4* c1 = reinterpret_cast<const float4*>(cosv + pos * head_dim + j + half);
        const float4* s1 = reinterpret_cast<const float4*>(sinv + pos * head_dim + j + half);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&va[u]);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&vb[u]);
        uint4 oa, ob;
        __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
        __nv_bfloat162* qb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
        for (int q = 0; q < 2; ++q) {       // four elements of each half per pass: keeps the live cos / sin values at 16
          const float4 ca = __ldg(c0 + q), sa = __ldg(s0 + q), cb = __ldg(c1 + q), sb = __ldg(s1 + q);
          const float2 a0 = __bfloat1622float2(pa[2 * q]), a1 = __bfloat1622float2(pa[2 * q + 1]);
          const float2 b0 = __bfloat1622float2(pb[2 * q]), b1 = __bfloat1622float2(pb[2 * q + 1]);
          qa[2 * q] = __floats2bfloat162_rn(a0.x * ca.x - b0.x * sa.x * sin_sign, a0.y * ca.y - b0.y * sa.y * sin_sign);
          qa[2 * q + 1] = __floats2bfloat162_rn(a1.x * ca.z - b1.x * sa.z * sin_sign, a1.y * ca.w - b1.y * sa.w * sin_sign);
          qb[2 * q] = __floats2bfloat162_rn(b0.x * cb.x + a0.x * sb.x * sin_sign, b0.y * cb.y + a0.y * sb.y * sin_sign);
          qb[2 * q + 1] = __floats2bfloat162_rn(b1.x * cb.z + a1.x * sb.z * sin_sign, b1.y * cb.w + a1.y * sb.w * sin_sign);
        }
        *reinterpret_cast<uint4*>(yo + j) = oa;
        *reinterpret_cast<uint4*>(yo + j + half) = ob;
      }
    }
  }
}
}  // namespace

MSB_API int msb_rope(const void* x, void* y, const float* cosv, const float* sinv, long long tokens, int heads,
                     int head_dim, int rot_dim, long long token_stride_in, long long head_stride_in,
                     long long token_stride_out, long long head_stride_out, int tokens_per_pos, int group_heads,
                     int rope_heads, int mode, int backward, int dtype, cudaStream_t s) {
  if (tokens == 0 || heads == 0) return 0;
  MSB_REQUIRE(rot_dim % 2 == 0 && rot_dim <= head_dim, "rope: bad rot_dim %d for head_dim %d", rot_dim, head_dim);
  const bool vec_ok = dtype == MSB_BF16 && mode == 0 && rot_dim == head_dim && head_dim % 16 == 0 && token_stride_in % 8 == 0 &&
                      head_stride_in % 8 == 0 && token_stride_out % 8 == 0 && head_stride_out % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(cosv) & 7) == 0 && (reinterpret_cast<uintptr_t>(sinv) & 7) == 0;
  const int vph = head_dim / 16;
  const bool cs16 = (reinterpret_cast<uintptr_t>(cosv) & 15) == 0 && (reinterpret_cast<uintptr_t>(sinv) & 15) == 0;
  if (vec_ok && cs16 && vph > 0 && (vph & (vph - 1)) == 0 && (long long)heads * vph <= (1 << 20)) {
    int shift = 0;
    while ((1 << shift) < vph) ++shift;
    constexpr int TOK = 2;
    const int per_token = heads * vph;
    int th = ((per_token + 31) / 32) * 32;
    if (th > 512) th = 512;
    long long gv = (tokens + TOK - 1) / TOK;
    const long long cap = (long long)msb::num_sms() * (th > 256 ? 2 : 4);   // resident blocks at <= 64 registers
    if (gv > cap) gv = cap;
    rope_bf16_token_kernel<TOK><<<(int)gv, th, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, cosv, sinv, tokens, heads, head_dim,
                                                       token_stride_in, head_stride_in, token_stride_out, head_stride_out,
                                                       tokens_per_pos, group_heads, rope_heads, backward ? -1.f : 1.f, shift);
    MSB_CHECK_LAUNCH("rope_bf16_token");
    return 0;
  }
  if (vec_ok) {
    const long long total = tokens * heads * (head_dim / 16);
    long long gv = (total + 255) / 256;
    const long long cap = (long long)msb::num_sms() * 16;
    if (gv > cap) gv = cap;
    rope_bf16_vec_kernel<<<(int)gv, 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, cosv, sinv, tokens, heads, head_dim,
                                                 token_stride_in, head_stride_in, token_stride_out, head_stride_out, tokens_per_pos,
                                                 group_heads, rope_heads, backward ? -1.f : 1.f);
    MSB_CHECK_LAUNCH("rope_bf16_vec");
    return 0;
  }
  dim3 block(32, 8);
  long long work = tokens * heads;
  long long g = (work + block.y - 1) / block.y;
  int grid = (int)(g > (long long)msb::num_sms() * 32 ? (long long)msb::num_sms() * 32 : g);
  MSB_DISPATCH_FLOAT(dtype, T, rope_kernel<T><<<grid, block, 0, s>>>((const T*)x, (T*)y, cosv, sinv, tokens, heads, head_dim, rot_dim,
      token_stride_in, head_stride_in, token_stride_out, head_stride_out, tokens_per_pos, group_heads, rope_heads, mode,
      backward ? -1.f : 1.f));
  MSB_CHECK_LAUNCH("rope");
  return 0;
}
