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
