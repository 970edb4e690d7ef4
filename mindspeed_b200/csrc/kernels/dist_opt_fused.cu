// Distributed-optimizer step as ONE peer-memory kernel: gradient reduce-scatter + scale (+ clip) + sharded AdamW +
// parameter all-gather, for a data-parallel group inside one NVSwitch domain.
//
// Every rank keeps its full gradient bucket (fp32 or bf16) and its full bf16 parameter bucket in a symmetric heap.
// Rank r owns elements [r*n, (r+1)*n) of the bucket ("the shard") and holds fp32 master weights and Adam moments for
// it.  For each 4-element vector of its shard a thread
//     pulls the vector from every peer's gradient bucket (plain ld.global.cg over NVLink), adds them in rank order in
//     fp32 and multiplies by grad_scale (1 / number of micro-batches x data-parallel size) [reduce-scatter + scale],
//     optionally accumulates the squared sum [gradient norm] and stores the reduced vector locally,
//     applies AdamW to master / m / v [optimizer],
//     rounds the new weights to bf16 and stores them into every peer's parameter bucket [all-gather]
// so gradients cross NVLink once, parameters once, and nothing is staged through NCCL buffers.  Modes:
//     pull + adam + push          the whole step in one launch (no gradient clipping)
//     pull + norm (no adam)       first pass when clipping is on: reduced shard + its squared norm
//     local + adam + push         second pass: reads the reduced shard, applies the clip coefficient from device memory
// Synchronisation: entry handshake (every peer has finished writing its gradients / reading its parameters), exit flag
// after the last CTA's pushes are visible; ``msb_dist_opt_wait_params`` is the bounded wait the next forward needs
// before it reads the parameter bucket.  Results are deterministic (fixed summation order).
// reference semantics being fused: the reduce-scatter of mindspeed/core/distributed/param_and_grad_buffer.py:57-239, the
// sharded Adam of the distributed optimizer and its parameter all-gather.
#include "msb_common.cuh"
#include "msb_sm100.cuh"

namespace {

constexpr int DO_MAX_RANKS = 8;
constexpr int DO_FLAG_BASE = 1024;   // u32 index inside the heap flag block: [+0,+8) entry, [+8,+16) exit, +16 counter

struct DistOptParams {
  const void* peer_grad[DO_MAX_RANKS];   // every rank's gradient bucket base
  void* peer_param[DO_MAX_RANKS];        // every rank's bf16 parameter bucket base
  float* reduced;                        // local [n] reduced gradients (written in pull mode when non-null, read in local mode)
  float* master; float* m; float* v;     // local [n]
  float* sumsq;                          // one float, atomically accumulated (may be null)
  const float* clip_coef;                // device scalar multiplied into the gradient before Adam (may be null)
  const float* found_inf;                // device scalar: non-zero skips the update (may be null)
  long long n;                           // shard elements (multiple of 4)
  long long shard_offset;                // first bucket element of this rank's shard
  float grad_scale, lr, beta1, beta2, eps, wd, bc1, bc2_sqrt;
  int world, rank, grad_is_bf16, pull, do_adam, push;
  unsigned int epoch;
  unsigned int* flag_local;
  unsigned int* flag_peer[DO_MAX_RANKS];
  unsigned int* status;
  unsigned long long limit_ns;
};

__device__ __forceinline__ float4 ld_grad4(const void* base, long long idx, int is_bf16) {
  if (is_bf16) {
    uint2 raw;
    const uint2* p = reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + idx);
    asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(raw.x), "=r"(raw.y) : "l"(p));
    const float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  float4 v;
  const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ bool do_wait_flag(const unsigned int* flag, unsigned int value, unsigned int* status, unsigned int code,
                                             unsigned long long limit_ns) {
  const uint64_t t0 = msb::sm100::globaltimer_ns();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int)(v - value) >= 0) return true;
    if (msb::sm100::globaltimer_ns() - t0 > limit_ns) { atomicCAS(status, 0u, code); return false; }
    if (*((volatile unsigned int*)status) != 0u) return false;
    __nanosleep(200);
  }
}

__global__ void __launch_bounds__(256) dist_opt_fused_kernel(const DistOptParams p) {
  __shared__ float red[32];
  __shared__ unsigned int is_last;
  bool alive = true;
  if (p.world > 1 && (p.pull || p.push)) {
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
      __threadfence_system();
      unsigned int* dst = p.flag_peer[threadIdx.x] + DO_FLAG_BASE + p.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(p.epoch) : "memory");
    }
    if (threadIdx.x < p.world) alive = do_wait_flag(p.flag_local + DO_FLAG_BASE + threadIdx.x, p.epoch, p.status, 0x500u + threadIdx.x, p.limit_ns);
    alive = __syncthreads_and(alive);
  }
  float local_sq = 0.f;
  const bool skip = p.found_inf && *p.found_inf != 0.f;
  if (alive) {
    const float clip = p.clip_coef ? *p.clip_coef : 1.f;
    const long long nv = p.n >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
      const long long e = i << 2;
      float4 g;
      if (p.pull) {
        g = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < p.world; ++r) {
          const float4 t = ld_grad4(p.peer_grad[r], p.shard_offset + e, p.grad_is_bf16);
          g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
        }
        g.x *= p.grad_scale; g.y *= p.grad_scale; g.z *= p.grad_scale; g.w *= p.grad_scale;
        if (p.reduced) *reinterpret_cast<float4*>(p.reduced + e) = g;
      } else {
        g = *reinterpret_cast<const float4*>(p.reduced + e);
      }
      local_sq += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
      if (p.do_adam && !skip) {
        float4 w = *reinterpret_cast<float4*>(p.master + e);
        float4 mm = *reinterpret_cast<float4*>(p.m + e);
        float4 vv = *reinterpret_cast<float4*>(p.v + e);
        auto upd = [&](float& pf, float gf, float& mf, float& vf) {
          gf *= clip;
          mf = p.beta1 * mf + (1.f - p.beta1) * gf;
          vf = p.beta2 * vf + (1.f - p.beta2) * gf * gf;
          const float step = (mf / p.bc1) / (sqrtf(vf) / p.bc2_sqrt + p.eps);
          pf = pf * (1.f - p.lr * p.wd) - p.lr * step;
        };
        upd(w.x, g.x, mm.x, vv.x); upd(w.y, g.y, mm.y, vv.y); upd(w.z, g.z, mm.z, vv.z); upd(w.w, g.w, mm.w, vv.w);
        *reinterpret_cast<float4*>(p.master + e) = w;
        *reinterpret_cast<float4*>(p.m + e) = mm;
        *reinterpret_cast<float4*>(p.v + e) = vv;
        __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
        uint2 packed = make_uint2(*reinterpret_cast<unsigned int*>(&lo), *reinterpret_cast<unsigned int*>(&hi));
        if (p.push) {
          for (int r = 0; r < p.world; ++r)
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.peer_param[r]) + p.shard_offset + e) = packed;
        } else {
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.peer_param[p.rank]) + p.shard_offset + e) = packed;
        }
      }
    }
  }
  if (p.sumsq) {
    const float s = msb::block_sum(local_sq, red);
    if (threadIdx.x == 0 && s != 0.f) atomicAdd(p.sumsq, s);
  }
  // exit: the last CTA tells every peer that this rank's pushes (and its reads of their gradients) are complete
  if (p.world > 1 && (p.pull || p.push)) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int prev = atomicAdd(p.flag_local + DO_FLAG_BASE + 16, 1u);
      is_last = (prev == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (is_last && threadIdx.x < p.world) {
      if (threadIdx.x == 0) p.flag_local[DO_FLAG_BASE + 16] = 0u;
      __threadfence_system();
      unsigned int* dst = p.flag_peer[threadIdx.x] + DO_FLAG_BASE + 8 + p.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(p.epoch) : "memory");
    }
  }
}

__global__ void dist_opt_wait_kernel(const unsigned int* flag_local, unsigned int epoch, int world, unsigned int* status,
                                     unsigned long long limit_ns) {
  if (threadIdx.x < world) do_wait_flag(flag_local + DO_FLAG_BASE + 8 + threadIdx.x, epoch, status, 0x520u + threadIdx.x, limit_ns);
}

}  // namespace

struct MsbDistOptArgs {
  const void* peer_grad[8];
  void* peer_param[8];
  float* reduced; float* master; float* m; float* v; float* sumsq;
  const float* clip_coef; const float* found_inf;
  long long n; long long shard_offset;
  float grad_scale, lr, beta1, beta2, eps, wd;
  int step, world, rank, grad_is_bf16, pull, do_adam, push;
  unsigned int epoch;
  unsigned int* flag_local;
  unsigned int* flag_peer[8];
  unsigned int* status;
  int wait_limit_ms;
};

MSB_API int msb_dist_opt_fused(const MsbDistOptArgs* a, cudaStream_t s) {
  MSB_REQUIRE(a != nullptr, "dist_opt_fused: null arguments");
  MSB_REQUIRE(a->world >= 1 && a->world <= DO_MAX_RANKS && a->rank >= 0 && a->rank < a->world, "dist_opt_fused: bad world/rank %d/%d", a->world, a->rank);
  MSB_REQUIRE(a->n >= 0 && a->n % 4 == 0 && a->shard_offset % 4 == 0, "dist_opt_fused: shard size %lld and offset %lld must be multiples of 4", a->n, a->shard_offset);
  MSB_REQUIRE(a->status && a->flag_local, "dist_opt_fused: status word and flags are required");
  MSB_REQUIRE(a->pull || a->reduced, "dist_opt_fused: local mode needs the reduced-gradient buffer");
  MSB_REQUIRE(!a->do_adam || (a->master && a->m && a->v && a->step >= 1), "dist_opt_fused: Adam needs master / m / v and step >= 1");
  DistOptParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < DO_MAX_RANKS; ++i) {
    p.peer_grad[i] = a->peer_grad[i]; p.peer_param[i] = a->peer_param[i]; p.flag_peer[i] = a->flag_peer[i];
    if (i < a->world) {
      MSB_REQUIRE(!a->pull || a->peer_grad[i], "dist_opt_fused: missing gradient pointer of rank %d", i);
      MSB_REQUIRE(!(a->do_adam && (a->push || i == a->rank)) || a->peer_param[i], "dist_opt_fused: missing parameter pointer of rank %d", i);
      MSB_REQUIRE(a->world == 1 || a->flag_peer[i], "dist_opt_fused: missing flags of rank %d", i);
    }
  }
  p.reduced = a->reduced; p.master = a->master; p.m = a->m; p.v = a->v; p.sumsq = a->sumsq;
  p.clip_coef = a->clip_coef; p.found_inf = a->found_inf; p.n = a->n; p.shard_offset = a->shard_offset;
  p.grad_scale = a->grad_scale; p.lr = a->lr; p.beta1 = a->beta1; p.beta2 = a->beta2; p.eps = a->eps; p.wd = a->wd;
  p.bc1 = 1.f - powf(a->beta1, (float)(a->step > 0 ? a->step : 1));
  p.bc2_sqrt = sqrtf(1.f - powf(a->beta2, (float)(a->step > 0 ? a->step : 1)));
  p.world = a->world; p.rank = a->rank; p.grad_is_bf16 = a->grad_is_bf16; p.pull = a->pull; p.do_adam = a->do_adam; p.push = a->push;
  p.epoch = a->epoch; p.flag_local = a->flag_local; p.status = a->status;
  p.limit_ns = (a->wait_limit_ms > 0 ? (unsigned long long)a->wait_limit_ms : 10000ull) * 1000000ull;
  long long g = (a->n / 4 + 255) / 256;
  const long long cap = (long long)msb::num_sms() * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  dist_opt_fused_kernel<<<(int)g, 256, 0, s>>>(p);
  MSB_CHECK_LAUNCH("dist_opt_fused");
  return 0;
}

// Bounded wait until every peer's exit flag of ``epoch`` has arrived (its parameter pushes into this GPU are visible).
MSB_API int msb_dist_opt_wait_params(const unsigned int* flag_local, unsigned int epoch, int world, unsigned int* status,
                                     int wait_limit_ms, cudaStream_t s) {
  MSB_REQUIRE(flag_local && status && world >= 1 && world <= DO_MAX_RANKS, "dist_opt_wait_params: bad arguments");
  dist_opt_wait_kernel<<<1, 32, 0, s>>>(flag_local, epoch, world, status,
                                        (wait_limit_ms > 0 ? (unsigned long long)wait_limit_ms : 10000ull) * 1000000ull);
  MSB_CHECK_LAUNCH("dist_opt_wait_params");
  return 0;
}
