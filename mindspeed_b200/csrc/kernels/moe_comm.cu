// MoE token dispatch and combine over NVLink peer memory (expert parallelism inside one NVSwitch domain).
//
// The library path is permute -> all-to-all-v -> regroup (three passes over the routed rows plus NCCL's staging).
// Here every rank stages its *unpermuted* hidden states once in a symmetric buffer and publishes a sorted token
// list; the expert owner then gathers exactly the rows it needs straight into the expert-sorted layout the
// grouped GEMM consumes ("dispatch").  The way back is the mirror image: the token owner pulls the (already
// probability-weighted) expert outputs of each of its tokens from the expert owners and sums them in fp32 in
// ascending expert order ("combine"), which makes the result run-to-run deterministic.  The backward of either
// kernel is the other one, so two kernels cover the four transfers of a training step.
//
// Synchronisation: both kernels start with an all-to-all epoch handshake on flag words of the symmetric heap (the
// same scheme as the fused GEMM kernels, on separate words).  A rank raises its flag on every peer after its own
// staging copies (earlier in stream order) are complete, and waits, with a time limit, until every peer has
// done the same.  Staging buffers alternate between two slots per call, and a slot is rewritten only after a
// later call's handshake has shown that every peer has left the call that read it, so no exit flags are needed.
// Peer memory is only ever *read* here (plain ld.global.cg vector loads); nothing in this file issues a TMA
// or multicast operation.
//
// reference semantics: mindspeed/core/transformer/moe/moe_feature/overlap/token_dispatcher.py:519-975 (all-to-all
// dispatcher) and the fused dispatch/combine vendor ops used by --moe-alltoall-mc2
// (mindspeed/ops/npu_moe_distribute_dispatch / npu_moe_distribute_combine wrappers).
#include "msb_common.cuh"
#include "msb_sm100.cuh"

namespace {

constexpr int MOE_MAX_RANKS = 8;
constexpr int MOE_FLAG_BASE = 32;   // u32 index of this family's entry flags inside the heap's flag block
constexpr int MOE_MAX_TOPK = 32;

struct MoeParams {
  void* out;                                 // dispatch: [R, H] rows ; combine: [T, H] rows
  float* out_probs;                          // dispatch: [R] ; combine: dense [T, E] (only routed entries written) ; may be null
  const void* peer_rows[MOE_MAX_RANKS];      // dispatch: peer's staged [T, H] ; combine: peer's staged [R_peer, H]
  const int* peer_tok[MOE_MAX_RANKS];        // dispatch: peer's token ids sorted by global expert
  const float* peer_probs[MOE_MAX_RANKS];    // dispatch: peer's sorted probabilities ; combine: peer's per-row values ; may be null
  const long long* chunk_dst_start;          // dispatch: [n_chunks + 1] first output row of chunk (local expert, source rank)
  const long long* chunk_src_start;          // dispatch: [n_chunks] offset of the chunk in the source's sorted list
  const unsigned char* map;                  // combine: [T, E] routing map
  const int* rank_in_expert;                 // combine: [T, E] position of token t among the tokens this rank sends to expert e
  const long long* dst_row_base;             // combine: [E] first row of this rank's chunk in the owner's layout
  long long R;
  long long row_cap;                         // combine: rows a peer's staged buffer can hold (bound for the computed row)
  int T, E, E_loc, row_v4, world, rank, n_chunks;
  unsigned int epoch;
  unsigned int* flag_local;
  unsigned int* flag_peer[MOE_MAX_RANKS];
  unsigned int* status;
  unsigned long long limit_ns;
};

__device__ __forceinline__ uint4 ld_peer_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ int ld_peer_s32(const int* p) {
  int v;
  asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_peer_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ bool moe_wait_flag(const unsigned int* flag, unsigned int value, unsigned int* status,
                                              unsigned int code, unsigned long long limit_ns) {
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

// Every CTA waits for all peers; CTA 0 announces this rank.  Returns false when a wait ran out.
__device__ __forceinline__ bool moe_entry_handshake(const MoeParams& p) {
  bool alive = true;
  if (p.world > 1) {
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
      __threadfence_system();
      unsigned int* dst = p.flag_peer[threadIdx.x] + MOE_FLAG_BASE + p.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(p.epoch) : "memory");
    }
    if (threadIdx.x < p.world)
      alive = moe_wait_flag(p.flag_local + MOE_FLAG_BASE + threadIdx.x, p.epoch, p.status, 0x300u + threadIdx.x, p.limit_ns);
    alive = __syncthreads_and(alive);
  }
  return alive;
}

// dispatch: one warp per output row.  Row r belongs to chunk c = (local expert, source rank) found by binary
// search over the chunk starts; the source's sorted token list gives the row of its staged hidden states.
__global__ void __launch_bounds__(256) moe_dispatch_kernel(const MoeParams p) {
  if (!moe_entry_handshake(p)) return;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarp = (long long)gridDim.x * (blockDim.x >> 5);
  uint4* out = reinterpret_cast<uint4*>(p.out);
  for (long long r = warp0; r < p.R; r += nwarp) {
    int lo = 0, hi = p.n_chunks;            // largest c with chunk_dst_start[c] <= r
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(p.chunk_dst_start + mid) <= r) lo = mid; else hi = mid;
    }
    const int c = lo;
    const int s = c % p.world;
    const long long i = __ldg(p.chunk_src_start + c) + (r - __ldg(p.chunk_dst_start + c));
    int t = 0;
    float pr = 0.f;
    if (lane == 0) {
      t = ld_peer_s32(p.peer_tok[s] + i);
      if (p.out_probs && p.peer_probs[s]) pr = ld_peer_f32(p.peer_probs[s] + i);
    }
    t = __shfl_sync(0xffffffffu, t, 0);
    if (t < 0 || t >= p.T) {               // corrupt index: record it and skip the access
      if (lane == 0) atomicCAS(p.status, 0u, 0x3f0u);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(p.peer_rows[s]) + (long long)t * p.row_v4;
    uint4* dst = out + r * p.row_v4;
    int j = lane;
    for (; j + 7 * 32 < p.row_v4; j += 8 * 32) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = ld_peer_v4(src + j + u * 32);
#pragma unroll
      for (int u = 0; u < 8; ++u) dst[j + u * 32] = v[u];
    }
    for (; j < p.row_v4; j += 32) dst[j] = ld_peer_v4(src + j);
    if (lane == 0 && p.out_probs) p.out_probs[r] = pr;
  }
}

// combine: one warp per token.  The routed experts of the token are listed in ascending order, their rows are
// pulled from the owners and added in fp32 in that order.
__global__ void __launch_bounds__(256) moe_combine_kernel(const MoeParams p) {
  if (!moe_entry_handshake(p)) return;
  __shared__ const uint4* s_rows[8][MOE_MAX_TOPK];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + wib;
  const long long nwarp = (long long)gridDim.x * (blockDim.x >> 5);
  uint4* out = reinterpret_cast<uint4*>(p.out);
  for (long long t = warp0; t < p.T; t += nwarp) {
    int cnt = 0;
    for (int e0 = 0; e0 < p.E; e0 += 32) {
      const int e = e0 + lane;
      const bool hit = e < p.E && p.map[t * p.E + e] != 0;
      const unsigned int m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int pos = cnt + __popc(m & ((1u << lane) - 1u));
        const int d = e / p.E_loc;
        const long long row = __ldg(p.dst_row_base + e) + p.rank_in_expert[t * p.E + e];
        const bool ok = row >= 0 && row < p.row_cap;
        if (!ok) atomicCAS(p.status, 0u, 0x3f2u);          // inconsistent tables: record it, read row 0 instead
        const long long rr = ok ? row : 0;
        if (pos < MOE_MAX_TOPK) s_rows[wib][pos] = reinterpret_cast<const uint4*>(p.peer_rows[d]) + rr * p.row_v4;
        if (p.out_probs && p.peer_probs[d]) p.out_probs[t * p.E + e] = ld_peer_f32(p.peer_probs[d] + rr);
      }
      cnt += __popc(m);
    }
    if (cnt > MOE_MAX_TOPK) {
      if (lane == 0) atomicCAS(p.status, 0u, 0x3f1u);
      cnt = MOE_MAX_TOPK;
    }
    __syncwarp();
    uint4* dst = out + t * p.row_v4;
    for (int j = lane; j < p.row_v4; j += 4 * 32) {
      float acc[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[u][q] = 0.f;
      for (int k = 0; k < cnt; ++k) {
        const uint4* src = s_rows[wib][k];
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = (j + u * 32 < p.row_v4) ? ld_peer_v4(src + j + u * 32) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
          for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(h[q]); acc[u][2 * q] += f.x; acc[u][2 * q + 1] += f.y; }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (j + u * 32 < p.row_v4) {
          uint4 o;
          __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int q = 0; q < 4; ++q) ho[q] = __floats2bfloat162_rn(acc[u][2 * q], acc[u][2 * q + 1]);
          dst[j + u * 32] = o;
        }
      }
    }
    __syncwarp();
  }
}

// Builds every index table of a dispatch / combine pair in one launch (replaces ~25 small tensor operations whose host
// launch cost dominated the layer): CTA e scans column e of the routing map and writes, for every routed token, its
// position among this rank's tokens for expert e, the token id and its probability into the sorted lists (directly in
// the staging slot the peers read); CTA 0 afterwards fills the chunk tables and the destination row bases from the
// all-gathered count matrix ``counts`` [ep, ld] (ld >= E, row s = source rank s).
template <typename PT>
__global__ void __launch_bounds__(1024) moe_build_plan_kernel(const unsigned char* __restrict__ map, const PT* __restrict__ probs,
                                                               const long long* __restrict__ counts, int ld, int T, int E, int E_loc, int ep,
                                                               int me, int* __restrict__ rank_in_expert, int* __restrict__ sorted_tok,
                                                               float* __restrict__ sorted_probs, long long* __restrict__ chunk_dst_start,
                                                               long long* __restrict__ chunk_src_start, long long* __restrict__ dst_row_base,
                                                               long long list_cap) {
  __shared__ int warp_tot[32];
  __shared__ long long s_src_off;
  __shared__ int s_running;
  const int e = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (tid == 0) {
    long long off = 0;
    for (int k = 0; k < e; ++k) off += counts[(long long)me * ld + k];
    s_src_off = off;
    s_running = 0;
  }
  __syncthreads();
  const long long src_off = s_src_off;
  for (int base = 0; base < T; base += blockDim.x) {
    const int t = base + tid;
    const int flag = (t < T && map[(long long)t * E + e] != 0) ? 1 : 0;
    int incl = flag;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
    if (lane == 31) warp_tot[wid] = incl;
    __syncthreads();
    if (wid == 0) {
      int v = (lane < (int)(blockDim.x >> 5)) ? warp_tot[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
      warp_tot[lane] = v;                       // inclusive prefix of the warp totals
    }
    __syncthreads();
    const int before = s_running + (wid ? warp_tot[wid - 1] : 0) + incl - flag;
    if (t < T) {
      rank_in_expert[(long long)t * E + e] = flag ? before : -1;
      if (flag) {
        const long long pos = src_off + before;
        if (pos < list_cap) {
          sorted_tok[pos] = t;
          sorted_probs[pos] = (float)probs[(long long)t * E + e];
        }
      }
    }
    __syncthreads();
    if (tid == 0) s_running += warp_tot[(blockDim.x >> 5) - 1];
    __syncthreads();
  }
  if (e != 0) return;
  // ---- tables from the count matrix ----
  const int n_chunks = E_loc * ep;
  const int lo = me * E_loc;
  for (int c = tid; c < n_chunks; c += blockDim.x) {          // chunk c = (local expert el, source rank s)
    const int el = c / ep, sr = c % ep;
    long long off = 0;
    for (int k = 0; k < lo + el; ++k) off += counts[(long long)sr * ld + k];
    chunk_src_start[c] = off;
  }
  for (int ee = tid; ee < E; ee += blockDim.x) {
    const int owner = ee / E_loc;
    long long first = 0;
    for (int k = owner * E_loc; k < ee; ++k)
      for (int sr = 0; sr < ep; ++sr) first += counts[(long long)sr * ld + k];
    for (int sr = 0; sr < me; ++sr) first += counts[(long long)sr * ld + ee];
    dst_row_base[ee] = first;
  }
  if (tid == 0) {
    long long acc = 0;
    for (int c = 0; c < n_chunks; ++c) {
      chunk_dst_start[c] = acc;
      acc += counts[(long long)(c % ep) * ld + lo + c / ep];
    }
    chunk_dst_start[n_chunks] = acc;
  }
}

}  // namespace

// Host-visible argument block (mirrored by a ctypes.Structure in mindspeed_b200/ops/moe_comm.py).
struct MsbMoeCommArgs {
  void* out;
  float* out_probs;
  const void* peer_rows[8];
  const int* peer_tok[8];
  const float* peer_probs[8];
  const long long* chunk_dst_start;
  const long long* chunk_src_start;
  const unsigned char* map;
  const int* rank_in_expert;
  const long long* dst_row_base;
  long long R;
  long long row_cap;
  int T, E, E_loc, row_bytes, world, rank, n_chunks;
  unsigned int epoch;
  unsigned int* flag_local;
  unsigned int* flag_peer[8];
  unsigned int* status;
  int wait_limit_ms;   // 0: default (10 s)
};

static int fill(MoeParams& p, const MsbMoeCommArgs* a, const char* what) {
  MSB_REQUIRE(a != nullptr, "%s: null argument block", what);
  MSB_REQUIRE(a->world >= 1 && a->world <= MOE_MAX_RANKS && a->rank >= 0 && a->rank < a->world, "%s: bad world/rank %d/%d", what, a->world, a->rank);
  MSB_REQUIRE(a->row_bytes > 0 && a->row_bytes % 16 == 0, "%s: row size %d bytes must be a multiple of 16", what, a->row_bytes);
  MSB_REQUIRE(a->status && a->flag_local, "%s: status word and flags are required", what);
  MSB_REQUIRE(a->out != nullptr || (a->R == 0 && a->T == 0), "%s: null output", what);
  MSB_REQUIRE(a->E > 0 && a->E_loc > 0 && a->E == a->E_loc * a->world, "%s: E=%d must equal E_loc=%d x world=%d", what, a->E, a->E_loc, a->world);
  p.out = a->out; p.out_probs = a->out_probs;
  for (int i = 0; i < MOE_MAX_RANKS; ++i) {
    p.peer_rows[i] = a->peer_rows[i]; p.peer_tok[i] = a->peer_tok[i]; p.peer_probs[i] = a->peer_probs[i];
    p.flag_peer[i] = a->flag_peer[i];
    if (i < a->world) MSB_REQUIRE(a->peer_rows[i] && a->flag_peer[i], "%s: missing pointers of peer %d", what, i);
  }
  p.chunk_dst_start = a->chunk_dst_start; p.chunk_src_start = a->chunk_src_start;
  p.map = a->map; p.rank_in_expert = a->rank_in_expert; p.dst_row_base = a->dst_row_base;
  p.R = a->R; p.row_cap = a->row_cap; p.T = a->T; p.E = a->E; p.E_loc = a->E_loc; p.row_v4 = a->row_bytes / 16;
  p.world = a->world; p.rank = a->rank; p.n_chunks = a->n_chunks; p.epoch = a->epoch;
  p.flag_local = a->flag_local; p.status = a->status;
  p.limit_ns = (a->wait_limit_ms > 0 ? (unsigned long long)a->wait_limit_ms : 10000ull) * 1000000ull;
  return 0;
}

static int grid_for(long long items) {
  long long g = (items + 7) / 8;          // 8 warps per CTA, one item per warp per trip
  const long long cap = 148 * 4;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

// out[r, :] = staged_rows[src(r)][tok(r), :] for the R rows this rank's experts receive (and their probabilities).
MSB_API int msb_moe_dispatch(const MsbMoeCommArgs* a, cudaStream_t stream) {
  MoeParams p;
  if (int rc = fill(p, a, "moe_dispatch")) return rc;
  MSB_REQUIRE(a->n_chunks == a->E_loc * a->world && a->chunk_dst_start && a->chunk_src_start, "moe_dispatch: chunk tables are required");
  for (int i = 0; i < a->world; ++i) MSB_REQUIRE(a->peer_tok[i] != nullptr, "moe_dispatch: missing token list of peer %d", i);
  moe_dispatch_kernel<<<grid_for(p.R), 256, 0, stream>>>(p);
  MSB_CHECK_LAUNCH("moe_dispatch");
  return 0;
}

// out[t, :] = sum over the experts e routed for token t of staged_rows[owner(e)][row(t, e), :]  (bf16 rows, fp32 sum).
MSB_API int msb_moe_combine(const MsbMoeCommArgs* a, cudaStream_t stream) {
  MoeParams p;
  if (int rc = fill(p, a, "moe_combine")) return rc;
  MSB_REQUIRE(a->map && a->rank_in_expert && a->dst_row_base, "moe_combine: routing tables are required");
  MSB_REQUIRE(a->row_cap > 0, "moe_combine: row_cap must be positive");
  moe_combine_kernel<<<grid_for(p.T), 256, 0, stream>>>(p);
  MSB_CHECK_LAUNCH("moe_combine");
  return 0;
}

// One launch that fills rank_in_expert [T, E], the sorted token / probability lists (at most ``list_cap`` entries) and the
// chunk / row-base tables from the routing map and the all-gathered count matrix.  probs_dtype: MSB_F32 or MSB_BF16.
MSB_API int msb_moe_build_plan(const unsigned char* map, const void* probs, int probs_dtype, const long long* counts, int ld, int T, int E,
                               int E_loc, int ep, int me, int* rank_in_expert, int* sorted_tok, float* sorted_probs,
                               long long* chunk_dst_start, long long* chunk_src_start, long long* dst_row_base, long long list_cap,
                               cudaStream_t s) {
  MSB_REQUIRE(map && probs && counts && rank_in_expert && sorted_tok && sorted_probs && chunk_dst_start && chunk_src_start && dst_row_base,
              "moe_build_plan: null argument");
  MSB_REQUIRE(T > 0 && E > 0 && E_loc > 0 && ep > 0 && E == E_loc * ep && me >= 0 && me < ep && ld >= E, "moe_build_plan: bad sizes");
  if (probs_dtype == MSB_BF16)
    moe_build_plan_kernel<__nv_bfloat16><<<E, 1024, 0, s>>>(map, (const __nv_bfloat16*)probs, counts, ld, T, E, E_loc, ep, me, rank_in_expert,
                                                            sorted_tok, sorted_probs, chunk_dst_start, chunk_src_start, dst_row_base, list_cap);
  else if (probs_dtype == MSB_F32)
    moe_build_plan_kernel<float><<<E, 1024, 0, s>>>(map, (const float*)probs, counts, ld, T, E, E_loc, ep, me, rank_in_expert, sorted_tok,
                                                    sorted_probs, chunk_dst_start, chunk_src_start, dst_row_base, list_cap);
  else { msb_set_error("moe_build_plan: unsupported probability dtype %d", probs_dtype); return 2; }
  MSB_CHECK_LAUNCH("moe_build_plan");
  return 0;
}

