// All-to-all with the layout transform folded in: every rank pulls, from each peer's staged tensor, the strided rows it
// needs and writes them straight into their final position.  Used by Ulysses context parallelism, where the exchange
// sequence-shards <-> head-shards is otherwise permute + contiguous copy + all-to-all (+ a second permute on the way
// back): here it is one staging copy and one kernel.
//
//   for src in ranks, r in [0, rows):
//       copy row_bytes from   peer[src] + src_base + r * src_row_stride
//                       to    out + src * dst_src_stride + r * dst_row_stride
//
// Peer memory is only read (ld.global.cg, 16 B per lane, 8 in flight); the entry handshake (epoch flags in the
// symmetric heap, bounded wait) proves every peer has staged its tensor and has left the previous call that read the
// slot being reused.  reference semantics: the all-to-alls of
// mindspeed/core/context_parallel/ulysses_context_parallel/ulysses_context_parallel.py:83-108.
#include "msb_common.cuh"
#include "msb_sm100.cuh"

namespace {
constexpr int A2A_MAX_RANKS = 8;
constexpr int A2A_FLAG_BASE = 1536;   // u32 index of this family's entry flags inside the heap's flag block

struct A2AParams {
  const char* peer[A2A_MAX_RANKS];
  char* out;
  long long rows, src_base, src_row_stride, dst_src_stride, dst_row_stride;
  int row_v4, world, rank;
  unsigned int epoch;
  unsigned int* flag_local;
  unsigned int* flag_peer[A2A_MAX_RANKS];
  unsigned int* status;
  unsigned long long limit_ns;
};

__device__ __forceinline__ uint4 a2a_ld(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ bool a2a_wait(const unsigned int* flag, unsigned int value, unsigned int* status, unsigned int code,
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

__global__ void __launch_bounds__(256) a2a_strided_pull_kernel(const A2AParams p) {
  bool alive = true;
  if (p.world > 1) {
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
      __threadfence_system();
      unsigned int* dst = p.flag_peer[threadIdx.x] + A2A_FLAG_BASE + p.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(p.epoch) : "memory");
    }
    if (threadIdx.x < p.world) alive = a2a_wait(p.flag_local + A2A_FLAG_BASE + threadIdx.x, p.epoch, p.status, 0x600u + threadIdx.x, p.limit_ns);
    alive = __syncthreads_and(alive);
  }
  if (!alive) return;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarp = (long long)gridDim.x * (blockDim.x >> 5);
  const long long total = p.rows * p.world;
  for (long long w = warp0; w < total; w += nwarp) {
    // sources interleaved so that consecutive warps pull from different peers (spreads the load over all links)
    const int src = (int)((w + p.rank) % p.world);
    const long long r = w / p.world;
    const uint4* from = reinterpret_cast<const uint4*>(p.peer[src] + p.src_base + r * p.src_row_stride);
    uint4* to = reinterpret_cast<uint4*>(p.out + src * p.dst_src_stride + r * p.dst_row_stride);
    int j = lane;
    for (; j + 7 * 32 < p.row_v4; j += 8 * 32) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = a2a_ld(from + j + u * 32);
#pragma unroll
      for (int u = 0; u < 8; ++u) to[j + u * 32] = v[u];
    }
    for (; j < p.row_v4; j += 32) to[j] = a2a_ld(from + j);
  }
}
}  // namespace

struct MsbA2AArgs {
  const void* peer[8];
  void* out;
  long long rows, src_base, src_row_stride, dst_src_stride, dst_row_stride;
  int row_bytes, world, rank;
  unsigned int epoch;
  unsigned int* flag_local;
  unsigned int* flag_peer[8];
  unsigned int* status;
  int wait_limit_ms;
};

MSB_API int msb_a2a_strided_pull(const MsbA2AArgs* a, cudaStream_t s) {
  MSB_REQUIRE(a != nullptr && a->out != nullptr, "a2a_strided_pull: null arguments");
  MSB_REQUIRE(a->world >= 1 && a->world <= A2A_MAX_RANKS && a->rank >= 0 && a->rank < a->world, "a2a_strided_pull: bad world/rank %d/%d", a->world, a->rank);
  MSB_REQUIRE(a->row_bytes > 0 && a->row_bytes % 16 == 0, "a2a_strided_pull: row size %d must be a multiple of 16 bytes", a->row_bytes);
  MSB_REQUIRE(a->src_base % 16 == 0 && a->src_row_stride % 16 == 0 && a->dst_src_stride % 16 == 0 && a->dst_row_stride % 16 == 0,
              "a2a_strided_pull: offsets and strides must be multiples of 16 bytes");
  MSB_REQUIRE(a->status && a->flag_local, "a2a_strided_pull: status word and flags are required");
  A2AParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < A2A_MAX_RANKS; ++i) {
    p.peer[i] = reinterpret_cast<const char*>(a->peer[i]);
    p.flag_peer[i] = a->flag_peer[i];
    if (i < a->world) MSB_REQUIRE(a->peer[i] && (a->world == 1 || a->flag_peer[i]), "a2a_strided_pull: missing pointers of peer %d", i);
  }
  p.out = reinterpret_cast<char*>(a->out);
  p.rows = a->rows; p.src_base = a->src_base; p.src_row_stride = a->src_row_stride;
  p.dst_src_stride = a->dst_src_stride; p.dst_row_stride = a->dst_row_stride;
  p.row_v4 = a->row_bytes / 16; p.world = a->world; p.rank = a->rank; p.epoch = a->epoch;
  p.flag_local = a->flag_local; p.status = a->status;
  p.limit_ns = (a->wait_limit_ms > 0 ? (unsigned long long)a->wait_limit_ms : 10000ull) * 1000000ull;
  long long g = (a->rows * a->world + 7) / 8;
  const long long cap = 148 * 4;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  a2a_strided_pull_kernel<<<(int)g, 256, 0, s>>>(p);
  MSB_CHECK_LAUNCH("a2a_strided_pull");
  return 0;
}
