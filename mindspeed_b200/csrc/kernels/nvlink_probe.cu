// Bandwidth probe for SM-initiated NVLink writes (used by mindspeed_b200/benchmarks/microbench_nvlink.py to choose how the
// fused GEMM + collective kernels move data).  Every CTA pushes 8 KB / 16 KB chunks of a local buffer into peers' buffers:
//   mode 0  bulk copy engine of the SM (TMA): global -> shared ring -> peer, one issuing thread per CTA
//   mode 1  plain loads and 16-byte stores by all threads of the CTA
//   mode 2  TMA stores only, from a shared-memory buffer that is never refilled (upper bound of the store path)
// Destination policy: `spread` = 0 sends everything to rank+1, `spread` = 1 sends chunk c to peer 1 + (c mod (world-1)).
// No cross-GPU waits: each rank only writes; the host times the launch with events and synchronises afterwards.
#include "msb_common.cuh"
#include "msb_sm100.cuh"

using namespace msb;
using namespace msb::sm100;

namespace {
struct ProbeParams {
  const uint8_t* src;
  uint8_t* peer[8];
  size_t bytes;      // bytes pushed by this GPU in total
  int chunk;         // bytes per chunk (multiple of 16, <= 16384)
  int world, rank, spread, mode, ring;
  unsigned int* status;
};

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}

__global__ void __launch_bounds__(256, 1) nvlink_probe_kernel(const ProbeParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + 8 * 16384;
  const long long n_chunks = (long long)(p.bytes / p.chunk);
  auto dst_of = [&](long long c) {
    const int hop = p.spread ? 1 + (int)(c % (p.world - 1)) : 1;
    return (p.rank + hop) % p.world;
  };
  if (p.mode == 1) {
    const uint4* s4 = reinterpret_cast<const uint4*>(p.src);
    const int v4 = p.chunk / 16;
    for (long long c = blockIdx.x; c < n_chunks; c += gridDim.x) {
      uint4* d4 = reinterpret_cast<uint4*>(p.peer[dst_of(c)]) + c * v4;
      const uint4* f = s4 + c * v4;
      for (int i = threadIdx.x; i < v4; i += 4 * blockDim.x) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) if (i + j * blockDim.x < v4) v[j] = f[i + j * blockDim.x];
#pragma unroll
        for (int j = 0; j < 4; ++j) if (i + j * blockDim.x < v4) d4[i + j * blockDim.x] = v[j];
      }
    }
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < 8; ++i) mbar_init(bars + 8 * i, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const int R = p.ring;
  if (p.mode == 2) {
    long long issued = 0;
    for (long long c = blockIdx.x; c < n_chunks; c += gridDim.x, ++issued) {
      bulk_s2g(p.peer[dst_of(c)] + c * p.chunk, base + (uint32_t)(issued % R) * 16384u, p.chunk);
      tma_store_commit();
    }
    tma_store_wait<0>();
    return;
  }
  // mode 0: loads run 2 items ahead of stores; a slot is reused when its store has read it
  uint32_t phase = 0;
  long long j = 0, stored = 0;
  long long my = (n_chunks - blockIdx.x + gridDim.x - 1) / gridDim.x;
  auto chunk_of = [&](long long i) { return (long long)blockIdx.x + i * gridDim.x; };
  auto store = [&](long long k) -> bool {
    const int slot = (int)(k % R);
    if (!mbar_wait(bars + 8 * slot, (phase >> slot) & 1u, p.status, 0x701u)) return false;
    phase ^= 1u << slot;
    const long long c = chunk_of(k);
    bulk_s2g(p.peer[dst_of(c)] + c * p.chunk, base + (uint32_t)slot * 16384u, p.chunk);
    tma_store_commit();
    ++stored;
    return true;
  };
  const int LAG = R / 2;
  for (; j < my; ++j) {
    if (j >= R) {
      if (R - LAG - 1 <= 0) tma_store_wait_read<0>();
      else if (R - LAG - 1 == 1) tma_store_wait_read<1>();
      else if (R - LAG - 1 == 2) tma_store_wait_read<2>();
      else tma_store_wait_read<3>();
    }
    const int slot = (int)(j % R);
    mbar_arrive_expect_tx(bars + 8 * slot, p.chunk);
    bulk_g2s(base + (uint32_t)slot * 16384u, p.src + chunk_of(j) * p.chunk, p.chunk, bars + 8 * slot);
    if (j >= LAG && !store(j - LAG)) return;
  }
  for (long long k = (my > LAG ? my - LAG : 0); k < my; ++k)
    if (!store(k)) return;
  tma_store_wait<0>();
}
}  // namespace

// Pushes `bytes` of `src` into the peers' buffers at the same offsets.  ring <= 8 slots of 16 KB.
MSB_API int msb_nvlink_probe(const void* src, void* const* peer, size_t bytes, int chunk, int world, int rank, int spread, int mode,
                             int ring, int ctas, unsigned int* status, cudaStream_t s) {
  MSB_REQUIRE(world >= 2 && world <= 8 && chunk % 16 == 0 && chunk > 0 && chunk <= 16384 && ring >= 2 && ring <= 8,
              "nvlink_probe: bad arguments");
  ProbeParams p;
  p.src = (const uint8_t*)src;
  for (int i = 0; i < 8; ++i) p.peer[i] = i < world ? (uint8_t*)peer[i] : nullptr;
  p.bytes = bytes; p.chunk = chunk; p.world = world; p.rank = rank; p.spread = spread; p.mode = mode; p.ring = ring; p.status = status;
  const int smem = 8 * 16384 + 64 + 1024;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(nvlink_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr = true;
  }
  nvlink_probe_kernel<<<ctas > 0 ? ctas : msb::num_sms(), 256, smem, s>>>(p);
  MSB_CHECK_LAUNCH("nvlink_probe");
  return 0;
}
