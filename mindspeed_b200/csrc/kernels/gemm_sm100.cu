// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
//   D[M,N] (+)= A[M,K] * B[K,N]      fp32 accumulation in tensor memory
//
// Operand layouts (row-major tensors in global memory), chosen per call:
//   A "K-major"  : stored [M, K]   (activation x in y = x W^T, grad dy in dx = dy W)
//   A "MN-major" : stored [K, M]   (dy in dW = dy^T x: the reduction dim is the row index)
//   B "K-major"  : stored [N, K]   (weight W [out,in] in y = x W^T)
//   B "MN-major" : stored [K, N]   (W in dx = dy W, x in dW = dy^T x)
// so forward, data-gradient and weight-gradient GEMMs of a linear layer all run without a transpose copy.
//
// CTA = 6 warps: warp 0 TMA producer (one lane), warp 1 MMA issuer (one lane; also owns TMEM alloc/dealloc),
// warps 2-5 epilogue (each owns the 32 TMEM lanes its warp-id modulo 4 selects).  Tile 128 x BN x 64 with
// BN in {128, 256}; NSTAGE shared-memory stages; two TMEM accumulators so the epilogue of tile i overlaps
// the main loop of tile i+1.  Grid = min(tiles, SMs), static round-robin tile order with M-grouping for L2 reuse.
//
// Epilogues: bf16 store (optional bias), fp32 store, fp32 accumulate-in-place (wgrad into main_grad).
// Multi-source A (one tensor map per source, rows_per_src rows each) and multi-destination D (one base pointer
// per owner) let the same kernel read an all-gathered operand shard by shard from peer GPUs and write
// reduce-scatter partials straight to their owners (mindspeed_b200/ops/fused_comm.py drives that).
//
// reference semantics being replaced: torch.matmul in the TP linears, npu_matmul_add_fp32
// (mindspeed/ops/npu_matmul_add.py:51-66) and the fused vendor ops npu_all_gather_base_mm / npu_mm_reduce_scatter_base
// (mindspeed/core/tensor_parallel/mc2_feature/linear_function.py:40,169).
#include "msb_common.cuh"
#include "msb_sm100.cuh"

using namespace msb;
using namespace msb::sm100;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int MAX_SRC = 8;

enum Epi : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ACC = 2 };

struct GemmParams {
  CUtensorMap tmA[MAX_SRC];
  CUtensorMap tmB;
  void* D[MAX_SRC];          // destination base per owner
  const void* bias;          // optional bf16 [N]
  int M, N, K;
  int a_rows_per_src;        // rows of the logical M served by each A source (>= M when single source)
  int d_rows_per_dst;        // rows of the logical M owned by each destination (>= M when single)
  long long ldd;             // leading dimension of D in elements
  long long d_row_offset;    // added to the local row index inside a destination (reduce-scatter slot)
  int m_tile_rot;            // rotation of the m-tile order (start at the local shard)
  int group_m;               // m-tiles per L2 group
  unsigned int* status;      // 0 = ok; else the code of the wait that timed out
  // cross-GPU handshake (world == 1: unused)
  int world, rank;
  unsigned int epoch;
  unsigned int* flag_local;              // [world] slots in this GPU's memory, written by peers
  unsigned int* flag_peer[MAX_SRC];      // peer r's flag array (mapped)
  int wait_peers_before;                 // all sources must be written before the main loop reads them
  int signal_peers_after;                // tell peers this GPU has finished reading/writing
};

template <int BN, int NSTAGE>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = NSTAGE * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int group_m, int rot, int& m, int& n) {
  const int per_group = group_m * num_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsz = min(num_m - first_m, group_m);
  const int r = t - g * per_group;
  m = first_m + (r % gsz);
  n = r / gsz;
  m = (m + rot) % num_m;
}

// Bounded spin on a flag in this GPU's memory written by a peer (system-scope acquire).
__device__ __forceinline__ bool wait_flag_ge(const unsigned int* flag, unsigned int value, unsigned int* status,
                                             unsigned int code, uint64_t limit_ns) {
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int)(v - value) >= 0) return true;
    if (globaltimer_ns() - t0 > limit_ns) { atomicCAS(status, 0u, code); return false; }
    if (*((volatile unsigned int*)status) != 0u) return false;
    __nanosleep(200);
  }
}

template <int BN, int NSTAGE, int EPI, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1) gemm_sm100_kernel(const __grid_constant__ GemmParams p) {
  using L = SmemLayout<BN, NSTAGE>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128B swizzle pattern is a function of address bits [4,10)
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (NSTAGE + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * NSTAGE + 4);
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = (BN <= 128) ? 256u : 512u;  // power of two >= 2 * BN

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 128); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // ---- cross-GPU entry handshake: every source buffer must be complete before any CTA reads it ----
  bool alive = true;
  if (p.world > 1 && p.wait_peers_before) {
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
      // tell peer `threadIdx.x` that this GPU's producer kernels (earlier in stream order) are done
      __threadfence_system();
      unsigned int* dst = p.flag_peer[threadIdx.x] + p.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(p.epoch) : "memory");
    }
    if (threadIdx.x < p.world) alive = wait_flag_ge(p.flag_local + threadIdx.x, p.epoch, p.status, 0x100u + threadIdx.x, 10000000000ull);
    alive = __syncthreads_and(alive);
  }

  if (alive) {
    if (warp == 0) {
      // ===================== TMA producer =====================
      if (lane == 0) {
        tma_prefetch_desc(&p.tmB);
        int stage = 0; uint32_t phase = 0;
        for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
          int m_blk, n_blk;
          tile_coords(t, num_m, num_n, p.group_m, p.m_tile_rot, m_blk, n_blk);
          const int m0 = m_blk * BM, n0 = n_blk * BN;
          const int src = m0 / p.a_rows_per_src;
          const int m_local = m0 - src * p.a_rows_per_src;
          const CUtensorMap* tmA = &p.tmA[src];
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 0x10u)) { alive = false; break; }
            const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
            const uint32_t sb = sa + L::A_BYTES;
            mbar_arrive_expect_tx(full_bar(stage), L::STAGE_BYTES);
            const int k0 = kb * BK;
            if (!A_MN) {
              tma_load_2d(sa, tmA, full_bar(stage), k0, m_local);                       // box [128 rows x 64 k]
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)                                          // boxes [64 k x 64 m]
                tma_load_2d(sa + j * (BK * 128), tmA, full_bar(stage), m_local + j * 64, k0);
            }
            if (!B_MN) {
              tma_load_2d(sb, &p.tmB, full_bar(stage), k0, n0);                          // box [BN rows x 64 k]
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * (BK * 128), &p.tmB, full_bar(stage), n0 + j * 64, k0);
            }
            if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
          }
        }
      }
    } else if (warp == 1) {
      // ===================== MMA issuer =====================
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc_f16(BM, BN, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
        int stage = 0; uint32_t phase = 0;
        int acc = 0; uint32_t acc_phase = 0;
        for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
          if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, p.status, 0x20u)) { alive = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, p.status, 0x21u)) { alive = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
            const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // K-major: advance 16 elements = 32 bytes inside the swizzled row; MN-major: 16 k-rows = 2048 bytes
              const uint64_t adesc = A_MN ? make_smem_desc(sa + k * (UMMA_K * 128), BK * 128, 1024)
                                          : make_smem_desc(sa + k * (UMMA_K * 2), 0, 1024);
              const uint64_t bdesc = B_MN ? make_smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024)
                                          : make_smem_desc(sb + k * (UMMA_K * 2), 0, 1024);
              umma_f16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(empty_bar(stage));          // stage reusable once these MMAs have read it
            if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
          }
          if (!alive) break;
          umma_commit(tfull_bar(acc));              // accumulator complete
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
      }
    } else {
      // ===================== epilogue (warps 2..5) =====================
      const int q = warp & 3;                      // TMEM lane quarter this warp may access
      int acc = 0; uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(t, num_m, num_n, p.group_m, p.m_tile_rot, m_blk, n_blk);
        if (!mbar_wait(tfull_bar(acc), acc_phase, p.status, 0x30u)) { alive = false; break; }
        tc_fence_after();
        const int row = m_blk * BM + q * 32 + lane;
        const int dst = row / p.d_rows_per_dst;
        const long long row_local = (long long)(row - dst * p.d_rows_per_dst) + p.d_row_offset;
        const bool row_ok = row < p.M;
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
        for (int c2 = 0; c2 < BN; c2 += 64) {
          uint32_t rr[2][32];
          tmem_ld_32x32(t_row + (uint32_t)c2, rr[0]);          // two loads in flight per wait
          tmem_ld_32x32(t_row + (uint32_t)(c2 + 32), rr[1]);
          tmem_ld_wait();
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
          uint32_t* r = rr[hh];
          const int c = c2 + hh * 32;
          const int col0 = n_blk * BN + c;
          if (row_ok && col0 < p.N) {
            if (EPI == EPI_BF16) {
              __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D[dst]) + row_local * p.ldd + col0;
              const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.bias);
              if (col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(drow) & 15) == 0)) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  uint32_t pk[4];
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    float a = __uint_as_float(r[v * 8 + 2 * j]), b = __uint_as_float(r[v * 8 + 2 * j + 1]);
                    if (bias) { a += __bfloat162float(bias[col0 + v * 8 + 2 * j]); b += __bfloat162float(bias[col0 + v * 8 + 2 * j + 1]); }
                    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                    pk[j] = *reinterpret_cast<uint32_t*>(&h);
                  }
                  *reinterpret_cast<uint4*>(drow + v * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
              } else {
                for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
                  float a = __uint_as_float(r[j]);
                  if (bias) a += __bfloat162float(bias[col0 + j]);
                  drow[j] = __float2bfloat16_rn(a);
                }
              }
            } else {
              float* drow = reinterpret_cast<float*>(p.D[dst]) + row_local * p.ldd + col0;
              if (col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(drow) & 15) == 0)) {
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                  float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]),
                                         __uint_as_float(r[4 * v + 3]));
                  if (EPI == EPI_F32_ACC) {
                    float4 old = *reinterpret_cast<float4*>(drow + 4 * v);
                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                  }
                  *reinterpret_cast<float4*>(drow + 4 * v) = o;
                }
              } else {
                for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
                  float a = __uint_as_float(r[j]);
                  drow[j] = (EPI == EPI_F32_ACC) ? drow[j] + a : a;
                }
              }
            }
          }
        }
          }
        tc_fence_before();
        mbar_arrive(tempty_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  }

  // ---- teardown: all roles meet, TMEM is returned ----
  tc_fence_before();
  __syncthreads();
  if (p.world > 1 && p.signal_peers_after) {
    // per-CTA arrival counter in flag_local[world]; the last CTA publishes this GPU's "done" to every peer
    __shared__ unsigned int is_last;
    if (threadIdx.x == 0) {
      __threadfence_system();
      unsigned int prev = atomicAdd(p.flag_local + 2 * MAX_SRC, 1u);
      is_last = (prev == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (is_last && threadIdx.x < p.world) {
      if (threadIdx.x == 0) p.flag_local[2 * MAX_SRC] = 0u;
      unsigned int* dstf = p.flag_peer[threadIdx.x] + MAX_SRC + p.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dstf), "r"(p.epoch) : "memory");
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// =====================================================================================================
// Fused GEMM + collective over NVLink peer memory (one kernel, four extra "copy" warps per CTA).
//
// MODE_AG  all-gather -> GEMM.  The A operand is the all-gathered activation [M, K]; rank r owns rows
//          [r*rows_per_rank, (r+1)*rows_per_rank) of it and has written them into slab r of its own symmetric
//          buffer before the launch.  Copy warps pull the other ranks' slabs over NVLink (plain peer loads,
//          16 B per thread, 8 in flight) into this GPU's buffer in 16-row pieces and bump a per-m-tile counter;
//          the TMA producer waits (bounded) for an m-tile's counter before loading it from LOCAL memory, so a
//          remote tile crosses NVLink exactly once and every MMA operand read is a local TMA load.  Tiles are
//          visited m-major starting at the local slab, so compute starts at once.  The filled local buffer is
//          also the "gathered input" the backward pass needs.
// MODE_RS  GEMM -> reduce-scatter.  Each finished 128 x BN tile is stored to a local partial buffer; the copy
//          warps of the same CTA then push its rows (coalesced 512 B segments) into the owner rank's staging
//          slab [src rank][rows_per_rank, N].  Tiles are visited starting at the next rank's rows, own rows last.
//          When a GPU has pushed everything its last CTA publishes an exit flag to every peer; the separate
//          msb_rs_reduce kernel on the owner waits (bounded) for all exit flags and sums the slabs in rank order
//          (deterministic).
// Both modes begin with an all-to-all flag handshake (epoch counter) that proves every peer has finished the
// previous use of the shared buffers and has written its inputs.
// =====================================================================================================
enum CommMode : int { MODE_AG = 1, MODE_RS = 2 };
constexpr int AG_SUB = 8;   // pieces per 128-row m-tile pulled independently

struct CommParams {
  GemmParams g;
  // AG
  const uint4* ag_peer[MAX_SRC];   // peer r's symmetric gathered buffer (base)
  uint4* ag_local;                 // this GPU's gathered buffer (also the A operand)
  unsigned int* ready;             // [num_m_tiles] counters in local memory
  unsigned int ready_target;
  int rows_per_rank;
  // RS
  uint4* rs_stage_peer[MAX_SRC];   // owner o's staging base
  const uint4* rs_partial;         // local partial [M, N] bf16 (== g.D[0])
};

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_counter_ge(const unsigned int* ctr, unsigned int value, unsigned int* status,
                                                unsigned int code, uint64_t limit_ns) {
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if ((int)(v - value) >= 0) return true;
    if (globaltimer_ns() - t0 > limit_ns) { atomicCAS(status, 0u, code); return false; }
    if (*((volatile unsigned int*)status) != 0u) return false;
    __nanosleep(100);
  }
}

template <int BN, int NSTAGE, int MODE, bool B_MN>
__global__ void __launch_bounds__(448, 1) gemm_comm_sm100_kernel(const __grid_constant__ CommParams cp) {
  const GemmParams& p = cp.g;
  using L = SmemLayout<BN, NSTAGE>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (NSTAGE + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + 2 + a); };
  auto pfull_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + 4 + a); };
  auto pempty_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + 6 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * NSTAGE + 8);
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int tiles_per_rank = cp.rows_per_rank / BM;
  constexpr uint32_t TMEM_COLS = (BN <= 128) ? 256u : 512u;
  // tile order: groups of `group_m` m-tiles (inside a group n-major, so concurrently running CTAs share both A and B
  // tiles in L2), groups visited in rotated m order; group_m divides the per-rank slab, so a group never straddles ranks
  auto tile_mn = [&](int t, int& m, int& n) { tile_coords(t, num_m, num_n, p.group_m, p.m_tile_rot, m, n); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 128);
      mbar_init(pfull_bar(a), 128); mbar_init(pempty_bar(a), 128);
    }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // ---- entry handshake ----
  bool alive = true;
  {
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
      __threadfence_system();
      unsigned int* dst = p.flag_peer[threadIdx.x] + p.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(p.epoch) : "memory");
    }
    if (threadIdx.x < p.world)
      alive = wait_flag_ge(p.flag_local + threadIdx.x, p.epoch, p.status, 0x100u + threadIdx.x, 10000000000ull);
    alive = __syncthreads_and(alive);
  }

  if (alive) {
    if (warp == 0) {
      // ===================== TMA producer =====================
      if (lane == 0) {
        int stage = 0; uint32_t phase = 0;
        for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
          int m_blk, n_blk;
          tile_mn(t, m_blk, n_blk);
          if (MODE == MODE_AG && (m_blk / tiles_per_rank) != p.rank) {
            if (!wait_counter_ge(cp.ready + m_blk, cp.ready_target, p.status, 0x40u, 10000000000ull)) { alive = false; break; }
            asm volatile("fence.proxy.async.global;" ::: "memory");   // generic-proxy peer copies -> TMA (async proxy) reads
          }
          const int m0 = m_blk * BM, n0 = n_blk * BN;
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 0x10u)) { alive = false; break; }
            const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
            const uint32_t sb = sa + L::A_BYTES;
            mbar_arrive_expect_tx(full_bar(stage), L::STAGE_BYTES);
            const int k0 = kb * BK;
            tma_load_2d(sa, &p.tmA[0], full_bar(stage), k0, m0);
            if (!B_MN) {
              tma_load_2d(sb, &p.tmB, full_bar(stage), k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &p.tmB, full_bar(stage), n0 + j * 64, k0);
            }
            if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
          }
        }
      }
    } else if (warp == 1) {
      // ===================== MMA issuer =====================
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc_f16(BM, BN, 1, 0, B_MN ? 1 : 0);
        int stage = 0; uint32_t phase = 0;
        int acc = 0; uint32_t acc_phase = 0;
        for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
          if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, p.status, 0x20u)) { alive = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, p.status, 0x21u, 12000000000ull)) { alive = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
            const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t adesc = make_smem_desc(sa + k * (UMMA_K * 2), 0, 1024);
              const uint64_t bdesc = B_MN ? make_smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024)
                                          : make_smem_desc(sb + k * (UMMA_K * 2), 0, 1024);
              umma_f16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(empty_bar(stage));
            if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
          }
          if (!alive) break;
          umma_commit(tfull_bar(acc));
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
      }
    } else if (warp < 6) {
      // ===================== epilogue (warps 2..5) =====================
      const int q = warp & 3;
      int acc = 0; uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        int m_blk, n_blk;
        tile_mn(t, m_blk, n_blk);
        if (!mbar_wait(tfull_bar(acc), acc_phase, p.status, 0x30u, 14000000000ull)) { alive = false; break; }
        tc_fence_after();
        if (MODE == MODE_RS) {
          // the push of the tile that used this slot two tiles ago must have been picked up
          if (!mbar_wait(pempty_bar(acc), acc_phase ^ 1u, p.status, 0x31u, 14000000000ull)) { alive = false; break; }
        }
        const int row = m_blk * BM + q * 32 + lane;
        const bool row_ok = row < p.M;
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
        for (int c2 = 0; c2 < BN; c2 += 64) {
          uint32_t rr[2][32];
          tmem_ld_32x32(t_row + (uint32_t)c2, rr[0]);          // two loads in flight per wait
          tmem_ld_32x32(t_row + (uint32_t)(c2 + 32), rr[1]);
          tmem_ld_wait();
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t* r = rr[hh];
            const int col0 = n_blk * BN + c2 + hh * 32;
            if (row_ok && col0 < p.N) {
              __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D[0]) + (long long)row * p.ldd + col0;
              if (col0 + 32 <= p.N) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  uint32_t pk[4];
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
                    pk[j] = *reinterpret_cast<uint32_t*>(&h);
                  }
                  *reinterpret_cast<uint4*>(drow + v * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
              } else {
                for (int j = 0; j < 32 && col0 + j < p.N; ++j) drow[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
              }
            }
          }
        }
        tc_fence_before();
        mbar_arrive(tempty_bar(acc));
        if (MODE == MODE_RS) mbar_arrive(pfull_bar(acc));      // tile is in the local partial buffer (CTA-scope release)
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    } else {
      // ===================== copy warps (6..9): NVLink traffic =====================
      // two independent copy groups of four warps each (warps 6-9 and 10-13): twice the loads in flight per SM
      const int cgrp = (threadIdx.x - 192) >> 7;   // 0 or 1
      const int ct = (threadIdx.x - 192) & 127;    // 0..127 inside the group
      if (MODE == MODE_AG) {
        // work items in consumption order: shard (rank+1), (rank+2), ...; inside a shard m-tile by m-tile; AG_SUB pieces each
        const int items = (p.world - 1) * tiles_per_rank * AG_SUB;
        const size_t piece_v4 = (size_t)(BM / AG_SUB) * (size_t)p.K * 2 / 16;   // uint4 per piece (contiguous rows)
        for (int it = blockIdx.x * 2 + cgrp; it < items; it += 2 * gridDim.x) {
          const int sub = it % AG_SUB;
          const int mt_lin = it / AG_SUB;
          const int s = mt_lin / tiles_per_rank + 1;
          const int src = (p.rank + s) % p.world;
          const int mt = src * tiles_per_rank + (mt_lin % tiles_per_rank);
          const size_t base = ((size_t)mt * AG_SUB + sub) * piece_v4;
          const uint4* from = cp.ag_peer[src] + base;
          uint4* to = cp.ag_local + base;
          size_t i = ct;
          // 16 x 16 B per thread in flight: 32 KB per CTA, ~4.7 MB per GPU, about twice the NVLink bandwidth-delay product
          for (; i + 15 * 128 < piece_v4; i += 16 * 128) {
            uint4 v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = ld_cg_v4(from + i + j * 128);
#pragma unroll
            for (int j = 0; j < 16; ++j) to[i + j * 128] = v[j];
          }
          for (; i + 3 * 128 < piece_v4; i += 4 * 128) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = ld_cg_v4(from + i + j * 128);
#pragma unroll
            for (int j = 0; j < 4; ++j) to[i + j * 128] = v[j];
          }
          for (; i < piece_v4; i += 128) to[i] = ld_cg_v4(from + i);
          __threadfence();
          named_bar_sync(1 + cgrp, 128);
          if (ct == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(cp.ready + mt) : "memory");
        }
      } else {
        // group g pushes the tiles that used accumulator slot g (slots alternate tile by tile), so each group owns one
        // pfull/pempty barrier pair and its phase flips once per tile it handles
        int acc = 0; uint32_t my_phase = 0;
        const int cwarp = ct >> 5;
        for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x, acc ^= 1) {
          if (acc != cgrp) continue;
          int m_blk, n_blk;
          tile_mn(t, m_blk, n_blk);
          if (!mbar_wait(pfull_bar(acc), my_phase, p.status, 0x50u, 16000000000ull)) { alive = false; break; }
          const int owner = m_blk / tiles_per_rank;
          if (owner != p.rank) {
            const int n0 = n_blk * BN;
            const int ncols = min(BN, p.N - n0);
            const int v4_per_row = ncols / 8;                      // N is a multiple of 8
            const long long ld_v4 = p.ldd / 8;
            const uint4* src_base = cp.rs_partial + (long long)(m_blk * BM) * ld_v4 + n0 / 8;
            // owner's staging: [src rank][rows_per_rank][N]
            uint4* dst_base = cp.rs_stage_peer[owner] + ((long long)p.rank * cp.rows_per_rank + (m_blk % tiles_per_rank) * BM) * ld_v4 + n0 / 8;
            for (int r0 = cwarp; r0 < BM; r0 += 4 * 8) {
              uint4 v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int r = r0 + 4 * j;
                if (lane < v4_per_row && r < BM) v[j] = ld_cg_v4(src_base + (long long)r * ld_v4 + lane);
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int r = r0 + 4 * j;
                if (lane < v4_per_row && r < BM) dst_base[(long long)r * ld_v4 + lane] = v[j];
              }
            }
          }
          mbar_arrive(pempty_bar(acc));
          my_phase ^= 1u;
        }
        __threadfence_system();
      }
    }
  }

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (MODE == MODE_RS) {
    __shared__ unsigned int is_last;
    if (threadIdx.x == 0) {
      __threadfence_system();
      unsigned int prev = atomicAdd(p.flag_local + 2 * MAX_SRC, 1u);
      is_last = (prev == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (is_last && threadIdx.x < p.world) {
      if (threadIdx.x == 0) p.flag_local[2 * MAX_SRC] = 0u;
      __threadfence_system();
      unsigned int* dstf = p.flag_peer[threadIdx.x] + MAX_SRC + p.rank;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dstf), "r"(p.epoch) : "memory");
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Owner-side reduction of the reduce-scatter: out[rows, N] = sum over ranks of slab_r (own slab read from the
// local partial buffer), fixed rank order, fp32 accumulation.  Waits (bounded) for every peer's exit flag.
__global__ void __launch_bounds__(256) rs_reduce_kernel(const uint4* __restrict__ stage, const uint4* __restrict__ own_partial,
                                                         uint4* __restrict__ out, const __nv_bfloat16* __restrict__ residual,
                                                         long long n_v4, long long slab_v4, int world, int rank,
                                                         const unsigned int* flag_local, unsigned int epoch,
                                                         unsigned int* status, unsigned long long limit_ns) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < world && threadIdx.x != rank) {
    if (!wait_flag_ge(flag_local + MAX_SRC + threadIdx.x, epoch, status, 0x200u + threadIdx.x, limit_ns)) ok = 0;
  }
  __syncthreads();
  if (!ok) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_v4; i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r = 0; r < world; ++r) {
      uint4 v = (r == rank) ? ld_cg_v4(own_partial + i) : ld_cg_v4(stage + (long long)r * slab_v4 + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(h[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
    }
    if (residual) {
      uint4 v = *reinterpret_cast<const uint4*>(residual + i * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(h[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
    }
    uint4 o;
    __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) ho[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    out[i] = o;
  }
}

template <int BN, int NSTAGE, int MODE, bool B_MN>
int launch_comm_variant(const CommParams& cp, int grid, cudaStream_t s) {
  using L = SmemLayout<BN, NSTAGE>;
  auto kern = gemm_comm_sm100_kernel<BN, NSTAGE, MODE, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) { msb_set_error("gemm_comm_sm100: cannot set %d bytes of dynamic shared memory: %s", L::TOTAL, cudaGetErrorString(e)); return 1; }
    attr_set = true;
  }
  kern<<<grid, 448, L::TOTAL, s>>>(cp);
  MSB_CHECK_LAUNCH("gemm_comm_sm100");
  return 0;
}

template <int BN, int NSTAGE, int EPI, bool A_MN, bool B_MN>
int launch_variant(const GemmParams& p, int grid, cudaStream_t s) {
  using L = SmemLayout<BN, NSTAGE>;
  auto kern = gemm_sm100_kernel<BN, NSTAGE, EPI, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) { msb_set_error("gemm_sm100: cannot set %d bytes of dynamic shared memory: %s", L::TOTAL, cudaGetErrorString(e)); return 1; }
    attr_set = true;
  }
  kern<<<grid, 192, L::TOTAL, s>>>(p);
  MSB_CHECK_LAUNCH("gemm_sm100");
  return 0;
}

template <int BN, int NSTAGE, int EPI>
int launch_major(const GemmParams& p, int a_mn, int b_mn, int grid, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch_variant<BN, NSTAGE, EPI, false, false>(p, grid, s);
  if (!a_mn && b_mn) return launch_variant<BN, NSTAGE, EPI, false, true>(p, grid, s);
  if (a_mn && b_mn) return launch_variant<BN, NSTAGE, EPI, true, true>(p, grid, s);
  return launch_variant<BN, NSTAGE, EPI, true, false>(p, grid, s);
}

template <int BN, int NSTAGE>
int launch_epi(const GemmParams& p, int epi, int a_mn, int b_mn, int grid, cudaStream_t s) {
  switch (epi) {
    case EPI_BF16: return launch_major<BN, NSTAGE, EPI_BF16>(p, a_mn, b_mn, grid, s);
    case EPI_F32: return launch_major<BN, NSTAGE, EPI_F32>(p, a_mn, b_mn, grid, s);
    case EPI_F32_ACC: return launch_major<BN, NSTAGE, EPI_F32_ACC>(p, a_mn, b_mn, grid, s);
  }
  msb_set_error("gemm_sm100: unknown epilogue %d", epi);
  return 2;
}

int pick_bn(int M, int N, int sms) {
  // modelled time = waves * (tile width + fixed per-tile overhead); candidates 256 / 192 / 128
  if (N <= 128) return 128;
  const int cands[3] = {256, 192, 128};
  int best = 256; double best_t = 1e30;
  for (int i = 0; i < 3; ++i) {
    const int bn = cands[i];
    const long long tiles = (long long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    const long long waves = (tiles + sms - 1) / sms;
    const double t = (double)waves * (bn + 40.0);
    if (t < best_t * 0.97) { best_t = t; best = bn; }
  }
  return best;
}

}  // namespace

// Arguments of the multi-source / multi-destination form; the plain GEMM passes nsrc = ndst = 1.
struct MsbGemmArgs {
  const void* A[MAX_SRC];   // A source bases (each [a_rows_per_src, K] K-major or [K, a_rows_per_src] MN-major)
  const void* B;
  void* D[MAX_SRC];
  const void* bias;
  long long lda, ldb, ldd;  // leading dimensions in elements of the stored row-major tensors
  int M, N, K;
  int nsrc, a_rows_per_src;
  int ndst, d_rows_per_dst;
  long long d_row_offset;
  int a_mn_major, b_mn_major;
  int epilogue;             // 0 bf16 store, 1 fp32 store, 2 fp32 accumulate
  int m_tile_rot;
  int max_ctas;             // 0: all SMs
  unsigned int* status;
  int world, rank;
  unsigned int epoch;
  unsigned int* flag_local;
  unsigned int* flag_peer[MAX_SRC];
  int wait_peers_before, signal_peers_after;
};

namespace msb {
bool gemm2_eligible(const void* D, long long ldd, int epilogue);
int gemm2_launch(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda, long long ldb,
                 long long ldd, int a_mn, int b_mn, int epilogue, int bn, int max_ctas, int stream_k, unsigned int* status,
                 cudaStream_t s);
}

// Kernel choice for the plain GEMM: 0 = by the time model below, 1 = one-CTA kernel (this file), 2 / 3 = CTA-pair kernel
// (gemm2_sm100.cu) with 256 x 256 / 256 x 128 tiles.  Micro-benchmarks force a variant; training leaves it at 0.
static int g_variant = 0;
MSB_API void msb_gemm_set_variant(int v) { g_variant = (v >= 0 && v <= 3) ? v : 0; }
MSB_API int msb_gemm_get_variant() { return g_variant; }

// The CTA-pair kernel with 256 x 256 tiles wins on every measured layer shape; outputs at most 128 columns wide stay on
// the one-CTA kernel's 128 x 128 tiles (half-empty 256-wide tiles would waste the tensor pipe).
static int choose_variant(int M, int N, int sms) {
  (void)M; (void)sms;
  return N > 128 ? 2 : 1;
}

// Weight-gradient accumulation may balance k-blocks over the SMs (partial tiles summed by reduce-adds in an order that
// varies run to run).  1 = allowed (default), 0 = whole tiles only: bit-reproducible accumulation.
static int g_stream_k = 1;
MSB_API void msb_gemm_set_stream_k(int v) { g_stream_k = v ? 1 : 0; }
MSB_API int msb_gemm_get_stream_k() { return g_stream_k; }

// Process-wide cap on the number of CTAs the persistent GEMM-class kernels launch (0 = no cap).  Two such kernels
// on different streams share the GPU by SM count when each is capped (one CTA occupies a whole SM here).
static int g_cta_limit = 0;
MSB_API void msb_gemm_set_cta_limit(int n) { g_cta_limit = n > 0 ? n : 0; }
MSB_API int msb_gemm_get_cta_limit() { return g_cta_limit; }

MSB_API int msb_gemm_bf16_ex(const MsbGemmArgs* a, cudaStream_t s) {
  MSB_REQUIRE(a->M > 0 && a->N > 0 && a->K > 0, "gemm: empty problem %dx%dx%d", a->M, a->N, a->K);
  MSB_REQUIRE(a->nsrc >= 1 && a->nsrc <= MAX_SRC && a->ndst >= 1 && a->ndst <= MAX_SRC, "gemm: bad source/destination count");
  MSB_REQUIRE(a->status != nullptr, "gemm: status word is required");
  MSB_REQUIRE(a->a_rows_per_src % BM == 0 || a->nsrc == 1, "gemm: rows per A source must be a multiple of %d", BM);
  MSB_REQUIRE(a->d_rows_per_dst % 32 == 0 || a->ndst == 1, "gemm: rows per destination must be a multiple of 32");
  const int sms = msb::num_sms();
  if (a->nsrc == 1 && a->ndst == 1 && a->world <= 1 && a->m_tile_rot == 0 && a->d_row_offset == 0 && g_variant != 1 &&
      msb::gemm2_eligible(a->D[0], a->ldd, a->epilogue)) {
    int cap = a->max_ctas;
    if (g_cta_limit > 0 && (cap == 0 || cap > g_cta_limit)) cap = g_cta_limit;
    const int v = g_variant ? g_variant : choose_variant(a->M, a->N, cap > 0 && cap < sms ? cap : sms);
    if (v != 1)
      return msb::gemm2_launch(a->A[0], a->B, a->D[0], a->bias, a->M, a->N, a->K, a->lda, a->ldb, a->ldd, a->a_mn_major,
                               a->b_mn_major, a->epilogue, v == 2 ? 256 : 128, cap, g_stream_k, a->status, s);
  }
  const int bn = pick_bn(a->M, a->N, sms);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < a->nsrc; ++i) {
    int rc;
    const uint64_t rows = (a->nsrc == 1) ? (uint64_t)a->M : (uint64_t)a->a_rows_per_src;
    if (!a->a_mn_major) rc = make_tmap_2d(&p.tmA[i], a->A[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, a->K, a->lda, BM, BK);
    else rc = make_tmap_2d(&p.tmA[i], a->A[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->K, rows, a->lda, BK, 64);
    if (rc) return rc;
  }
  {
    int rc;
    if (!a->b_mn_major) rc = make_tmap_2d(&p.tmB, a->B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->N, a->K, a->ldb, bn, BK);
    else rc = make_tmap_2d(&p.tmB, a->B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->K, a->N, a->ldb, BK, 64);
    if (rc) return rc;
  }
  for (int i = 0; i < a->ndst; ++i) p.D[i] = a->D[i];
  p.bias = a->bias;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.a_rows_per_src = (a->nsrc == 1) ? ((a->M + BM - 1) / BM) * BM + BM : a->a_rows_per_src;
  p.d_rows_per_dst = (a->ndst == 1) ? 0x7fffffff : a->d_rows_per_dst;
  p.ldd = a->ldd; p.d_row_offset = a->d_row_offset;
  const int num_m = (a->M + BM - 1) / BM;
  p.m_tile_rot = ((a->m_tile_rot % num_m) + num_m) % num_m;
  p.group_m = (a->m_tile_rot != 0 || a->nsrc > 1 || a->ndst > 1) ? num_m : 16;
  if (p.group_m > num_m) p.group_m = num_m;
  p.status = a->status;
  p.world = a->world; p.rank = a->rank; p.epoch = a->epoch;
  p.flag_local = a->flag_local;
  for (int i = 0; i < MAX_SRC; ++i) p.flag_peer[i] = a->flag_peer[i];
  p.wait_peers_before = a->wait_peers_before; p.signal_peers_after = a->signal_peers_after;
  const long long tiles = (long long)num_m * ((a->N + bn - 1) / bn);
  int grid = (int)(tiles < sms ? tiles : sms);
  if (a->max_ctas > 0 && grid > a->max_ctas) grid = a->max_ctas;
  if (g_cta_limit > 0 && grid > g_cta_limit) grid = g_cta_limit;
  if (bn == 256) return launch_epi<256, 4>(p, a->epilogue, a->a_mn_major, a->b_mn_major, grid, s);
  if (bn == 192) return launch_epi<192, 5>(p, a->epilogue, a->a_mn_major, a->b_mn_major, grid, s);
  return launch_epi<128, 6>(p, a->epilogue, a->a_mn_major, a->b_mn_major, grid, s);
}

// Plain GEMM: D[M,N] (+)= A * B with the layouts described at the top of the file.
MSB_API int msb_gemm_bf16(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda,
                          long long ldb, long long ldd, int a_mn_major, int b_mn_major, int epilogue, unsigned int* status,
                          cudaStream_t s) {
  MsbGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.A[0] = A; a.B = B; a.D[0] = D; a.bias = bias;
  a.lda = lda; a.ldb = ldb; a.ldd = ldd;
  a.M = M; a.N = N; a.K = K;
  a.nsrc = 1; a.ndst = 1; a.a_rows_per_src = M; a.d_rows_per_dst = M;
  a.a_mn_major = a_mn_major; a.b_mn_major = b_mn_major; a.epilogue = epilogue;
  a.status = status; a.world = 1;
  return msb_gemm_bf16_ex(&a, s);
}

// ---------------------------------------------------------------------------------------------------------
// Fused GEMM + collective launchers
// ---------------------------------------------------------------------------------------------------------
struct MsbCommArgs {
  const void* A;                 // AG: this GPU's gathered buffer [M, K]; RS: local activation [M, K]
  const void* B;                 // weight, K-major [N, K] (b_mn_major = 0) or MN-major [K, N] (1)
  void* D;                       // AG: output [M, N]; RS: local partial buffer [M, N]
  const void* peer_buf[MAX_SRC]; // AG: every rank's gathered buffer; RS: every rank's staging [world][rows_per_rank, N]
  int M, N, K;
  int b_mn_major;
  int world, rank;
  unsigned int epoch;
  unsigned int* flag_local;
  unsigned int* flag_peer[MAX_SRC];
  unsigned int* ready;           // AG: [M/128] counters, zeroed by the launcher
  unsigned int* status;
};

static int fill_comm(CommParams& cp, const MsbCommArgs* a, int mode, int bn) {
  memset(&cp, 0, sizeof(cp));
  GemmParams& p = cp.g;
  int rc = make_tmap_2d(&p.tmA[0], a->A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->M, a->K, a->K, BM, BK);
  if (rc) return rc;
  if (!a->b_mn_major) rc = make_tmap_2d(&p.tmB, a->B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->N, a->K, a->K, bn, BK);
  else rc = make_tmap_2d(&p.tmB, a->B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->K, a->N, a->N, BK, 64);
  if (rc) return rc;
  p.D[0] = a->D;
  p.M = a->M; p.N = a->N; p.K = a->K; p.ldd = a->N;
  p.status = a->status; p.world = a->world; p.rank = a->rank; p.epoch = a->epoch;
  p.flag_local = a->flag_local;
  for (int i = 0; i < MAX_SRC; ++i) p.flag_peer[i] = a->flag_peer[i];
  cp.rows_per_rank = a->M / a->world;
  const int tiles_per_rank = cp.rows_per_rank / BM;
  p.group_m = 8;
  while (tiles_per_rank % p.group_m != 0) p.group_m >>= 1;   // 8, 4, 2 or 1: a divisor of the per-rank slab
  if (mode == MODE_AG) {
    p.m_tile_rot = a->rank * tiles_per_rank;
    for (int i = 0; i < a->world; ++i) cp.ag_peer[i] = reinterpret_cast<const uint4*>(a->peer_buf[i]);
    cp.ag_local = reinterpret_cast<uint4*>(const_cast<void*>(a->A));
    cp.ready = a->ready; cp.ready_target = AG_SUB;
  } else {
    p.m_tile_rot = ((a->rank + 1) % a->world) * tiles_per_rank;
    for (int i = 0; i < a->world; ++i) cp.rs_stage_peer[i] = reinterpret_cast<uint4*>(const_cast<void*>(a->peer_buf[i]));
    cp.rs_partial = reinterpret_cast<const uint4*>(a->D);
  }
  return 0;
}

static int check_comm(const MsbCommArgs* a, const char* what) {
  MSB_REQUIRE(a->world >= 2 && a->world <= MAX_SRC, "%s: world size %d not in [2, %d]", what, a->world, MAX_SRC);
  MSB_REQUIRE(a->M % (a->world * BM) == 0, "%s: M=%d must be a multiple of world*128", what, a->M);
  MSB_REQUIRE(a->N % 8 == 0 && a->K % 8 == 0, "%s: N=%d and K=%d must be multiples of 8", what, a->N, a->K);
  MSB_REQUIRE(a->status && a->flag_local, "%s: status and flags are required", what);
  return 0;
}

// Y[M, N] = allgather(x)[M, K] * B.  Every rank has already stored its rows into slab `rank` of its own gathered buffer.
MSB_API int msb_gemm_allgather(const MsbCommArgs* a, cudaStream_t s) {
  int rc = check_comm(a, "gemm_allgather");
  if (rc) return rc;
  MSB_REQUIRE((a->K * 2 * (BM / AG_SUB)) % 16 == 0, "gemm_allgather: K=%d too small", a->K);
  const int bn = pick_bn(a->M, a->N, msb::num_sms());
  CommParams cp;
  rc = fill_comm(cp, a, MODE_AG, bn);
  if (rc) return rc;
  if (cudaMemsetAsync(a->ready, 0, sizeof(unsigned int) * (a->M / BM), s) != cudaSuccess) { msb_set_error("gemm_allgather: memset failed"); return 1; }
  int grid = msb::num_sms();
  if (g_cta_limit > 0 && grid > g_cta_limit) grid = g_cta_limit;
  if (bn == 256) return a->b_mn_major ? launch_comm_variant<256, 4, MODE_AG, true>(cp, grid, s) : launch_comm_variant<256, 4, MODE_AG, false>(cp, grid, s);
  if (bn == 192) return a->b_mn_major ? launch_comm_variant<192, 5, MODE_AG, true>(cp, grid, s) : launch_comm_variant<192, 5, MODE_AG, false>(cp, grid, s);
  return a->b_mn_major ? launch_comm_variant<128, 6, MODE_AG, true>(cp, grid, s) : launch_comm_variant<128, 6, MODE_AG, false>(cp, grid, s);
}

// partial[M, N] = x[M, K] * B, rows pushed to their owners' staging; follow with msb_rs_reduce on every rank.
MSB_API int msb_gemm_reduce_scatter(const MsbCommArgs* a, cudaStream_t s) {
  int rc = check_comm(a, "gemm_reduce_scatter");
  if (rc) return rc;
  const int bn = pick_bn(a->M, a->N, msb::num_sms());
  CommParams cp;
  rc = fill_comm(cp, a, MODE_RS, bn);
  if (rc) return rc;
  const long long tiles = (long long)(a->M / BM) * ((a->N + bn - 1) / bn);
  const int sms = msb::num_sms();
  int grid = (int)(tiles < sms ? tiles : sms);
  if (g_cta_limit > 0 && grid > g_cta_limit) grid = g_cta_limit;
  if (bn == 256) return a->b_mn_major ? launch_comm_variant<256, 4, MODE_RS, true>(cp, grid, s) : launch_comm_variant<256, 4, MODE_RS, false>(cp, grid, s);
  if (bn == 192) return a->b_mn_major ? launch_comm_variant<192, 5, MODE_RS, true>(cp, grid, s) : launch_comm_variant<192, 5, MODE_RS, false>(cp, grid, s);
  return a->b_mn_major ? launch_comm_variant<128, 6, MODE_RS, true>(cp, grid, s) : launch_comm_variant<128, 6, MODE_RS, false>(cp, grid, s);
}

// out[rows, N] = sum_r slab_r (+ residual); slab `rank` comes from own_partial, the others from `stage`.
MSB_API int msb_rs_reduce(const void* stage, const void* own_partial, void* out, const void* residual, long long rows, int N,
                          int world, int rank, const unsigned int* flag_local, unsigned int epoch, unsigned int* status,
                          int wait_limit_ms, cudaStream_t s) {
  MSB_REQUIRE(N % 8 == 0, "rs_reduce: N=%d must be a multiple of 8", N);
  const long long n_v4 = rows * N / 8;
  int grid = (int)((n_v4 + 255) / 256);
  if (grid > msb::num_sms() * 8) grid = msb::num_sms() * 8;
  rs_reduce_kernel<<<grid, 256, 0, s>>>((const uint4*)stage, (const uint4*)own_partial, (uint4*)out, (const __nv_bfloat16*)residual,
                                        n_v4, n_v4, world, rank, flag_local, epoch, status,
                                        wait_limit_ms > 0 ? (unsigned long long)wait_limit_ms * 1000000ull : 10000000000ull);
  MSB_CHECK_LAUNCH("rs_reduce");
  return 0;
}
