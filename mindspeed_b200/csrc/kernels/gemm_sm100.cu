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
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: power of two

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
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + (uint32_t)c, r);
          tmem_ld_wait();
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
  // fewer, larger tiles unless the last wave would be mostly idle
  auto eff = [&](int bn) {
    long long tiles = (long long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    long long waves = (tiles + sms - 1) / sms;
    return (double)tiles / (double)(waves * sms);
  };
  if (N <= 128) return 128;
  double e256 = eff(256), e128 = eff(128);
  return (e128 > e256 * 1.12) ? 128 : 256;
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

MSB_API int msb_gemm_bf16_ex(const MsbGemmArgs* a, cudaStream_t s) {
  MSB_REQUIRE(a->M > 0 && a->N > 0 && a->K > 0, "gemm: empty problem %dx%dx%d", a->M, a->N, a->K);
  MSB_REQUIRE(a->nsrc >= 1 && a->nsrc <= MAX_SRC && a->ndst >= 1 && a->ndst <= MAX_SRC, "gemm: bad source/destination count");
  MSB_REQUIRE(a->status != nullptr, "gemm: status word is required");
  MSB_REQUIRE(a->a_rows_per_src % BM == 0 || a->nsrc == 1, "gemm: rows per A source must be a multiple of %d", BM);
  MSB_REQUIRE(a->d_rows_per_dst % 32 == 0 || a->ndst == 1, "gemm: rows per destination must be a multiple of 32");
  const int sms = msb::num_sms();
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
  if (bn == 256) return launch_epi<256, 4>(p, a->epilogue, a->a_mn_major, a->b_mn_major, grid, s);
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
