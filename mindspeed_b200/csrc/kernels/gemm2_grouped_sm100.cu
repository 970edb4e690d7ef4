// Grouped bf16 GEMM on CTA pairs (tcgen05 cta_group::2): one persistent launch covers every expert; the row ranges of the
// experts are read from device memory, so no host synchronisation is needed to launch it.
//
//   GG_ROWS   Y[rows of e, N] = X[rows of e, K] * op(W[e])      forward (W[e] stored [K, N]) and data gradient (W[e] stored
//             [N_out, K_red]): X is K-major, W comes from one 3-D tensor map over the stacked weights [E, ., .]
//   GG_WGRAD  dW[e][Kx, N] (+)= X[rows of e, Kx]^T * dY[rows of e, N]   reduction over the expert's rows, both operands
//             MN-major; output through a 3-D tensor map over the stacked [E, Kx, N] tensor: bf16 / fp32 store or fp32
//             reduce-add (accumulation into main_grad).  Only whole 64-row blocks of every expert are reduced
//             (rows [start_e, start_e + 64 * floor(n_e / 64))); the caller adds the remaining < 64 rows per expert with a
//             second launch on zero-padded copies (mindspeed_b200/ops/grouped_gemm.py).
//
// Expert e owns rows [offs[e], offs[e+1]) (int32 prefix sums in global memory).  A tile is (expert, 256-row block of the
// expert, 256-column block); tiles are numbered expert by expert and dealt round-robin to the CTA pairs; every role
// thread walks the same sequence with a running (expert, first tile of expert) cursor, so finding a tile costs O(1)
// amortised.  In GG_ROWS a 128-row half tile that ends inside the expert's range goes out by TMA store; the last,
// ragged half tile of an expert is written with predicated 16-byte stores so the next expert's rows are not touched.
//
// Pipeline, barriers and epilogue staging are those of gemm2_sm100.cu.
// reference semantics: npu_gmm / npu_gmm_backward (mindspeed/ops/gmm.py:20-175, mindspeed/ops/csrc/cann/gmm.cpp:169-300).
#include "msb_common.cuh"
#include "msb_sm100.cuh"

using namespace msb;
using namespace msb::sm100;

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;

enum GGMode : int { GG_ROWS = 0, GG_WGRAD = 1 };
enum Epi : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ACC = 2 };

struct GroupedParams {
  CUtensorMap tmA;        // GG_ROWS: X [rows, K] box [128 x 64];  GG_WGRAD: X [rows, Kx] box [64 rows x 64]
  CUtensorMap tmB;        // GG_ROWS: W 3-D {inner, outer, E};     GG_WGRAD: dY [rows, N] box [64 rows x 64]
  CUtensorMap tmD;        // GG_ROWS: Y [rows, N] box [32 x 64];   GG_WGRAD: dW 3-D {N, Kx, E} box [64|32, 32, 1]
  const int* offs;        // [E + 1] row prefix sums
  void* D;                // GG_ROWS: Y base for the predicated edge stores
  int E;
  int N;                  // output columns
  int K;                  // GG_ROWS: reduction length; GG_WGRAD: Kx (output rows per expert)
  long long ldd;
  unsigned int* status;
};

template <int NSTAGE, int EPI>
struct SmemG {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BUF = (EPI == EPI_BF16) ? 4096 : 8192;
  static constexpr int EPI_OFFSET = NSTAGE * STAGE_BYTES;
  static constexpr int BAR_OFFSET = EPI_OFFSET + 4 * 2 * EPI_BUF;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
  static_assert(TOTAL <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const void* tmap, uint32_t cluster_bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(cluster_bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(reinterpret_cast<uint64_t>(tmap)),
               "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const void* tmap, uint32_t src, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}

// Walks the tile sequence pair, pair + npairs, ... and yields (expert, m block, n block, row range).
template <int MODE>
struct TileCursor {
  const int* offs;
  int E, num_n, kx_tiles;
  int e, first;           // current expert and the global index of its first tile
  int start, end;         // its row range
  int t, stride;
  __device__ TileCursor(const GroupedParams& p, int pair, int npairs)
      : offs(p.offs), E(p.E), num_n((p.N + BN - 1) / BN), kx_tiles((p.K + 2 * BM - 1) / (2 * BM)), e(-1), first(0), start(0), end(0),
        t(pair), stride(npairs) {}
  __device__ int tiles_of(int s, int en) const {
    if (MODE == GG_ROWS) return ((en - s + 2 * BM - 1) / (2 * BM)) * num_n;
    return (en - s) >= BK ? kx_tiles * num_n : 0;       // no whole 64-row block: nothing to reduce here
  }
  // false when the sequence is exhausted
  __device__ bool next(int& m_blk, int& n_blk) {
    int cnt = (e < 0) ? 0 : tiles_of(start, end);
    while (e < 0 || t >= first + cnt) {
      first += cnt;
      if (++e >= E) return false;
      start = offs[e]; end = offs[e + 1];
      cnt = tiles_of(start, end);
    }
    const int r = t - first;
    // n fastest inside an expert's m block row so pairs running together share the A rows; weights of one expert stay hot in L2
    m_blk = r / num_n;
    n_blk = r - m_blk * num_n;
    t += stride;
    return true;
  }
};

template <int NSTAGE, int MODE, int EPI, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1) gemm2_grouped_kernel(const __grid_constant__ GroupedParams p) {
  using L = SmemG<NSTAGE, EPI>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (NSTAGE + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * NSTAGE + 4);
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  constexpr uint32_t TMEM_COLS = 512u;
  constexpr bool A_MN = (MODE == GG_WGRAD);

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  bool alive = true;
  if (warp == 0) {
    // ===================== TMA producer (both CTAs) =====================
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      TileCursor<MODE> cur(p, pair, npairs);
      int m_blk, n_blk;
      while (alive && cur.next(m_blk, n_blk)) {
        const int n0 = n_blk * BN + (int)cta * (BN / 2);
        int num_kb, m0;
        if (MODE == GG_ROWS) { num_kb = (p.K + BK - 1) / BK; m0 = cur.start + m_blk * (2 * BM) + (int)cta * BM; }
        else { num_kb = (cur.end - cur.start) / BK; m0 = m_blk * (2 * BM) + (int)cta * BM; }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 0x10u)) { alive = false; break; }
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sb = sa + L::A_BYTES;
          if (cta == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
          const uint32_t lead_full = mapa_u32(full_bar(stage), 0);
          if (MODE == GG_ROWS) {
            const int k0 = kb * BK;
            tma_load_2d_pair(sa, &p.tmA, lead_full, k0, m0);                                    // [128 rows x 64 k]
            if (!B_MN) {
              tma_load_3d_pair(sb, &p.tmB, lead_full, k0, n0, cur.e);                           // W[e] stored [N, K]: [128 n x 64 k]
            } else {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j)                                                // W[e] stored [K, N]: [64 k x 64 n]
                tma_load_3d_pair(sb + j * (BK * 128), &p.tmB, lead_full, n0 + j * 64, k0, cur.e);
            }
          } else {
            const int r0 = cur.start + kb * BK;                                                 // 64 rows of the expert
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &p.tmA, lead_full, m0 + j * 64, r0);
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) tma_load_2d_pair(sb + j * (BK * 128), &p.tmB, lead_full, n0 + j * 64, r0);
          }
          if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
        }
      }
      for (int i = 0; i < NSTAGE && alive; ++i) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 0x11u)) { alive = false; break; }
        if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (leader CTA) =====================
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = make_idesc_f16(2 * BM, BN, 1, A_MN ? 1 : 0, (A_MN || B_MN) ? 1 : 0);
      constexpr bool BMN = A_MN || B_MN;
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      TileCursor<MODE> cur(p, pair, npairs);
      int m_blk, n_blk;
      while (alive && cur.next(m_blk, n_blk)) {
        const int num_kb = (MODE == GG_ROWS) ? (p.K + BK - 1) / BK : (cur.end - cur.start) / BK;
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
            const uint64_t adesc = A_MN ? make_smem_desc(sa + k * (UMMA_K * 128), BK * 128, 1024)
                                        : make_smem_desc(sa + k * (UMMA_K * 2), 0, 1024);
            const uint64_t bdesc = BMN ? make_smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024)
                                       : make_smem_desc(sb + k * (UMMA_K * 2), 0, 1024);
            umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage), 3);
          if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        umma_commit_pair(tfull_bar(acc), 3);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ===================== epilogue (warps 2..5, both CTAs) =====================
    const int q = warp & 3;
    const uint32_t buf_base = smem_base + L::EPI_OFFSET + (uint32_t)q * 2u * L::EPI_BUF;
    const uint32_t lead_tempty[2] = {mapa_u32(tempty_bar(0), 0), mapa_u32(tempty_bar(1), 0)};
    int acc = 0; uint32_t acc_phase = 0;
    uint32_t chunk = 0;
    TileCursor<MODE> cur(p, pair, npairs);
    int m_blk, n_blk;
    while (alive && cur.next(m_blk, n_blk)) {
      if (!mbar_wait_warp(tfull_bar(acc), acc_phase, p.status, 0x30u)) { alive = false; break; }
      tc_fence_after();
      // first output row of this warp; GG_ROWS: absolute row of Y, rows at or beyond `limit` belong to the next expert
      const int row0 = (MODE == GG_ROWS ? cur.start : 0) + m_blk * (2 * BM) + (int)cta * BM + q * 32;
      const int limit = (MODE == GG_ROWS) ? cur.end : p.K;
      const bool whole = row0 + 32 <= limit;            // all 32 rows of this warp are inside: TMA store
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
      const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll 1
      for (int c2 = 0; c2 < BN; c2 += 64, ++chunk) {
        const int col0 = n_blk * BN + c2;
        if (col0 >= p.N) break;
        uint32_t rr[2][32];
        tmem_ld_32x32(t_row + (uint32_t)c2, rr[0]);
        tmem_ld_32x32(t_row + (uint32_t)(c2 + 32), rr[1]);
        tmem_ld_wait();
        if (MODE == GG_ROWS && !whole) {
          // ragged end of an expert: predicated stores straight from registers (bf16 output only in this mode)
          const int row = row0 + lane;
          if (row < limit) {
            __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)row * p.ldd + col0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (col0 + 8 * j + 8 <= p.N) {
                uint32_t pk[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int c = 8 * j + 2 * e;
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(rr[c >> 5][c & 31]), __uint_as_float(rr[(c + 1) >> 5][(c + 1) & 31]));
                  pk[e] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(drow + 8 * j) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              }
            }
          }
          if (lane == 0) tma_store_commit();            // keeps the one-group-per-chunk count of the staging buffers
          continue;
        }
        const uint32_t buf = buf_base + (chunk & 1u) * L::EPI_BUF;
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        const uint32_t row_addr = buf + (uint32_t)lane * 128u;
        if (EPI == EPI_BF16) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int c = 8 * j + 2 * e;
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(rr[c >> 5][c & 31]), __uint_as_float(rr[(c + 1) >> 5][(c + 1) & 31]));
              pk[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + ((((uint32_t)j) ^ sw) << 4)), "r"(pk[0]), "r"(pk[1]),
                         "r"(pk[2]), "r"(pk[3])
                         : "memory");
          }
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (uint32_t)h * 4096u + ((((uint32_t)j) ^ sw) << 4)),
                           "r"(rr[h][4 * j]), "r"(rr[h][4 * j + 1]), "r"(rr[h][4 * j + 2]), "r"(rr[h][4 * j + 3])
                           : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (row0 < limit) {
            if (MODE == GG_ROWS) {
              tma_store_2d(&p.tmD, buf, col0, row0);
            } else if (EPI == EPI_BF16) {
              tma_store_3d(&p.tmD, buf, col0, row0, cur.e);
            } else if (EPI == EPI_F32) {
              tma_store_3d(&p.tmD, buf, col0, row0, cur.e);
              if (col0 + 32 < p.N) tma_store_3d(&p.tmD, buf + 4096u, col0 + 32, row0, cur.e);
            } else {
              tma_reduce_add_3d(&p.tmD, buf, col0, row0, cur.e);
              if (col0 + 32 < p.N) tma_reduce_add_3d(&p.tmD, buf + 4096u, col0 + 32, row0, cur.e);
            }
          }
          tma_store_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_tempty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int NSTAGE, int MODE, int EPI, bool B_MN>
int launch_grouped(const GroupedParams& p, int pairs, cudaStream_t s) {
  using L = SmemG<NSTAGE, EPI>;
  auto kern = gemm2_grouped_kernel<NSTAGE, MODE, EPI, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) { msb_set_error("gemm2_grouped: cannot set %d bytes of dynamic shared memory: %s", L::TOTAL, cudaGetErrorString(e)); return 1; }
    attr_set = true;
  }
  kern<<<2 * pairs, 192, L::TOTAL, s>>>(p);
  MSB_CHECK_LAUNCH("gemm2_grouped");
  return 0;
}

int make_map3(CUtensorMap* tm, const void* base, CUtensorMapDataType dt, int esz, uint64_t inner, uint64_t outer, uint64_t E,
              uint32_t box_inner, uint32_t box_outer) {
  uint64_t dims[3] = {inner, outer, E};
  uint64_t str[2] = {inner * (uint64_t)esz, inner * outer * (uint64_t)esz};
  uint32_t box[3] = {box_inner, box_outer, 1};
  return make_tmap_nd(tm, base, dt, esz, 3, dims, str, box);
}

}  // namespace

// Y[rows of e, N] = X[rows of e, K] * op(W[e]) for every expert e; offs = int32 [E + 1] row prefix sums ON THE DEVICE.
//   w_is_kn = 1: W stacked [E, K, N] (forward);  w_is_kn = 0: W stacked [E, N, K] (data gradient: y = dy W^T)
// X [rows_total, K] and Y [rows_total, N] bf16 contiguous; rows_total bounds the tensor maps (rows beyond offs[E] are untouched).
MSB_API int msb_grouped_gemm_rows(const void* X, const void* W, void* Y, const int* offs, int E, int rows_total, int N, int K,
                                  int w_is_kn, unsigned int* status, cudaStream_t s) {
  MSB_REQUIRE(E > 0 && rows_total > 0 && N % 8 == 0 && K % 8 == 0, "grouped_gemm_rows: bad shape E=%d rows=%d N=%d K=%d", E, rows_total, N, K);
  MSB_REQUIRE(status != nullptr, "grouped_gemm_rows: status word is required");
  GroupedParams p;
  memset(&p, 0, sizeof(p));
  int rc = make_tmap_2d(&p.tmA, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, K, K, BM, BK);
  if (rc) return rc;
  if (w_is_kn) rc = make_map3(&p.tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, E, 64, BK);        // [64 k x 64 n] boxes
  else rc = make_map3(&p.tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, E, BK, BN / 2);            // [128 n x 64 k] boxes
  if (rc) return rc;
  rc = make_tmap_2d(&p.tmD, Y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, N, N, 32, 64);
  if (rc) return rc;
  p.offs = offs; p.D = Y; p.E = E; p.N = N; p.K = K; p.ldd = N; p.status = status;
  const int pairs = msb::num_sms() / 2;
  return w_is_kn ? launch_grouped<6, GG_ROWS, EPI_BF16, true>(p, pairs, s) : launch_grouped<6, GG_ROWS, EPI_BF16, false>(p, pairs, s);
}

// dW[e][Kx, N] (+)= X[rows of e, Kx]^T * dY[rows of e, N] over the whole 64-row blocks of every expert.
//   epilogue 0: bf16 store, 1: fp32 store, 2: fp32 accumulate.  Experts with fewer than 64 rows are not written at all.
MSB_API int msb_grouped_gemm_wgrad(const void* X, const void* dY, void* dW, const int* offs, int E, int rows_total, int Kx, int N,
                                   int epilogue, unsigned int* status, cudaStream_t s) {
  MSB_REQUIRE(E > 0 && rows_total > 0 && N % 8 == 0 && Kx % 8 == 0, "grouped_gemm_wgrad: bad shape E=%d rows=%d Kx=%d N=%d", E, rows_total, Kx, N);
  MSB_REQUIRE(status != nullptr, "grouped_gemm_wgrad: status word is required");
  GroupedParams p;
  memset(&p, 0, sizeof(p));
  int rc = make_tmap_2d(&p.tmA, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, Kx, Kx, BK, 64);
  if (rc) return rc;
  rc = make_tmap_2d(&p.tmB, dY, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, N, N, BK, 64);
  if (rc) return rc;
  if (epilogue == EPI_BF16) rc = make_map3(&p.tmD, dW, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, Kx, E, 64, 32);
  else rc = make_map3(&p.tmD, dW, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, N, Kx, E, 32, 32);
  if (rc) return rc;
  p.offs = offs; p.D = dW; p.E = E; p.N = N; p.K = Kx; p.ldd = N; p.status = status;
  const int pairs = msb::num_sms() / 2;
  switch (epilogue) {
    case EPI_BF16: return launch_grouped<6, GG_WGRAD, EPI_BF16, true>(p, pairs, s);
    case EPI_F32: return launch_grouped<5, GG_WGRAD, EPI_F32, true>(p, pairs, s);
    case EPI_F32_ACC: return launch_grouped<5, GG_WGRAD, EPI_F32_ACC, true>(p, pairs, s);
  }
  msb_set_error("grouped_gemm_wgrad: unknown epilogue %d", epilogue);
  return 2;
}
