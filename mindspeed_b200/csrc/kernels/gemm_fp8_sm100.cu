// Block-scaled fp8 (e4m3 / e5m2) GEMM and grouped GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma kind::f8f6f4
// -> TMEM -> scaled promotion in registers -> bf16 / fp32 output.
//
//   D[m, n] = sum over k-blocks kb of  sA[m, kb] * sB[., kb] * ( A_q[m, kb*128 : (kb+1)*128] . B_q[n, same] )
//
// Both operands are K-major fp8: A_q [M, K], B_q [G*N, K] (G weight matrices stacked along rows for the grouped
// form).  Scales: sA is "1 x 128" (one per row per 128 columns), passed TRANSPOSED as [K/128, M] so that the 32
// rows a warp handles read consecutive floats; sB is either "128 x 128" ([G*N/128, K/128], one scalar per tile and
// k-block: weights) or "1 x 128" ([K/128, G*N] transposed like sA: used when both operands are activations, i.e. for
// the weight-gradient GEMM).  This is the scaling scheme of the "blockwise" fp8 recipe
// (mindspeed/te/pytorch/fp8/recipes/float8_block_scaling_recipe.py:15-26) and of DeepSeek-V3 style expert GEMMs
// (mindspeed/core/transformer/moe/grouped_matmul_util.py:138-397 drives the vendor quant-GMM with these scales).
//
// Why promotion in registers: the per-k-block scale differs per row, so partial sums of different k-blocks cannot
// share one tensor-memory accumulator.  Each k-block (128 fp8 = one 128-byte swizzle row, four K=32 MMAs) is
// accumulated into one of four TMEM buffers; while the tensor core works on the next k-block, the eight epilogue warps
// read the finished 128 x 128 partial sum from TMEM and fold it into fp32 registers with one FMA per element.
// Per k-block the tensor core needs ~0.14 us at the fp8 peak and the promotion ~0.1 us, so the two overlap.
//
// Grouped form (MoE experts): rows are laid out expert after expert, each expert padded to a multiple of 128 rows;
// `m_tile_group[m_tile]` names the expert of every 128-row tile (-1 = padding tile, skipped), and selects the row
// offset g*N into B_q and sB.  With G = 1 and a null table the kernel is a plain GEMM.
//
// CTA = 10 warps (TMA producer, MMA issuer, 8 promotion/epilogue warps: 4 lane quarters x 2 column halves), tile
// 128 x 128 x 128, 6 stages of 32 KB.
// All waits are bounded (status word), TMEM is freed on every exit path.
#include "msb_common.cuh"
#include "msb_sm100.cuh"

using namespace msb;
using namespace msb::sm100;

namespace {

constexpr int FBM = 128, FBN = 128, FBK = 128;   // FBK in fp8 elements = bytes
constexpr int FSTAGES = 6;
constexpr int F_UMMA_K = 32;
constexpr int A_BYTES = FBM * FBK, B_BYTES = FBN * FBK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int BAR_OFFSET = FSTAGES * STAGE_BYTES;
constexpr int SMEM_TOTAL = BAR_OFFSET + 256 + 1024;
constexpr int NACC = 4;                          // accumulator buffers in flight (k-blocks between MMA and promotion)
constexpr uint32_t F_TMEM_COLS = 512;            // four 128-column accumulators: the whole tensor memory of the SM

enum FEpi : int { FEPI_BF16 = 0, FEPI_F32 = 1, FEPI_F32_ACC = 2 };

struct Fp8Params {
  CUtensorMap tmA, tmB;
  const float* sA;            // [K/128, M_total]
  const float* sB;            // block: [G*N/128, K/128]   row: [K/128, G*N]
  void* D;                    // [M_total, N]
  const int* m_tile_group;    // [M_total/128] or null
  int M, N, K, G;
  int b_scale_rowwise;
  int fmt_a, fmt_b;           // 0 = e4m3, 1 = e5m2
  long long ldd;
  unsigned int* status;
};

template <int EPI>
__global__ void __launch_bounds__(320, 1) gemm_fp8_blockscaled_kernel(const __grid_constant__ Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (FSTAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * FSTAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * FSTAGES + NACC + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * FSTAGES + 2 * NACC);
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + FBM - 1) / FBM, num_n = (p.N + FBN - 1) / FBN;
  const int num_tiles = num_m * num_n;
  const int num_kb = p.K / FBK;
  // n-major inside groups of 8 m-tiles: concurrently running CTAs share A and B tiles in L2
  auto tile_mn = [&](int t, int& m, int& n) {
    const int gm = 8, per_group = gm * num_n;
    const int g = t / per_group, first = g * gm;
    const int gsz = min(num_m - first, gm);
    const int r = t - g * per_group;
    m = first + (r % gsz);
    n = r / gsz;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < FSTAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < NACC; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 256); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, F_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  bool alive = true;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      tma_prefetch_desc(&p.tmA);
      tma_prefetch_desc(&p.tmB);
      int stage = 0; uint32_t phase = 0;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        int m_blk, n_blk;
        tile_mn(t, m_blk, n_blk);
        const int g = p.m_tile_group ? p.m_tile_group[m_blk] : 0;
        if (g < 0) continue;
        const int m0 = m_blk * FBM, nrow0 = g * p.N + n_blk * FBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 0x410u)) { alive = false; break; }
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          mbar_arrive_expect_tx(full_bar(stage), STAGE_BYTES);
          tma_load_2d(sa, &p.tmA, full_bar(stage), kb * FBK, m0);
          tma_load_2d(sa + A_BYTES, &p.tmB, full_bar(stage), kb * FBK, nrow0);
          if (++stage == FSTAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer: one accumulator buffer per k-block =====================
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f8(FBM, FBN, p.fmt_a, p.fmt_b);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        int m_blk, n_blk;
        tile_mn(t, m_blk, n_blk);
        if (p.m_tile_group && p.m_tile_group[m_blk] < 0) continue;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, p.status, 0x420u)) { alive = false; break; }
          if (!mbar_wait(full_bar(stage), phase, p.status, 0x421u)) { alive = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * FBN);
#pragma unroll
          for (int k = 0; k < FBK / F_UMMA_K; ++k) {
            const uint64_t adesc = make_smem_desc(sa + k * F_UMMA_K, 0, 1024);
            const uint64_t bdesc = make_smem_desc(sb + k * F_UMMA_K, 0, 1024);
            umma_f8f6f4(d_tmem, adesc, bdesc, idesc, k != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));     // shared-memory stage free once these MMAs have read it
          umma_commit(tfull_bar(acc));       // partial sum of this k-block complete
          if (++stage == FSTAGES) { stage = 0; phase ^= 1u; }
          if (++acc == NACC) { acc = 0; acc_phase ^= 1u; }
        }
      }
    }
  } else {
    // ===================== promotion + epilogue (warps 2..9) =====================
    // warp w owns TMEM lanes 32*(w&3).. and the column half (w-2)>>2 of the tile: 64 fp32 accumulators per thread
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int HC = FBN / 2;
    int acc = 0; uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
      int m_blk, n_blk;
      tile_mn(t, m_blk, n_blk);
      const int g = p.m_tile_group ? p.m_tile_group[m_blk] : 0;
      if (g < 0) continue;
      const int row = m_blk * FBM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const int ncol0 = g * p.N + n_blk * FBN;          // column index into the stacked B rows (for row-wise sB)
      const int cbase = half * HC;
      float accum[HC];
#pragma unroll
      for (int c = 0; c < HC; ++c) accum[c] = 0.f;
      const float* sb_blk = p.sB + (long long)(ncol0 / FBN) * num_kb;
      // scales of the next k-block are fetched while the current one is folded in (a global load per k-block would
      // otherwise sit on the critical path of every promotion)
      float sa_next = row_ok ? __ldg(p.sA + row) : 0.f;
      float sbs_next = p.b_scale_rowwise ? 1.f : __ldg(sb_blk);
      for (int kb = 0; kb < num_kb; ++kb) {
        const float sa = sa_next, sbs = sbs_next;
        if (kb + 1 < num_kb) {
          sa_next = row_ok ? __ldg(p.sA + (long long)(kb + 1) * p.M + row) : 0.f;
          if (!p.b_scale_rowwise) sbs_next = __ldg(sb_blk + kb + 1);
        }
        if (!mbar_wait(tfull_bar(acc), acc_phase, p.status, 0x430u)) { alive = false; break; }
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * FBN + cbase);
        if (!p.b_scale_rowwise) {
          const float s = sa * sbs;
#pragma unroll
          for (int c2 = 0; c2 < HC; c2 += 32) {
            uint32_t r0[16], r1[16];                       // two 16-column loads in flight per wait
            tmem_ld_32x16(t_row + (uint32_t)c2, r0);
            tmem_ld_32x16(t_row + (uint32_t)(c2 + 16), r1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              accum[c2 + j] = fmaf(s, __uint_as_float(r0[j]), accum[c2 + j]);
              accum[c2 + 16 + j] = fmaf(s, __uint_as_float(r1[j]), accum[c2 + 16 + j]);
            }
          }
        } else {
          const float* sbrow = p.sB + (long long)kb * ((long long)p.G * p.N) + ncol0 + cbase;
#pragma unroll
          for (int c2 = 0; c2 < HC; c2 += 32) {
            uint32_t r0[16], r1[16];
            tmem_ld_32x16(t_row + (uint32_t)c2, r0);
            tmem_ld_32x16(t_row + (uint32_t)(c2 + 16), r1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int ca = c2 + j, cb = c2 + 16 + j;
              const float sb0 = (n_blk * FBN + cbase + ca < p.N) ? __ldg(sbrow + ca) : 0.f;
              const float sb1 = (n_blk * FBN + cbase + cb < p.N) ? __ldg(sbrow + cb) : 0.f;
              accum[ca] = fmaf(sa * sb0, __uint_as_float(r0[j]), accum[ca]);
              accum[cb] = fmaf(sa * sb1, __uint_as_float(r1[j]), accum[cb]);
            }
          }
        }
        tc_fence_before();
        mbar_arrive(tempty_bar(acc));
        if (++acc == NACC) { acc = 0; acc_phase ^= 1u; }
      }
      if (!alive) break;
      if (row_ok) {
        const int col_base = n_blk * FBN + cbase;
        if (EPI == FEPI_BF16) {
          __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)row * p.ldd + col_base;
          if (col_base + HC <= p.N && ((reinterpret_cast<uintptr_t>(drow) & 15) == 0)) {
#pragma unroll
            for (int v = 0; v < HC / 8; ++v) {
              uint32_t pk[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(accum[v * 8 + 2 * j], accum[v * 8 + 2 * j + 1]);
                pk[j] = *reinterpret_cast<uint32_t*>(&h);
              }
              *reinterpret_cast<uint4*>(drow + v * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          } else {
#pragma unroll
            for (int c = 0; c < HC; ++c) if (col_base + c < p.N) drow[c] = __float2bfloat16_rn(accum[c]);
          }
        } else {
          float* drow = reinterpret_cast<float*>(p.D) + (long long)row * p.ldd + col_base;
          if (col_base + HC <= p.N && ((reinterpret_cast<uintptr_t>(drow) & 15) == 0)) {
#pragma unroll
            for (int v = 0; v < HC / 4; ++v) {
              float4 o = make_float4(accum[4 * v], accum[4 * v + 1], accum[4 * v + 2], accum[4 * v + 3]);
              if (EPI == FEPI_F32_ACC) {
                const float4 old = *reinterpret_cast<float4*>(drow + 4 * v);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(drow + 4 * v) = o;
            }
          } else {
#pragma unroll
            for (int c = 0; c < HC; ++c)
              if (col_base + c < p.N) drow[c] = (EPI == FEPI_F32_ACC) ? drow[c] + accum[c] : accum[c];
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, F_TMEM_COLS);
  }
}

template <int EPI>
int launch_fp8(const Fp8Params& p, int grid, cudaStream_t s) {
  auto kern = gemm_fp8_blockscaled_kernel<EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) { msb_set_error("gemm_fp8: cannot set %d bytes of dynamic shared memory: %s", SMEM_TOTAL, cudaGetErrorString(e)); return 1; }
    attr_set = true;
  }
  kern<<<grid, 320, SMEM_TOTAL, s>>>(p);
  MSB_CHECK_LAUNCH("gemm_fp8_blockscaled");
  return 0;
}

}  // namespace

// D[M_total, N] = blockscaled( A_q[M_total, K], B_q[G*N, K] ).  See the top of the file for layouts.
//   epilogue: 0 = bf16 store, 1 = fp32 store, 2 = fp32 accumulate into D.
//   m_tile_group: null (plain GEMM, G must be 1) or one int per 128-row tile (expert id, -1 = skip).
MSB_API int msb_gemm_fp8_blockscaled(const void* A, const float* sA_t, const void* B, const float* sB, void* D,
                                     const int* m_tile_group, int M_total, int N, int K, int G, int b_scale_rowwise,
                                     int fmt_a, int fmt_b, int epilogue, long long ldd, unsigned int* status, cudaStream_t s) {
  MSB_REQUIRE(A && B && D && sA_t && sB && status, "gemm_fp8: null argument");
  MSB_REQUIRE(M_total > 0 && N > 0 && K > 0 && G >= 1, "gemm_fp8: bad sizes M=%d N=%d K=%d G=%d", M_total, N, K, G);
  MSB_REQUIRE(K % FBK == 0, "gemm_fp8: K=%d must be a multiple of 128", K);
  MSB_REQUIRE(N % 128 == 0 || G == 1, "gemm_fp8: grouped form needs N=%d to be a multiple of 128", N);
  MSB_REQUIRE(b_scale_rowwise || N % 128 == 0, "gemm_fp8: 128x128 weight scales need N=%d to be a multiple of 128", N);
  MSB_REQUIRE(m_tile_group != nullptr || G == 1, "gemm_fp8: grouped form needs the tile -> group table");
  MSB_REQUIRE(m_tile_group == nullptr || M_total % FBM == 0, "gemm_fp8: grouped rows must be padded to multiples of 128");
  MSB_REQUIRE((fmt_a == 0 || fmt_a == 1) && (fmt_b == 0 || fmt_b == 1), "gemm_fp8: formats must be 0 (e4m3) or 1 (e5m2)");
  MSB_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_fp8: bad epilogue %d", epilogue);
  Fp8Params p;
  memset(&p, 0, sizeof(p));
  int rc = make_tmap_2d(&p.tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)M_total, (uint64_t)K, (uint64_t)K, FBM, FBK);
  if (rc) return rc;
  rc = make_tmap_2d(&p.tmB, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)G * N, (uint64_t)K, (uint64_t)K, FBN, FBK);
  if (rc) return rc;
  p.sA = sA_t; p.sB = sB; p.D = D; p.m_tile_group = m_tile_group;
  p.M = M_total; p.N = N; p.K = K; p.G = G; p.b_scale_rowwise = b_scale_rowwise;
  p.fmt_a = fmt_a; p.fmt_b = fmt_b; p.ldd = ldd; p.status = status;
  const long long tiles = (long long)((M_total + FBM - 1) / FBM) * ((N + FBN - 1) / FBN);
  const int sms = msb::num_sms();
  const int grid = (int)(tiles < sms ? tiles : sms);
  if (epilogue == FEPI_BF16) return launch_fp8<FEPI_BF16>(p, grid, s);
  if (epilogue == FEPI_F32) return launch_fp8<FEPI_F32>(p, grid, s);
  return launch_fp8<FEPI_F32_ACC>(p, grid, s);
}
