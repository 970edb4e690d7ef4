// bf16 GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a:  D[M,N] (+)= A[M,K] * B[K,N], fp32 accumulation in TMEM.
//
// Two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x BN output tile.  Each CTA loads its own 128 rows of A and
// its own half of the B columns with plain TMA loads (no load is shared between CTAs), the even CTA issues one 256-row
// tcgen05.mma per 16 k that reads both CTAs' shared memory, and each CTA ends up with its 128 x BN accumulator rows in its
// own tensor memory.  Against the one-CTA kernel (gemm_sm100.cu) every CTA stages half as many B bytes per MMA, which is
// what the shared-memory bandwidth of one SM needs to keep a 256-wide tile fed.
//
// Per CTA, 6 warps: warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane, leader CTA only; the warp also owns
// the TMEM allocation in both CTAs), warps 2-5 = epilogue.  Persistent over tiles (grid = CTA pairs), two accumulators in
// TMEM so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Epilogue: TMEM -> registers -> 128B-swizzled shared-memory staging (per warp, double buffered) -> TMA store of
// [32 rows x 64 columns] boxes (bf16) or [32 x 32] boxes (fp32).  The accumulate-in-place form (weight gradient into the
// fp32 main_grad) is a TMA reduce-add, so the old value is never read into the SM.  Edges are clipped by TMA.
//
// Barrier protocol (s = pipeline stage, a = accumulator):
//   full[s]   leader only; the leader's producer arrives with expect_tx = both CTAs' stage bytes, both CTAs' loads
//             complete_tx on it (the second CTA addresses it through its cluster-wide address)
//   empty[s]  in each CTA; the MMA thread's commit arrives on both (stage may be overwritten)
//   tfull[a]  in each CTA; commit after the last k-block arrives on both (accumulator complete)
//   tempty[a] leader only; one arrive per epilogue warp of both CTAs (8) once the accumulator has been read
// Every wait is bounded (msb_sm100.cuh); a time-out sets the status word and all roles fall through to the teardown.
//
// Operand layouts as in gemm_sm100.cu: A "K-major" [M,K] or "MN-major" [K,M]; B "K-major" [N,K] or "MN-major" [K,N].
// reference semantics being replaced: torch.matmul in the parallel linears and npu_matmul_add_fp32
// (mindspeed/ops/npu_matmul_add.py:51-66).
#include "msb_common.cuh"
#include "msb_sm100.cuh"

using namespace msb;
using namespace msb::sm100;

namespace {

constexpr int BM = 128;          // rows per CTA; the pair covers 256
constexpr int BK = 64;           // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;

enum Epi : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ACC = 2 };

struct Gemm2Params {
  CUtensorMap tmA, tmB, tmD;
  const void* bias;            // optional bf16 [N] (bf16 epilogue only)
  int M, N, K;
  int group_m;                 // 256-row tile rows per L2 group
  int stream_k;                // accumulate epilogue only: split the (tile, k-block) space evenly over the CTA pairs
  unsigned int* status;
};

// The sequence of work items of one CTA pair; producer, MMA and epilogue roles each walk their own copy.
//   static    whole tiles pair, pair + npairs, ...: pairs running at the same time work on neighbouring tiles, which
//             share A and B panels in L2
//   stream-K  the full waves run as above; the tiles of the last, partial wave are cut along K so that every pair gets
//             the same number of k-blocks of them.  A tile cut this way is finished by several pairs, each adding its
//             partial sum into global memory (only valid with the reduce-add epilogue).
struct WorkIter {
  int tile, kb0, kb1;
  int next_tile, stride, full_tiles, num_kb;
  long long u, u_end;
  __device__ WorkIter(int pair, int npairs, int num_tiles, int num_kb_, bool sk)
      : tile(0), kb0(0), kb1(0), next_tile(pair), stride(npairs), num_kb(num_kb_) {
    full_tiles = sk ? (num_tiles / npairs) * npairs : num_tiles;
    const long long tail = (long long)(num_tiles - full_tiles) * num_kb_;
    u = (long long)full_tiles * num_kb_ + tail * pair / npairs;
    u_end = (long long)full_tiles * num_kb_ + tail * (pair + 1) / npairs;
  }
  __device__ bool next() {
    if (next_tile < full_tiles) {
      tile = next_tile; next_tile += stride; kb0 = 0; kb1 = num_kb;
      return true;
    }
    if (u >= u_end) return false;
    tile = (int)(u / num_kb);
    kb0 = (int)(u - (long long)tile * num_kb);
    const long long e = min(u_end, (long long)(tile + 1) * num_kb);
    kb1 = kb0 + (int)(e - u);
    u = e;
    return true;
  }
};

template <int BN, int NSTAGE, int EPI>
struct Smem2 {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BUF = (EPI == EPI_BF16) ? 4096 : 8192;   // 32 rows x 64 columns of the output type
  static constexpr int EPI_OFFSET = NSTAGE * STAGE_BYTES;
  static constexpr int BAR_OFFSET = EPI_OFFSET + 4 * 2 * EPI_BUF;    // 4 warps, double buffered
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;              // barriers + alignment slack
  static_assert(TOTAL <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

__device__ __forceinline__ void tile_coords2(int t, int num_m, int num_n, int group_m, int& m, int& n) {
  const int per_group = group_m * num_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsz = min(num_m - first_m, group_m);
  const int r = t - g * per_group;
  m = first_m + (r % gsz);
  n = r / gsz;
}

template <int BN, int NSTAGE, int EPI, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1) gemm2_sm100_kernel(const __grid_constant__ Gemm2Params p) {
  using L = Smem2<BN, NSTAGE, EPI>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // identical in both CTAs of the pair
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (NSTAGE + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * NSTAGE + 4);
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();                 // 0 = leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int num_m = (p.M + 2 * BM - 1) / (2 * BM), num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = (BN <= 128) ? 256u : 512u;   // two accumulators of BN columns
  const bool sk = (EPI == EPI_F32_ACC) && p.stream_k != 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();          // barriers of both CTAs are initialised before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  bool alive = true;
  if (warp == 0) {
    // ===================== TMA producer (both CTAs) =====================
    if (lane == 0) {
      tma_prefetch_desc(&p.tmA);
      tma_prefetch_desc(&p.tmB);
      int stage = 0; uint32_t phase = 0;
      WorkIter it(pair, npairs, num_tiles, num_kb, sk);
      while (alive && it.next()) {
        int m_blk, n_blk;
        tile_coords2(it.tile, num_m, num_n, p.group_m, m_blk, n_blk);
        const int m0 = m_blk * (2 * BM) + (int)cta * BM;
        const int n0 = n_blk * BN + (int)cta * (BN / 2);
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 0x10u)) { alive = false; break; }
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sb = sa + L::A_BYTES;
          if (cta == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
          const uint32_t lead_full = mapa_u32(full_bar(stage), 0);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d_pair(sa, &p.tmA, lead_full, k0, m0);                           // box [128 rows x 64 k]
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)                                          // boxes [64 k x 64 m]
              tma_load_2d_pair(sa + j * (BK * 128), &p.tmA, lead_full, m0 + j * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &p.tmB, lead_full, k0, n0);                           // box [BN/2 rows x 64 k]
          } else {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)                                         // boxes [64 k x 64 n]
              tma_load_2d_pair(sb + j * (BK * 128), &p.tmB, lead_full, n0 + j * 64, k0);
          }
          if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
        }
      }
      // tail: every commit aimed at this CTA's empty barriers must have landed before the CTA may exit
      for (int i = 0; i < NSTAGE && alive; ++i) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 0x11u)) { alive = false; break; }
        if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (leader CTA, one thread) =====================
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = make_idesc_f16(2 * BM, BN, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      WorkIter it(pair, npairs, num_tiles, num_kb, sk);
      while (alive && it.next()) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, p.status, 0x20u)) { alive = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
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
            umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb != it.kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage), 3);      // both CTAs may refill this stage once these MMAs have read it
          if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        umma_commit_pair(tfull_bar(acc), 3);          // accumulator complete in both CTAs
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ===================== epilogue (warps 2..5, both CTAs) =====================
    const int q = warp & 3;                          // TMEM lane quarter this warp may access
    const uint32_t buf_base = smem_base + L::EPI_OFFSET + (uint32_t)q * 2u * L::EPI_BUF;
    const uint32_t lead_tempty[2] = {mapa_u32(tempty_bar(0), 0), mapa_u32(tempty_bar(1), 0)};
    int acc = 0; uint32_t acc_phase = 0;
    uint32_t chunk = 0;
    WorkIter it(pair, npairs, num_tiles, num_kb, sk);
    while (alive && it.next()) {
      int m_blk, n_blk;
      tile_coords2(it.tile, num_m, num_n, p.group_m, m_blk, n_blk);
      if (!mbar_wait_warp(tfull_bar(acc), acc_phase, p.status, 0x30u)) { alive = false; break; }
      tc_fence_after();
      const int row0 = m_blk * (2 * BM) + (int)cta * BM + q * 32;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
      const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll 1
      for (int c2 = 0; c2 < BN; c2 += 64, ++chunk) {
        const int col0 = n_blk * BN + c2;
        if (col0 >= p.N) break;                       // the rest of this tile is beyond the last column
        uint32_t rr[2][32];
        tmem_ld_32x32(t_row + (uint32_t)c2, rr[0]);
        tmem_ld_32x32(t_row + (uint32_t)(c2 + 32), rr[1]);
        tmem_ld_wait();
        const uint32_t buf = buf_base + (chunk & 1u) * L::EPI_BUF;
        if (lane == 0) tma_store_wait_read<1>();      // the store that last read this buffer (two chunks ago) is done with it
        __syncwarp();
        const uint32_t row_addr = buf + (uint32_t)lane * 128u;
        if (EPI == EPI_BF16) {
          const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.bias);
#pragma unroll
          for (int j = 0; j < 8; ++j) {                 // 16-byte chunk j = columns 8j .. 8j+7
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int c = 8 * j + 2 * e;
              float a = __uint_as_float(rr[c >> 5][c & 31]), b = __uint_as_float(rr[(c + 1) >> 5][(c + 1) & 31]);
              if (bias) {
                if (col0 + c < p.N) a += __bfloat162float(bias[col0 + c]);
                if (col0 + c + 1 < p.N) b += __bfloat162float(bias[col0 + c + 1]);
              }
              __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
              pk[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + ((((uint32_t)j) ^ sw) << 4)), "r"(pk[0]), "r"(pk[1]),
                         "r"(pk[2]), "r"(pk[3])
                         : "memory");
          }
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h)                   // two [32 x 32] fp32 boxes per 64 columns
#pragma unroll
            for (int j = 0; j < 8; ++j)                 // 16-byte chunk j = columns 4j .. 4j+3 of the box
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (uint32_t)h * 4096u + ((((uint32_t)j) ^ sw) << 4)),
                           "r"(rr[h][4 * j]), "r"(rr[h][4 * j + 1]), "r"(rr[h][4 * j + 2]), "r"(rr[h][4 * j + 3])
                           : "memory");
        }
        fence_proxy_async_smem();                       // generic-proxy writes -> visible to the TMA store
        __syncwarp();
        if (lane == 0) {
          if (row0 < p.M) {
            if (EPI == EPI_BF16) {
              tma_store_2d(&p.tmD, buf, col0, row0);
            } else if (EPI == EPI_F32) {
              tma_store_2d(&p.tmD, buf, col0, row0);
              if (col0 + 32 < p.N) tma_store_2d(&p.tmD, buf + 4096u, col0 + 32, row0);
            } else {
              tma_reduce_add_2d(&p.tmD, buf, col0, row0);
              if (col0 + 32 < p.N) tma_reduce_add_2d(&p.tmD, buf + 4096u, col0 + 32, row0);
            }
          }
          tma_store_commit();                           // one group per chunk, empty or not: the wait above counts groups
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_tempty[acc]);   // this warp has read its lanes of the accumulator
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) tma_store_wait<0>();                 // staging buffers are read and the stores are complete before exit
  }

  // ---- teardown: both CTAs meet, TMEM is returned ----
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int BN, int NSTAGE, int EPI, bool A_MN, bool B_MN>
int launch2_variant(const Gemm2Params& p, int pairs, cudaStream_t s) {
  using L = Smem2<BN, NSTAGE, EPI>;
  auto kern = gemm2_sm100_kernel<BN, NSTAGE, EPI, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) { msb_set_error("gemm2_sm100: cannot set %d bytes of dynamic shared memory: %s", L::TOTAL, cudaGetErrorString(e)); return 1; }
    attr_set = true;
  }
  kern<<<2 * pairs, 192, L::TOTAL, s>>>(p);
  MSB_CHECK_LAUNCH("gemm2_sm100");
  return 0;
}

template <int BN, int NSTAGE, int EPI>
int launch2_major(const Gemm2Params& p, int a_mn, int b_mn, int pairs, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch2_variant<BN, NSTAGE, EPI, false, false>(p, pairs, s);
  if (!a_mn && b_mn) return launch2_variant<BN, NSTAGE, EPI, false, true>(p, pairs, s);
  if (a_mn && b_mn) return launch2_variant<BN, NSTAGE, EPI, true, true>(p, pairs, s);
  return launch2_variant<BN, NSTAGE, EPI, true, false>(p, pairs, s);
}

}  // namespace

namespace msb {

// True when the CTA-pair kernel can run this problem: TMA-store friendly output (16-byte aligned base and row pitch).
bool gemm2_eligible(const void* D, long long ldd, int epilogue) {
  const int esz = epilogue == EPI_BF16 ? 2 : 4;
  return (reinterpret_cast<uintptr_t>(D) & 15) == 0 && (ldd * esz) % 16 == 0;
}

// D[M,N] (+)= A * B on CTA pairs with 256 x `bn` tiles (bn = 256 or 128); at most `max_ctas` CTAs (0 = all SMs).
// `stream_k` (accumulate epilogue only) balances k-blocks instead of tiles over the pairs; partial tiles are summed in
// global memory in an order that varies from run to run, so callers that need bit-reproducible sums pass 0.
int gemm2_launch(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, long long lda, long long ldb,
                 long long ldd, int a_mn, int b_mn, int epilogue, int bn, int max_ctas, int stream_k, unsigned int* status,
                 cudaStream_t s) {
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  int rc;
  if (!a_mn) rc = make_tmap_2d(&p.tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK);
  else rc = make_tmap_2d(&p.tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_2d(&p.tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, bn / 2, BK);
  else rc = make_tmap_2d(&p.tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64);
  if (rc) return rc;
  if (epilogue == EPI_BF16) rc = make_tmap_2d(&p.tmD, D, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldd, 32, 64);
  else rc = make_tmap_2d(&p.tmD, D, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldd, 32, 32);
  if (rc) return rc;
  p.bias = bias;
  p.M = M; p.N = N; p.K = K;
  p.status = status;
  const int num_m = (M + 2 * BM - 1) / (2 * BM);
  const long long tiles = (long long)num_m * ((N + bn - 1) / bn);
  p.group_m = num_m < 8 ? num_m : 8;
  int pairs = msb::num_sms() / 2;
  if (max_ctas > 0 && pairs > max_ctas / 2) pairs = max_ctas / 2;
  if (pairs < 1) pairs = 1;
  p.stream_k = (epilogue == EPI_F32_ACC && stream_k) ? 1 : 0;
  if (!p.stream_k && tiles < pairs) pairs = (int)tiles;
  if (p.stream_k) {
    const long long units = tiles * ((K + BK - 1) / BK);
    if (units < pairs) pairs = (int)units;
  }
  if (bn == 256) {
    switch (epilogue) {
      case EPI_BF16: return launch2_major<256, 6, EPI_BF16>(p, a_mn, b_mn, pairs, s);
      case EPI_F32: return launch2_major<256, 5, EPI_F32>(p, a_mn, b_mn, pairs, s);
      case EPI_F32_ACC: return launch2_major<256, 5, EPI_F32_ACC>(p, a_mn, b_mn, pairs, s);
    }
  } else {
    switch (epilogue) {
      case EPI_BF16: return launch2_major<128, 8, EPI_BF16>(p, a_mn, b_mn, pairs, s);
      case EPI_F32: return launch2_major<128, 6, EPI_F32>(p, a_mn, b_mn, pairs, s);
      case EPI_F32_ACC: return launch2_major<128, 6, EPI_F32_ACC>(p, a_mn, b_mn, pairs, s);
    }
  }
  msb_set_error("gemm2_sm100: unknown epilogue %d", epilogue);
  return 2;
}

}  // namespace msb
