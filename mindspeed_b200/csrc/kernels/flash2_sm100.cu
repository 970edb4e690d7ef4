// Flash attention forward for sm_100a, two query tiles per CTA: while the softmax warps of one tile work, the tensor core
// runs the other tile's MMAs.  head_dim 128, bf16, causal or full, GQA, query offset (for chunked / ring use).
//
// One CTA owns 256 query rows (two tiles of 128) of one (batch, head) and walks the key/value tiles of 128 keys.
//   TMEM (512 columns)  S0 | S1 | O0 | O1, 128 fp32 columns each.  The probabilities P_t overwrite the first 64 columns of
//                       S_t as packed bf16 and feed the P V MMA as its A operand straight from tensor memory.
//   warp 0              TMA producer: Q0 and Q1 once, K_j and V_j into separate 2-stage rings
//   warp 1              MMA issuer (one thread):  S_t = Q_t K_j^T,  O_t += P_t V_j.  Issue order
//                       S0 S1 | PV0 S0' | PV1 S1' | ...   so tile t's softmax overlaps the other tile's MMAs
//   warps 2-5 / 6-9     softmax of tile 0 / tile 1, one thread per query row: row maximum, exp2, row sum, P -> TMEM.
//                       O stays in tensor memory; it is rescaled only when the running maximum grew by more than 2^8
//                       since the last rescale (the stale maximum is used for P meanwhile, which stays within range),
//                       so most key tiles never touch O.
// Epilogue: O / l -> bf16 -> shared memory (the tile's Q buffer) -> TMA store; LSE (natural log) to global memory.
// reference semantics: torch_npu.npu_fusion_attention returning softmax max/sum
// (mindspeed/core/transformer/flash_attention/flash_attention/adaptor.py:21-85, mindspeed/ops/fusion_attention_v2.py:22-114).
#include "msb_common.cuh"
#include "msb_sm100.cuh"

using namespace msb;
using namespace msb::sm100;

namespace {
constexpr int FB = 128;                   // rows per Q tile, keys per KV tile
constexpr int FD = 128;                   // head dim
constexpr int TILE_BYTES = FB * FD * 2;   // 32 KB
constexpr int HALF_BYTES = FB * 128;      // one 64-wide column block: 128 rows x 128 B
constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units

struct Fwd2Params {
  CUtensorMap tmQ, tmK, tmV, tmO;  // dims {d, head, batch, seq}
  float* lse;                      // [b, nq, sq]
  __nv_bfloat16* O;                // [sq, b, nq, d] (direct stores for rows without any visible key)
  int sq, sk, b, nq, nkv;
  int causal;
  int q_offset;                    // key index visible to query row r is <= r + q_offset
  float scale_log2;                // softmax_scale * log2(e)
  unsigned int* status;
};

struct Fwd2Smem {
  static constexpr int Q_OFF = 0;                          // 2 tiles
  static constexpr int K_OFF = 2 * TILE_BYTES;             // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * TILE_BYTES;     // 2 stages
  static constexpr int BAR_OFF = V_OFF + 2 * TILE_BYTES;   // 192 KB
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ void named_bar(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

__device__ __forceinline__ void tma_store_4d(const void* tmap, uint32_t src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(src), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}

__global__ void __launch_bounds__(320, 1) flash_fwd2_sm100_kernel(const __grid_constant__ Fwd2Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar = base + Fwd2Smem::BAR_OFF;
  const uint32_t q_full = bar;
  auto k_full = [&](int s) { return bar + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar + 8u * (7 + s); };
  auto s_full = [&](int t) { return bar + 8u * (9 + t); };
  auto p_full = [&](int t) { return bar + 8u * (11 + t); };
  auto pv_done = [&](int t) { return bar + 8u * (13 + t); };
  const uint32_t tmem_slot = bar + 8u * 15;
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(base_ptr + Fwd2Smem::BAR_OFF + 8 * 15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first so the causal triangle balances across the grid
  const int m_blk = (p.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x);
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.nq / p.nkv);
  const int q0 = m_blk * 2 * FB;
  const int n_all = (p.sk + FB - 1) / FB;
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    int n = n_all;
    const int first = q0 + t * FB;
    if (first >= p.sq) n = 0;
    else if (p.causal) {
      const int last_key = min(first + FB - 1, p.sq - 1) + p.q_offset;    // last key any row of this tile may see
      n = last_key < 0 ? 0 : min(n, last_key / FB + 1);
    }
    n_t[t] = n;
  }
  const int n_max = max(n_t[0], n_t[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1); mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(s_full(t), 1); mbar_init(p_full(t), 4); mbar_init(pv_done(t), 1); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0 && n_max > 0) {
      mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const uint32_t qs = base + Fwd2Smem::Q_OFF + t * TILE_BYTES;
        tma_load_4d(qs, &p.tmQ, q_full, 0, head, batch, q0 + t * FB);
        tma_load_4d(qs + HALF_BYTES, &p.tmQ, q_full, 64, head, batch, q0 + t * FB);
      }
      bool ok = true;
      for (int j = 0; j < n_max && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!mbar_wait(k_empty(s), ph ^ 1u, p.status, 0x310u)) { ok = false; break; }
        mbar_arrive_expect_tx(k_full(s), TILE_BYTES);
        const uint32_t ks = base + Fwd2Smem::K_OFF + s * TILE_BYTES;
        tma_load_4d(ks, &p.tmK, k_full(s), 0, kv_head, batch, j * FB);
        tma_load_4d(ks + HALF_BYTES, &p.tmK, k_full(s), 64, kv_head, batch, j * FB);
        if (!mbar_wait(v_empty(s), ph ^ 1u, p.status, 0x311u)) { ok = false; break; }
        mbar_arrive_expect_tx(v_full(s), TILE_BYTES);
        const uint32_t vs = base + Fwd2Smem::V_OFF + s * TILE_BYTES;
        tma_load_4d(vs, &p.tmV, v_full(s), 0, kv_head, batch, j * FB);
        tma_load_4d(vs + HALF_BYTES, &p.tmV, v_full(s), 64, kv_head, batch, j * FB);
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0 && n_max > 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(128, 128, 1, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_f16(128, 128, 1, 0, 1);
      auto issue_s = [&](int t, int j) {
        const uint32_t qs = base + Fwd2Smem::Q_OFF + t * TILE_BYTES, ks = base + Fwd2Smem::K_OFF + (j & 1) * TILE_BYTES;
        const uint32_t tS = tmem_base + (uint32_t)(t * 128);
#pragma unroll
        for (int k = 0; k < FD / 16; ++k) {
          const uint32_t off = (uint32_t)((k >> 2) * HALF_BYTES + (k & 3) * 32);
          umma_f16(tS, make_smem_desc(qs + off, 0, 1024), make_smem_desc(ks + off, 0, 1024), idesc_qk, k ? 1u : 0u);
        }
        umma_commit(s_full(t));
      };
      auto issue_pv = [&](int t, int j) {
        const uint32_t vs = base + Fwd2Smem::V_OFF + (j & 1) * TILE_BYTES;
        const uint32_t tP = tmem_base + (uint32_t)(t * 128), tO = tmem_base + 256u + (uint32_t)(t * 128);
#pragma unroll
        for (int k = 0; k < FB / 16; ++k) {
          const uint64_t bdesc = make_smem_desc(vs + (uint32_t)(k * 16 * 128), HALF_BYTES, 1024);   // MN-major: 16 keys = 2048 B
          umma_f16_ts(tO, tP + (uint32_t)(k * 8), bdesc, idesc_pv, (j | k) ? 1u : 0u);               // 16 bf16 of P = 8 columns
        }
        umma_commit(pv_done(t));
      };
      bool ok = mbar_wait(q_full, 0, p.status, 0x320u);
      if (ok) ok = mbar_wait(k_full(0), 0, p.status, 0x321u);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t) if (n_t[t] > 0) issue_s(t, 0);
        umma_commit(k_empty(0));
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const uint32_t ph = (uint32_t)((j >> 1) & 1), jp = (uint32_t)(j & 1);
        if (!mbar_wait(v_full(j & 1), ph, p.status, 0x322u)) { ok = false; break; }
        bool k_next_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j < n_t[t]) {
            if (!mbar_wait(p_full(t), jp, p.status, 0x323u)) { ok = false; break; }
            tc_fence_after();
            issue_pv(t, j);
          }
          if (j + 1 < n_t[t]) {
            if (!k_next_ready) {
              if (!mbar_wait(k_full((j + 1) & 1), (uint32_t)(((j + 1) >> 1) & 1), p.status, 0x324u)) { ok = false; break; }
              tc_fence_after();
              k_next_ready = true;
            }
            issue_s(t, j + 1);
          }
        }
        if (!ok) break;
        umma_commit(v_empty(j & 1));
        if (j + 1 < n_max) umma_commit(k_empty((j + 1) & 1));
      }
    }
  } else {
    // ===================== softmax (warps 2-5: tile 0, warps 6-9: tile 1) =====================
    const int t = (warp - 2) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;                 // row inside the tile == TMEM lane
    const int q_idx = q0 + t * FB + row;
    const uint32_t lane_addr = ((uint32_t)(q * 32) << 16);
    const uint32_t tS = tmem_base + (uint32_t)(t * 128) + lane_addr;
    const uint32_t tO = tmem_base + 256u + (uint32_t)(t * 128) + lane_addr;
    const int n_kv = n_t[t];
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const uint32_t jp = (uint32_t)(j & 1);
      if (!mbar_wait(s_full(t), jp, p.status, 0x330u)) { ok = false; break; }
      tc_fence_after();
      const int key0 = j * FB;
      const int limit = p.causal ? (q_idx + p.q_offset - key0) : FB;    // keys [0, limit] of this tile are visible to this row
      const int vis = min(limit, p.sk - 1 - key0);
      const bool need_mask = vis < FB - 1;
      // the whole score row into registers (four loads in flight, one wait), masked where needed
      uint32_t sv[FB];
#pragma unroll
      for (int c = 0; c < FB; c += 32) tmem_ld_32x32(tS + (uint32_t)c, sv + c);
      tmem_ld_wait();
      if (__any_sync(0xffffffffu, need_mask)) {
#pragma unroll
        for (int i = 0; i < FB; ++i)
          if (i > vis) sv[i] = 0xff800000u;              // -inf
      }
      float m_tile = -INFINITY;
#pragma unroll
      for (int i = 0; i < FB; ++i) m_tile = fmaxf(m_tile, __uint_as_float(sv[i]));
      const float m_tile2 = m_tile * p.scale_log2;
      // rescale O only when the maximum has grown a lot (decision per warp: the TMEM accesses are warp-wide)
      const bool grow = m_tile2 > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && m_tile2 > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_used, m_tile2);
        const float alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
        if (j > 0) {
          if (!mbar_wait(pv_done(t), jp ^ 1u, p.status, 0x331u)) { ok = false; break; }   // P V of tile j-1 has landed in O
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < FD; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32(tO + (uint32_t)c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(tO + (uint32_t)c, r);
          }
          tmem_st_wait();
        }
        l_run *= alpha;
        m_used = m_new;
      }
      const float m_ref = (m_used == -INFINITY) ? 0.f : m_used;
      // probabilities -> packed bf16 over the first 64 columns of S, row sum (masked scores are -inf -> 0)
      float l_tile = 0.f;
      const float neg_ref = -m_ref;
#pragma unroll
      for (int c = 0; c < FB; c += 32) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float pa = exp2f(fmaf(__uint_as_float(sv[c + 2 * i]), p.scale_log2, neg_ref));
          const float pb = exp2f(fmaf(__uint_as_float(sv[c + 2 * i + 1]), p.scale_log2, neg_ref));
          l_tile += pa + pb;
          __nv_bfloat162 h = __floats2bfloat162_rn(pa, pb);
          pk[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        tmem_st_32x16(tS + (uint32_t)(c >> 1), pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(t));       // one arrival per warp: 128 arrivals on one barrier would serialise
      l_run += l_tile;
    }
    // ---- epilogue of this tile ----
    if (n_kv > 0) {
      if (ok) ok = mbar_wait(pv_done(t), (uint32_t)((n_kv - 1) & 1), p.status, 0x332u);
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      uint8_t* o_row = base_ptr + Fwd2Smem::Q_OFF + t * TILE_BYTES + row * 128;   // the tile's Q buffer: no MMA reads it any more
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < FD; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tO + (uint32_t)c, r);
          tmem_ld_wait();
          uint8_t* blk = o_row + (c >> 6) * HALF_BYTES;
          const int chunk0 = (c & 63) >> 3;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * ch + 2 * e]) * inv, __uint_as_float(r[8 * ch + 2 * e + 1]) * inv);
              pk[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(blk + (((chunk0 + ch) ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
        if (q_idx < p.sq)
          p.lse[((size_t)batch * p.nq + head) * p.sq + q_idx] =
              (l_run > 0.f) ? m_used * 0.6931471805599453f + __logf(l_run) : -INFINITY;
      }
      fence_proxy_async_smem();
      named_bar(1 + t, 128);
      if (ok && q == 0 && lane == 0) {     // warp 2 or 6, one thread: both 64-column halves of the tile (rows past sq are clipped)
        const uint32_t os = base + Fwd2Smem::Q_OFF + t * TILE_BYTES;
        tma_store_4d(&p.tmO, os, 0, head, batch, q0 + t * FB);
        tma_store_4d(&p.tmO, os + HALF_BYTES, 64, head, batch, q0 + t * FB);
        tma_store_commit();
        tma_store_wait<0>();
      }
    } else if (q_idx < p.sq) {
      // no key is visible to any row of this tile: zero output, -inf LSE
      __nv_bfloat16* orow = p.O + (((size_t)q_idx * p.b + batch) * p.nq + head) * FD;
      for (int c = 0; c < FD; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
      p.lse[((size_t)batch * p.nq + head) * p.sq + q_idx] = -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

int make_map4(CUtensorMap* tm, const void* base, int seq, int heads, int b, long long ss, long long sb, long long sh) {
  uint64_t dims[4] = {(uint64_t)FD, (uint64_t)heads, (uint64_t)b, (uint64_t)seq};
  uint64_t str[3] = {(uint64_t)sh * 2, (uint64_t)sb * 2, (uint64_t)ss * 2};
  uint32_t box[4] = {64, 1, 1, (uint32_t)FB};
  return make_tmap_nd(tm, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 4, dims, str, box);
}
}  // namespace

// q [sq, b, nq, 128], k / v [sk, b, nkv, 128] bf16 with element strides (seq, batch, head), last dim contiguous;
// o [sq, b, nq, 128] contiguous; lse [b, nq, sq] fp32 (natural log of the scaled scores' softmax denominator).
MSB_API int msb_flash_fwd2(const void* q, const void* k, const void* v, void* o, float* lse, int sq, int sk, int b, int nq, int nkv,
                           long long q_ss, long long q_sb, long long q_sh, long long k_ss, long long k_sb, long long k_sh,
                           long long v_ss, long long v_sb, long long v_sh, int causal, int q_offset, float scale,
                           unsigned int* status, cudaStream_t s) {
  MSB_REQUIRE(sq > 0 && sk > 0 && nq % nkv == 0, "flash_fwd2: bad shape sq=%d sk=%d nq=%d nkv=%d", sq, sk, nq, nkv);
  MSB_REQUIRE(status != nullptr, "flash_fwd2: status word is required");
  Fwd2Params p;
  memset(&p, 0, sizeof(p));
  int rc = make_map4(&p.tmQ, q, sq, nq, b, q_ss, q_sb, q_sh); if (rc) return rc;
  rc = make_map4(&p.tmK, k, sk, nkv, b, k_ss, k_sb, k_sh); if (rc) return rc;
  rc = make_map4(&p.tmV, v, sk, nkv, b, v_ss, v_sb, v_sh); if (rc) return rc;
  rc = make_map4(&p.tmO, o, sq, nq, b, (long long)b * nq * FD, (long long)nq * FD, FD); if (rc) return rc;
  p.O = (__nv_bfloat16*)o; p.lse = lse;
  p.sq = sq; p.sk = sk; p.b = b; p.nq = nq; p.nkv = nkv; p.causal = causal; p.q_offset = q_offset;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd2_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd2Smem::TOTAL);
    if (e != cudaSuccess) { msb_set_error("flash_fwd2: cannot set dynamic shared memory: %s", cudaGetErrorString(e)); return 1; }
    attr = true;
  }
  dim3 grid((sq + 2 * FB - 1) / (2 * FB), nq, b);
  flash_fwd2_sm100_kernel<<<grid, 320, Fwd2Smem::TOTAL, s>>>(p);
  MSB_CHECK_LAUNCH("flash_fwd2_sm100");
  return 0;
}

// =====================================================================================================================
// Flash attention backward for sm_100a.  head_dim 128, bf16, causal or full, GQA, query offset.
//
// One CTA owns a tile of 128 keys of one (batch, KV head) and walks every query tile of every query head of that KV head
// that can see it.  All five products of an iteration run on tcgen05 in the transposed formulation (keys on the TMEM lanes):
//     S^T  = K Q^T                 A = K  (smem, K-major)      B = Q  (smem, K-major)
//     dP^T = V dO^T                A = V  (smem, K-major)      B = dO (smem, K-major)
//     dV  += P^T dO                A = P^T  (TMEM, packed bf16 over the first half of S^T)      B = dO (smem, MN-major)
//     dK  += dS^T Q                A = dS^T (TMEM, packed bf16 over the first half of dP^T)     B = Q  (smem, MN-major)
//     dQ   = dS K   (2 x N = 64)   A = dS^T as written to smem [keys, q] = dS MN-major          B = K  (smem, MN-major)
// TMEM (512 columns): S^T | dP^T | dV | dK.  The two halves of dQ land in the upper 64 columns of S^T and dP^T, which are
// free once the compute warps have read the scores; dQ is scaled, staged in shared memory and added into the fp32 dQ
// buffer with TMA reduce-adds (other key tiles add into the same rows).
//   warp 0      TMA producer: K, V once; Q_i, dO_i, LSE_i, delta_i into a 2-stage ring
//   warp 1      MMA issuer (one thread)
//   warps 2-5   softmax: warp w owns key rows 32 (w mod 4) .. +31 and all 128 query columns of the tile:
//               P^T = exp2(S^T scale log2e - LSE log2e), dS^T = P^T (dP^T - delta)
//   warps 6-9   dQ: read the finished dQ tile out of tensor memory (which frees S^T / dP^T for the next iteration at
//               once), apply the softmax scale and add it into global memory, off the critical path of the next tile
//               (all eight warps share the final write-out of dK and dV, where the scale of dK is applied)
// delta = rowsum(dO * O) and the LSE in log2 units are prepared by flash_bwd_prep_kernel into buffers padded to whole tiles
// (padding rows get LSE = +inf so their probabilities are zero).
// reference semantics: the attention grad op of the reference, mindspeed/ops/csrc/cann/fusion_attention_v2.cpp:431-439.
// =====================================================================================================================
namespace {

struct BwdParams {
  CUtensorMap tmQ, tmK, tmV, tmdO;  // bf16, dims {d, head, batch, seq}
  CUtensorMap tmdQ;                 // fp32 [sq, b, nq, d], dims {d, head, batch, seq}, box {32, 1, 1, 32}
  CUtensorMap tmdK, tmdV;           // [sk, b, nkv, d] outputs: bf16 stores, or fp32 reduce-add targets (box {32,1,1,32}) when split_heads
  const float* lse2;                // [b, nq, sq_pad] LSE * log2(e) (+inf where no key is visible / padding)
  const float* delta;               // [b, nq, sq_pad]
  int sq, sk, b, nq, nkv, sq_pad;
  int causal, q_offset;
  float scale, scale_log2;
  int split_heads;                  // 1: one CTA per (key tile, QUERY head); dK / dV partial sums are added into fp32 buffers
  unsigned int* status;
};

struct BwdSmem {
  static constexpr int Q_OFF = 0;                          // 2 stages
  static constexpr int DO_OFF = 2 * TILE_BYTES;            // 2 stages
  static constexpr int K_OFF = 4 * TILE_BYTES;
  static constexpr int V_OFF = 5 * TILE_BYTES;
  static constexpr int DS_OFF = 6 * TILE_BYTES;            // dS^T [keys, q] bf16; doubles as the dQ staging area
  static constexpr int BAR_OFF = 7 * TILE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
  static_assert(TOTAL <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

__device__ __forceinline__ void bulk_g2s_bar(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_4d(const void* tmap, uint32_t src, int x, int y, int z, int w) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(src), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}

// delta[b, h, r] = sum_d dO * O; lse2 = LSE * log2(e) with -inf (no visible key) and padding rows mapped to +inf.
__global__ void flash_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout, long long do_ss,
                                      long long do_sb, long long do_sh, const float* __restrict__ lse, float* __restrict__ lse2,
                                      float* __restrict__ delta, int sq, int b, int nq, int sq_pad) {
  const int warp = (int)((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  const long long total = (long long)b * nq * sq_pad;
  if (warp >= total) return;
  const int r = warp % sq_pad, h = (warp / sq_pad) % nq, bb = warp / (sq_pad * nq);
  float acc = 0.f, l2 = INFINITY;
  if (r < sq) {
    const __nv_bfloat16* orow = o + (((size_t)r * b + bb) * nq + h) * FD + lane * 4;
    const __nv_bfloat16* drow = dout + (size_t)r * do_ss + (size_t)bb * do_sb + (size_t)h * do_sh + lane * 4;
    const uint2 ov = *reinterpret_cast<const uint2*>(orow), dv = *reinterpret_cast<const uint2*>(drow);
    const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&ov);
    const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 a = __bfloat1622float2(oh[i]), c = __bfloat1622float2(dh[i]);
      acc += a.x * c.x + a.y * c.y;
    }
    acc = warp_sum(acc);
    const float l = lse[((size_t)bb * nq + h) * sq + r];
    l2 = (l == -INFINITY) ? INFINITY : l * 1.4426950408889634f;
  }
  if (lane == 0) {
    delta[warp] = acc;
    lse2[warp] = l2;
  }
}

__global__ void __launch_bounds__(320, 1) flash_bwd_sm100_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar = base + BwdSmem::BAR_OFF;
  const uint32_t kv_full = bar;
  auto qdo_full = [&](int s) { return bar + 8u * (1 + s); };
  auto qdo_empty = [&](int s) { return bar + 8u * (3 + s); };
  const uint32_t st_full = bar + 8u * 5, dpt_full = bar + 8u * 6, pt_ready = bar + 8u * 7, ds_ready = bar + 8u * 8,
                 dq_full = bar + 8u * 9, dq_drained = bar + 8u * 10, acc_done = bar + 8u * 11, tmem_slot = bar + 8u * 12;
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(base_ptr + BwdSmem::BAR_OFF + 8 * 12);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // key tiles that many query tiles see (early ones, when causal) first
  const int j = (int)blockIdx.x;
  // without the split a CTA walks all query heads of its KV head; with it (few KV heads: too few CTAs otherwise) one each
  const int rep_all = p.nq / p.nkv;
  const int g = p.split_heads ? (int)blockIdx.y / rep_all : (int)blockIdx.y, batch = blockIdx.z;
  const int head0 = p.split_heads ? (int)blockIdx.y : g * rep_all;
  const int rep = p.split_heads ? 1 : rep_all;
  const int key0 = j * FB;
  const int n_q = (p.sq + FB - 1) / FB;
  int i_start = 0;
  if (p.causal) {
    const int first_q = key0 - p.q_offset;                 // first query row that sees key0
    i_start = first_q <= 0 ? 0 : first_q / FB;
  }
  const int n_i = max(n_q - i_start, 0);
  const int n_it = n_i * rep;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(qdo_full(s), 1); mbar_init(qdo_empty(s), 1); }
    mbar_init(st_full, 1); mbar_init(dpt_full, 1); mbar_init(pt_ready, 4); mbar_init(ds_ready, 4);
    mbar_init(dq_full, 1); mbar_init(dq_drained, 4); mbar_init(acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t tST = tmem_base, tDPT = tmem_base + 128u, tDV = tmem_base + 256u, tDK = tmem_base + 384u;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0 && n_it > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
      tma_load_4d(base + BwdSmem::K_OFF, &p.tmK, kv_full, 0, g, batch, key0);
      tma_load_4d(base + BwdSmem::K_OFF + HALF_BYTES, &p.tmK, kv_full, 64, g, batch, key0);
      tma_load_4d(base + BwdSmem::V_OFF, &p.tmV, kv_full, 0, g, batch, key0);
      tma_load_4d(base + BwdSmem::V_OFF + HALF_BYTES, &p.tmV, kv_full, 64, g, batch, key0);
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        const uint32_t ph = (uint32_t)((it >> 1) & 1);
        const int head = head0 + it / n_i, i = i_start + it % n_i;
        if (!mbar_wait(qdo_empty(s), ph ^ 1u, p.status, 0x410u)) { ok = false; break; }
        mbar_arrive_expect_tx(qdo_full(s), 2 * TILE_BYTES);
        const uint32_t qs = base + BwdSmem::Q_OFF + s * TILE_BYTES, ds = base + BwdSmem::DO_OFF + s * TILE_BYTES;
        tma_load_4d(qs, &p.tmQ, qdo_full(s), 0, head, batch, i * FB);
        tma_load_4d(qs + HALF_BYTES, &p.tmQ, qdo_full(s), 64, head, batch, i * FB);
        tma_load_4d(ds, &p.tmdO, qdo_full(s), 0, head, batch, i * FB);
        tma_load_4d(ds + HALF_BYTES, &p.tmdO, qdo_full(s), 64, head, batch, i * FB);
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_kk = make_idesc_f16(128, 128, 1, 0, 0);     // both operands K-major
      constexpr uint32_t idesc_tn = make_idesc_f16(128, 128, 1, 0, 1);     // A from TMEM, B MN-major
      constexpr uint32_t idesc_dq = make_idesc_f16(128, 64, 1, 1, 1);      // A and B MN-major, N = 64
      const uint32_t ks = base + BwdSmem::K_OFF, vs = base + BwdSmem::V_OFF, dss = base + BwdSmem::DS_OFF;
      bool ok = mbar_wait(kv_full, 0, p.status, 0x420u);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        const uint32_t ph = (uint32_t)((it >> 1) & 1), ip = (uint32_t)(it & 1);
        const uint32_t qs = base + BwdSmem::Q_OFF + s * TILE_BYTES, dos = base + BwdSmem::DO_OFF + s * TILE_BYTES;
        if (!mbar_wait(qdo_full(s), ph, p.status, 0x421u)) { ok = false; break; }
        if (it > 0 && !mbar_wait(dq_drained, ip ^ 1u, p.status, 0x422u)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < FD / 16; ++k) {
          const uint32_t off = (uint32_t)((k >> 2) * HALF_BYTES + (k & 3) * 32);
          umma_f16(tST, make_smem_desc(ks + off, 0, 1024), make_smem_desc(qs + off, 0, 1024), idesc_kk, k ? 1u : 0u);
        }
        umma_commit(st_full);
#pragma unroll
        for (int k = 0; k < FD / 16; ++k) {
          const uint32_t off = (uint32_t)((k >> 2) * HALF_BYTES + (k & 3) * 32);
          umma_f16(tDPT, make_smem_desc(vs + off, 0, 1024), make_smem_desc(dos + off, 0, 1024), idesc_kk, k ? 1u : 0u);
        }
        umma_commit(dpt_full);
        if (!mbar_wait(pt_ready, ip, p.status, 0x423u)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < FB / 16; ++k)      // reduction over the 128 query rows, 16 per MMA: P^T columns 8k.., dO rows 16k..
          umma_f16_ts(tDV, tST + (uint32_t)(k * 8), make_smem_desc(dos + (uint32_t)(k * 16 * 128), HALF_BYTES, 1024), idesc_tn,
                      (it | k) ? 1u : 0u);
        if (!mbar_wait(ds_ready, ip, p.status, 0x424u)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h) {          // dQ[:, 64h .. 64h+63] = dS K[:, 64h ..]: reduction over the 128 keys
          const uint32_t tD = (h == 0 ? tST : tDPT) + 64u;
#pragma unroll
          for (int k = 0; k < FB / 16; ++k)
            umma_f16(tD, make_smem_desc(dss + (uint32_t)(k * 16 * 128), HALF_BYTES, 1024),
                     make_smem_desc(ks + (uint32_t)(h * HALF_BYTES + k * 16 * 128), HALF_BYTES, 1024), idesc_dq, k ? 1u : 0u);
        }
        umma_commit(dq_full);
#pragma unroll
        for (int k = 0; k < FB / 16; ++k)
          umma_f16_ts(tDK, tDPT + (uint32_t)(k * 8), make_smem_desc(qs + (uint32_t)(k * 16 * 128), HALF_BYTES, 1024), idesc_tn,
                      (it | k) ? 1u : 0u);
        umma_commit(qdo_empty(s));             // Q_i and dO_i are free once everything issued so far has completed
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    // ===================== warps 2..5: P^T and dS^T;  warps 6..9: dQ out of the SM =====================
    const int q = warp & 3;
    const bool drainer = warp >= 6;
    const int ch = (warp - 2) >> 2;                    // column half this warp drains from dK / dV at the very end
    const int row = q * 32 + lane;                     // key row inside the tile == TMEM lane (query row when draining dQ)
    const int key = key0 + row;
    const uint32_t lane_addr = ((uint32_t)(q * 32) << 16);
    // rows 32q .. 32q+31 of the two 64-column halves of the dS^T buffer: 2 x 4 KB shared by softmax warp q (dS^T rows) and
    // drain warp q (dQ staging); the pair hands them back and forth over named barrier 3 + q
    uint8_t* piece_ptr[2] = {base_ptr + BwdSmem::DS_OFF + q * 4096, base_ptr + BwdSmem::DS_OFF + HALF_BYTES + q * 4096};
    const uint32_t piece[2] = {base + BwdSmem::DS_OFF + (uint32_t)(q * 4096), base + BwdSmem::DS_OFF + (uint32_t)(HALF_BYTES + q * 4096)};
    bool ok = true;
    if (!drainer) {
      // ---------------- softmax warps: one thread per key row, all 128 query columns ----------------
      auto load_stats = [&](int it2, float4& l, float4& d) {
        const size_t stat = ((size_t)batch * p.nq + (head0 + it2 / n_i)) * p.sq_pad + (size_t)(i_start + it2 % n_i) * FB;
        l = __ldg(reinterpret_cast<const float4*>(p.lse2 + stat) + lane);
        d = __ldg(reinterpret_cast<const float4*>(p.delta + stat) + lane);
      };
      // row statistics of the tile's 128 query columns: lane l holds columns 4l .. 4l+3, fetched one iteration ahead (an
      // L2 / HBM round trip is longer than a phase); the loops broadcast them with shuffles
      float4 nxt_lse = make_float4(0.f, 0.f, 0.f, 0.f), nxt_dlt = nxt_lse;
      if (n_it > 0) load_stats(0, nxt_lse, nxt_dlt);
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t ip = (uint32_t)(it & 1);
        const int i = i_start + it % n_i;
        const float4 my_lse = nxt_lse, my_dlt = nxt_dlt;
        if (it + 1 < n_it) load_stats(it + 1, nxt_lse, nxt_dlt);
        const float ls4[4] = {my_lse.x, my_lse.y, my_lse.z, my_lse.w};
        const float dl4[4] = {my_dlt.x, my_dlt.y, my_dlt.z, my_dlt.w};
        // keys of this tile visible to query row r: key <= r + q_offset (causal), key < sk
        // <=> query column c of the tile is visible to this thread's key iff c >= first_c
        const int first_c = (key >= p.sk) ? FB : (p.causal ? key - p.q_offset - i * FB : 0);
        uint32_t ppk[64];                              // P^T of this row, packed bf16 pairs (kept for dS^T)
        // ---- P^T = exp2(S^T scale log2e - LSE log2e), 64 columns at a time ----
        if (!mbar_wait(st_full, ip, p.status, 0x430u)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(tST + lane_addr + (uint32_t)(h * 64), r0);
          tmem_ld_32x32(tST + lane_addr + (uint32_t)(h * 64 + 32), r1);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            float pr[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int cc = 2 * c + e;
              const float ls = __shfl_sync(0xffffffffu, ls4[cc & 3], h * 16 + (cc >> 2));
              const float sc = __uint_as_float(cc < 32 ? r0[cc] : r1[cc - 32]);
              const float v = exp2f(fmaf(sc, p.scale_log2, -ls));
              pr[e] = (h * 64 + cc < first_c) ? 0.f : v;   // a select, never a branch (a short-circuit test per element costs one)
            }
            __nv_bfloat162 hh = __floats2bfloat162_rn(pr[0], pr[1]);
            ppk[h * 32 + c] = *reinterpret_cast<uint32_t*>(&hh);
          }
          // P^T columns [32h, 32h+32) overwrite S^T columns this warp has already read (nobody else touches these lanes)
          tmem_st_32x16(tST + lane_addr + (uint32_t)(h * 32), ppk + h * 32);
          tmem_st_32x16(tST + lane_addr + (uint32_t)(h * 32 + 16), ppk + h * 32 + 16);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pt_ready);
        // ---- dS^T = P^T (dP^T - delta) ----
        if (!mbar_wait(dpt_full, ip, p.status, 0x431u)) { ok = false; break; }
        tc_fence_after();
        named_bar(3 + q, 64);                           // drain warp q has handed the two staging pieces back
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(tDPT + lane_addr + (uint32_t)(h * 64), r0);
          tmem_ld_32x32(tDPT + lane_addr + (uint32_t)(h * 64 + 32), r1);
          tmem_ld_wait();
          uint32_t pk[32];
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float dl0 = __shfl_sync(0xffffffffu, dl4[(2 * c) & 3], h * 16 + ((2 * c) >> 2));
            const float dl1 = __shfl_sync(0xffffffffu, dl4[(2 * c + 1) & 3], h * 16 + ((2 * c + 1) >> 2));
            const uint32_t pp = ppk[h * 32 + c];
            const float p0 = __uint_as_float(pp << 16), p1 = __uint_as_float(pp & 0xffff0000u);
            const float d0 = p0 * (__uint_as_float(2 * c < 32 ? r0[2 * c] : r1[2 * c - 32]) - dl0);
            const float d1 = p1 * (__uint_as_float(2 * c + 1 < 32 ? r0[2 * c + 1] : r1[2 * c + 1 - 32]) - dl1);
            __nv_bfloat162 hh = __floats2bfloat162_rn(d0, d1);
            pk[c] = *reinterpret_cast<uint32_t*>(&hh);
          }
          tmem_st_32x16(tDPT + lane_addr + (uint32_t)(h * 32), pk);
          tmem_st_32x16(tDPT + lane_addr + (uint32_t)(h * 32 + 16), pk + 16);
          // shared-memory copy for the dQ MMA: row = key, 64 query columns = 8 chunks of 16 bytes, 128-byte swizzle
          uint8_t* srow = piece_ptr[h] + lane * 128;
#pragma unroll
          for (int cchunk = 0; cchunk < 8; ++cchunk)
            *reinterpret_cast<uint4*>(srow + ((cchunk ^ (row & 7)) << 4)) = make_uint4(pk[4 * cchunk], pk[4 * cchunk + 1], pk[4 * cchunk + 2], pk[4 * cchunk + 3]);
        }
        tmem_st_wait();
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_ready);
      }
    } else {
      // ---------------- drain warps: dQ (lanes = query rows) -> scale -> staging -> TMA reduce-add into the fp32 dQ ----------------
      asm volatile("bar.arrive %0, 64;" ::"r"(3 + q) : "memory");      // the staging pieces start out free
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t ip = (uint32_t)(it & 1);
        const int head = head0 + it / n_i, i = i_start + it % n_i;
        if (!mbar_wait(dq_full, ip, p.status, 0x432u)) { ok = false; break; }
        tc_fence_after();
        uint32_t r[4][32];                               // d columns 32k .. 32k+31 of this lane's query row
        tmem_ld_32x32(tST + 64u + lane_addr, r[0]);
        tmem_ld_32x32(tST + 96u + lane_addr, r[1]);
        tmem_ld_32x32(tDPT + 64u + lane_addr, r[2]);
        tmem_ld_32x32(tDPT + 96u + lane_addr, r[3]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_drained);          // the MMA thread may overwrite S^T / dP^T
        const int qr = i * FB + q * 32;                  // first query row of this warp's block
#pragma unroll
        for (int rnd = 0; rnd < 2; ++rnd) {
          if (rnd == 1) { if (lane == 0) tma_store_wait_read<0>(); __syncwarp(); }
#pragma unroll
          for (int b2 = 0; b2 < 2; ++b2) {
            const uint32_t* rr = r[rnd * 2 + b2];
            uint8_t* srow = piece_ptr[b2] + lane * 128;
#pragma unroll
            for (int cchunk = 0; cchunk < 8; ++cchunk) {
              float4 o4 = make_float4(__uint_as_float(rr[4 * cchunk]) * p.scale, __uint_as_float(rr[4 * cchunk + 1]) * p.scale,
                                      __uint_as_float(rr[4 * cchunk + 2]) * p.scale, __uint_as_float(rr[4 * cchunk + 3]) * p.scale);
              *reinterpret_cast<float4*>(srow + ((cchunk ^ (lane & 7)) << 4)) = o4;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && qr < p.sq) {
            tma_reduce_add_4d(&p.tmdQ, piece[0], rnd * 64, head, batch, qr);
            tma_reduce_add_4d(&p.tmdQ, piece[1], rnd * 64 + 32, head, batch, qr);
            tma_store_commit();
          }
        }
        if (it + 1 < n_it) {
          if (lane == 0) tma_store_wait_read<0>();       // the reduce-adds have read the staging: hand it back
          __syncwarp();
          asm volatile("bar.arrive %0, 64;" ::"r"(3 + q) : "memory");
        }
      }
    }
    // ---- dK, dV of this key tile: TMEM -> bf16 -> shared memory (the Q / dO stage buffers) -> TMA store ----
    if (n_it > 0) {
      if (ok) ok = mbar_wait(acc_done, 0, p.status, 0x433u);
      tc_fence_after();
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
      if (p.split_heads) {
        // partial sums of one query head: fp32 through this warp's own 8 KB of staging, two [32 x 32] boxes per tensor
        const uint32_t st_addr = base + BwdSmem::Q_OFF + (uint32_t)((warp - 2) * 8192);
        uint8_t* st_ptr = base_ptr + BwdSmem::Q_OFF + (warp - 2) * 8192;
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          const uint32_t tA = (which == 0 ? tDV : tDK) + lane_addr + (uint32_t)(ch * 64);
          const float mul = which == 0 ? 1.f : p.scale;
          if (which == 1) { if (lane == 0) tma_store_wait_read<0>(); __syncwarp(); }
#pragma unroll
          for (int b2 = 0; b2 < 2; ++b2) {
            uint32_t r[32];
            tmem_ld_32x32(tA + (uint32_t)(b2 * 32), r);
            tmem_ld_wait();
            uint8_t* srow = st_ptr + b2 * 4096 + lane * 128;
#pragma unroll
            for (int cchunk = 0; cchunk < 8; ++cchunk)
              *reinterpret_cast<float4*>(srow + ((cchunk ^ (lane & 7)) << 4)) =
                  make_float4(__uint_as_float(r[4 * cchunk]) * mul, __uint_as_float(r[4 * cchunk + 1]) * mul,
                              __uint_as_float(r[4 * cchunk + 2]) * mul, __uint_as_float(r[4 * cchunk + 3]) * mul);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (ok && lane == 0 && key0 + q * 32 < p.sk) {
            const CUtensorMap* tm = which == 0 ? &p.tmdV : &p.tmdK;
            tma_reduce_add_4d(tm, st_addr, ch * 64, g, batch, key0 + q * 32);
            tma_reduce_add_4d(tm, st_addr + 4096u, ch * 64 + 32, g, batch, key0 + q * 32);
            tma_store_commit();
          }
        }
        if (lane == 0) tma_store_wait<0>();
      } else {
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {          // 0: dV (no scale), 1: dK (softmax scale)
        const uint32_t tA = (which == 0 ? tDV : tDK) + lane_addr + (uint32_t)(ch * 64);
        const float mul = which == 0 ? 1.f : p.scale;
        uint8_t* srow = base_ptr + (which == 0 ? BwdSmem::Q_OFF : BwdSmem::DO_OFF) + ch * HALF_BYTES + row * 128;
#pragma unroll 1
        for (int c = 0; c < 64; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tA + (uint32_t)c, r);
          tmem_ld_wait();
#pragma unroll
          for (int cchunk = 0; cchunk < 4; ++cchunk) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(r[8 * cchunk + 2 * e]) * mul, __uint_as_float(r[8 * cchunk + 2 * e + 1]) * mul);
              pk[e] = *reinterpret_cast<uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(srow + ((((c >> 3) + cchunk) ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      }
      fence_proxy_async_smem();
      named_bar(2, 256);
      if (ok && warp == 2 && lane == 0) {
        tma_store_4d(&p.tmdV, base + BwdSmem::Q_OFF, 0, g, batch, key0);
        tma_store_4d(&p.tmdV, base + BwdSmem::Q_OFF + HALF_BYTES, 64, g, batch, key0);
        tma_store_4d(&p.tmdK, base + BwdSmem::DO_OFF, 0, g, batch, key0);
        tma_store_4d(&p.tmdK, base + BwdSmem::DO_OFF + HALF_BYTES, 64, g, batch, key0);
        tma_store_commit();
      }
      if (lane == 0) tma_store_wait<0>();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}
}  // namespace

// Gradients of flash attention.  q / k / v / dout strided like the forward's inputs, o [sq, b, nq, 128] contiguous,
// lse [b, nq, sq]; dq32 [sq, b, nq, 128] fp32 ZERO-INITIALISED by the caller (key tiles add into it), dk / dv
// [sk, b, nkv, 128] bf16 contiguous, zero-initialised when some key tile is visible to no query; lse2 / delta: scratch
// fp32 [b, nq, ceil(sq / 128) * 128] each.
// split_heads = 1: dk / dv are fp32 [sk, b, nkv, 128] ZERO-INITIALISED buffers that every query head adds into (use when
// ceil(sk / 128) * nkv * b is well below the SM count); 0: bf16 outputs written once.
MSB_API int msb_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                          float* dq32, void* dk, void* dv, float* lse2, float* delta, int split_heads, int sq, int sk, int b, int nq, int nkv,
                          long long q_ss, long long q_sb, long long q_sh, long long k_ss, long long k_sb, long long k_sh,
                          long long v_ss, long long v_sb, long long v_sh, long long do_ss, long long do_sb, long long do_sh,
                          int causal, int q_offset, float scale, unsigned int* status, cudaStream_t s) {
  MSB_REQUIRE(sq > 0 && sk > 0 && nq % nkv == 0, "flash_bwd: bad shape sq=%d sk=%d nq=%d nkv=%d", sq, sk, nq, nkv);
  MSB_REQUIRE(status != nullptr, "flash_bwd: status word is required");
  const int sq_pad = (sq + FB - 1) / FB * FB;
  {
    const long long rows = (long long)b * nq * sq_pad;
    const int threads = 256;
    const long long blocks = (rows * 32 + threads - 1) / threads;
    flash_bwd_prep_kernel<<<(unsigned)blocks, threads, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, do_ss, do_sb, do_sh,
                                                             lse, lse2, delta, sq, b, nq, sq_pad);
    MSB_CHECK_LAUNCH("flash_bwd_prep");
  }
  BwdParams p;
  memset(&p, 0, sizeof(p));
  int rc = make_map4(&p.tmQ, q, sq, nq, b, q_ss, q_sb, q_sh); if (rc) return rc;
  rc = make_map4(&p.tmK, k, sk, nkv, b, k_ss, k_sb, k_sh); if (rc) return rc;
  rc = make_map4(&p.tmV, v, sk, nkv, b, v_ss, v_sb, v_sh); if (rc) return rc;
  rc = make_map4(&p.tmdO, dout, sq, nq, b, do_ss, do_sb, do_sh); if (rc) return rc;
  if (!split_heads) {
    rc = make_map4(&p.tmdK, dk, sk, nkv, b, (long long)b * nkv * FD, (long long)nkv * FD, FD); if (rc) return rc;
    rc = make_map4(&p.tmdV, dv, sk, nkv, b, (long long)b * nkv * FD, (long long)nkv * FD, FD); if (rc) return rc;
  } else {
    uint64_t dims[4] = {(uint64_t)FD, (uint64_t)nkv, (uint64_t)b, (uint64_t)sk};
    uint64_t str[3] = {(uint64_t)FD * 4, (uint64_t)nkv * FD * 4, (uint64_t)b * nkv * FD * 4};
    uint32_t box[4] = {32, 1, 1, 32};
    rc = make_tmap_nd(&p.tmdK, dk, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, 4, dims, str, box); if (rc) return rc;
    rc = make_tmap_nd(&p.tmdV, dv, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, 4, dims, str, box); if (rc) return rc;
  }
  p.split_heads = split_heads ? 1 : 0;
  {
    uint64_t dims[4] = {(uint64_t)FD, (uint64_t)nq, (uint64_t)b, (uint64_t)sq};
    uint64_t str[3] = {(uint64_t)FD * 4, (uint64_t)nq * FD * 4, (uint64_t)b * nq * FD * 4};
    uint32_t box[4] = {32, 1, 1, 32};
    rc = make_tmap_nd(&p.tmdQ, dq32, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, 4, dims, str, box);
    if (rc) return rc;
  }
  p.lse2 = lse2; p.delta = delta;
  p.sq = sq; p.sk = sk; p.b = b; p.nq = nq; p.nkv = nkv; p.sq_pad = sq_pad; p.causal = causal; p.q_offset = q_offset;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(flash_bwd_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::TOTAL);
    if (e != cudaSuccess) { msb_set_error("flash_bwd: cannot set dynamic shared memory: %s", cudaGetErrorString(e)); return 1; }
    attr = true;
  }
  dim3 grid((sk + FB - 1) / FB, split_heads ? nq : nkv, b);
  flash_bwd_sm100_kernel<<<grid, 320, BwdSmem::TOTAL, s>>>(p);
  MSB_CHECK_LAUNCH("flash_bwd_sm100");
  return 0;
}
