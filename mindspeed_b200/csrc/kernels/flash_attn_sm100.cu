// Flash attention forward for sm_100a: S = Q K^T and O += P V on tcgen05 tensor cores with TMEM accumulators,
// operands staged by TMA, online softmax in registers.  head_dim 128, bf16, causal or full, GQA.
//
// One CTA owns 128 query rows of one (batch, head) and walks the key/value tiles of 128 keys it may see.
//   warp 0     TMA producer: Q once, then K_j / V_j into a 2-stage ring (4-D tensor maps over the strided
//              [seq, batch, head, dim] tensors, so packed-QKV views need no copy)
//   warp 1     MMA issuer: S_j = Q K_j^T (8 x UMMA 128x128x16, both operands K-major) into TMEM columns [0,128);
//              PV_j = P_j V_j (A = P from shared memory K-major, B = V MN-major) into TMEM columns [128,256)
//   warps 2-5  softmax: thread i owns query row i.  Two passes over S in TMEM (row max, then exp2 / row sum), P written
//              to shared memory as bf16 in the 128-byte-swizzled K-major layout the MMA expects, O kept in registers
//              and updated as O = O * alpha + PV_j.  S_{j+1} is issued right behind PV_j, so it runs while the
//              softmax threads fold PV_j into O.
// Outputs: O [seq, batch, head, dim] bf16 and LSE [batch, head, seq] fp32 (natural log of the row's softmax
// denominator including the scale), which the backward pass and ring attention need.
// reference semantics: torch_npu.npu_fusion_attention returning softmax max/sum
// (mindspeed/core/transformer/flash_attention/flash_attention/adaptor.py:21-85, mindspeed/ops/fusion_attention_v2.py:22-114).
#include "msb_common.cuh"
#include "msb_sm100.cuh"

using namespace msb;
using namespace msb::sm100;

namespace {
constexpr int FB = 128;            // rows per Q tile, keys per KV tile
constexpr int FD = 128;            // head dim
constexpr int TILE_BYTES = FB * FD * 2;   // 32 KB
constexpr int HALF_BYTES = FB * 128;      // one 64-wide column block: 128 rows x 128 B

struct FlashParams {
  CUtensorMap tmQ, tmK, tmV;       // dims {d, head, batch, seq}
  __nv_bfloat16* O;                // [sq, b, nq, d] contiguous
  float* lse;                      // [b, nq, sq]
  int sq, sk, b, nq, nkv;
  int causal;
  int q_offset;                    // absolute position of query row 0 minus absolute position of key 0
  float scale_log2;                // softmax_scale * log2(e)
  float scale;
  unsigned int* status;
};

struct FlashSmem {
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE_BYTES;                 // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * TILE_BYTES;     // 2 stages
  static constexpr int P_OFF = V_OFF + 2 * TILE_BYTES;
  static constexpr int BAR_OFF = P_OFF + TILE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__global__ void __launch_bounds__(192, 1) flash_fwd_sm100_kernel(const __grid_constant__ FlashParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar = base + FlashSmem::BAR_OFF;
  const uint32_t q_full = bar, kv_full0 = bar + 8, kv_empty0 = bar + 24, s_full = bar + 40, s_empty = bar + 48,
                 p_full = bar + 56, pv_full = bar + 64, o_empty = bar + 72, tmem_slot = bar + 80;
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(base_ptr + FlashSmem::BAR_OFF + 80);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first so the causal triangle balances across the grid
  const int m_blk = (p.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x);
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.nq / p.nkv);
  const int q0 = m_blk * FB;
  int n_kv = (p.sk + FB - 1) / FB;
  if (p.causal) {
    const int last_key = q0 + FB - 1 + p.q_offset;        // last key any row of this tile may see
    n_kv = min(n_kv, last_key / FB + 1);
    if (last_key < 0) n_kv = 0;
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
    mbar_init(s_full, 1); mbar_init(s_empty, 128); mbar_init(p_full, 128); mbar_init(pv_full, 1); mbar_init(o_empty, 128);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t tS = tmem_base, tO = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      mbar_arrive_expect_tx(q_full, TILE_BYTES);
      tma_load_4d(base + FlashSmem::Q_OFF, &p.tmQ, q_full, 0, head, batch, q0);
      tma_load_4d(base + FlashSmem::Q_OFF + HALF_BYTES, &p.tmQ, q_full, 64, head, batch, q0);
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!mbar_wait(kv_empty0 + 8 * s, ph ^ 1u, p.status, 0x310u)) { ok = false; break; }
        mbar_arrive_expect_tx(kv_full0 + 8 * s, 2 * TILE_BYTES);
        const uint32_t ks = base + FlashSmem::K_OFF + s * TILE_BYTES, vs = base + FlashSmem::V_OFF + s * TILE_BYTES;
        tma_load_4d(ks, &p.tmK, kv_full0 + 8 * s, 0, kv_head, batch, j * FB);
        tma_load_4d(ks + HALF_BYTES, &p.tmK, kv_full0 + 8 * s, 64, kv_head, batch, j * FB);
        tma_load_4d(vs, &p.tmV, kv_full0 + 8 * s, 0, kv_head, batch, j * FB);
        tma_load_4d(vs + HALF_BYTES, &p.tmV, kv_full0 + 8 * s, 64, kv_head, batch, j * FB);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(128, 128, 1, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_f16(128, 128, 1, 0, 1);
      bool ok = mbar_wait(q_full, 0, p.status, 0x320u);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1), jp = (uint32_t)(j & 1);
        if (!mbar_wait(kv_full0 + 8 * s, ph, p.status, 0x321u)) { ok = false; break; }
        if (!mbar_wait(s_empty, jp ^ 1u, p.status, 0x322u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t qs = base + FlashSmem::Q_OFF, ks = base + FlashSmem::K_OFF + s * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < FD / 16; ++k) {
          const uint32_t off = (uint32_t)((k >> 2) * HALF_BYTES + (k & 3) * 32);
          umma_f16(tS, make_smem_desc(qs + off, 0, 1024), make_smem_desc(ks + off, 0, 1024), idesc_qk, k ? 1u : 0u);
        }
        umma_commit(s_full);
        if (!mbar_wait(p_full, jp, p.status, 0x323u)) { ok = false; break; }
        if (!mbar_wait(o_empty, jp ^ 1u, p.status, 0x324u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ps = base + FlashSmem::P_OFF, vs = base + FlashSmem::V_OFF + s * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < FB / 16; ++k) {
          const uint64_t adesc = make_smem_desc(ps + (uint32_t)((k >> 2) * HALF_BYTES + (k & 3) * 32), 0, 1024);
          const uint64_t bdesc = make_smem_desc(vs + (uint32_t)(k * 16 * 128), HALF_BYTES, 1024);   // MN-major: 16 keys = 2048 B
          umma_f16(tO, adesc, bdesc, idesc_pv, k ? 1u : 0u);
        }
        umma_commit(pv_full);
        umma_commit(kv_empty0 + 8 * s);
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;                 // row inside the tile == TMEM lane
    const int q_idx = q0 + row;
    const uint32_t lane_addr = ((uint32_t)(q * 32) << 16);
    float o[FD];
#pragma unroll
    for (int i = 0; i < FD; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    uint8_t* p_row = base_ptr + FlashSmem::P_OFF + row * 128;
    for (int j = 0; j < n_kv && ok; ++j) {
      const uint32_t jp = (uint32_t)(j & 1);
      if (!mbar_wait(s_full, jp, p.status, 0x330u)) { ok = false; break; }
      tc_fence_after();
      const int key0 = j * FB;
      const int limit = p.causal ? (q_idx + p.q_offset - key0) : (p.sk - 1 - key0);   // keys [0, limit] of this tile are visible
      const bool need_mask = limit < FB - 1 || key0 + FB > p.sk;
      const int vis = min(limit, p.sk - 1 - key0);
      // pass 1: row maximum
      float m_tile = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < FB; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tS + lane_addr + (uint32_t)c, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(r[i]);
          if (need_mask && c + i > vis) v = -INFINITY;
          m_tile = fmaxf(m_tile, v);
        }
      }
      const float m_new = fmaxf(m_run, m_tile);
      const float m_scaled = (m_new == -INFINITY) ? 0.f : m_new * p.scale_log2;
      const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run * p.scale_log2 - m_scaled);
      // pass 2: probabilities -> shared memory (bf16, swizzled K-major), row sum
      float l_tile = 0.f;
#pragma unroll 1
      for (int c = 0; c < FB; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tS + lane_addr + (uint32_t)c, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float a = __uint_as_float(r[2 * i]), b = __uint_as_float(r[2 * i + 1]);
          float pa = (need_mask && c + 2 * i > vis) ? 0.f : exp2f(a * p.scale_log2 - m_scaled);
          float pb = (need_mask && c + 2 * i + 1 > vis) ? 0.f : exp2f(b * p.scale_log2 - m_scaled);
          l_tile += pa + pb;
          __nv_bfloat162 h = __floats2bfloat162_rn(pa, pb);
          pk[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        // 32 keys = 4 chunks of 16 bytes; chunk index inside the 128-byte row is XOR-ed with (row & 7)
        uint8_t* blk = p_row + (c >> 6) * HALF_BYTES;
        const int chunk0 = (c & 63) >> 3;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int phys = (chunk0 + ch) ^ (row & 7);
          *reinterpret_cast<uint4*>(blk + phys * 16) = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
        }
      }
      tc_fence_before();
      mbar_arrive(s_empty);
      fence_proxy_async_smem();
      mbar_arrive(p_full);
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      if (!mbar_wait(pv_full, jp, p.status, 0x331u)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < FD; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tO + lane_addr + (uint32_t)c, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * alpha + __uint_as_float(r[i]);
      }
      tc_fence_before();
      mbar_arrive(o_empty);
    }
    if (ok && q_idx < p.sq) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.O + (((size_t)q_idx * p.b + batch) * p.nq + head) * FD;
#pragma unroll
      for (int c = 0; c < FD; c += 8) {
        uint32_t pk[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 h = __floats2bfloat162_rn(o[c + 2 * i] * inv, o[c + 2 * i + 1] * inv);
          pk[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(orow + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      p.lse[((size_t)batch * p.nq + head) * p.sq + q_idx] = (l_run > 0.f) ? m_run * p.scale + __logf(l_run) : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}
}  // namespace

// q [sq, b, nq, 128], k / v [sk, b, nkv, 128] bf16 with element strides (seq, batch, head); last dim contiguous.
MSB_API int msb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int sq, int sk, int b, int nq, int nkv,
                          long long q_ss, long long q_sb, long long q_sh, long long k_ss, long long k_sb, long long k_sh,
                          long long v_ss, long long v_sb, long long v_sh, int causal, int q_offset, float scale,
                          unsigned int* status, cudaStream_t s) {
  MSB_REQUIRE(sq > 0 && sk > 0 && nq % nkv == 0, "flash_fwd: bad shape sq=%d sk=%d nq=%d nkv=%d", sq, sk, nq, nkv);
  MSB_REQUIRE(status != nullptr, "flash_fwd: status word is required");
  FlashParams p;
  memset(&p, 0, sizeof(p));
  auto mk = [&](CUtensorMap* tm, const void* base, int seq, int heads, long long ss, long long sb, long long sh) {
    uint64_t dims[4] = {(uint64_t)FD, (uint64_t)heads, (uint64_t)b, (uint64_t)seq};
    uint64_t str[3] = {(uint64_t)sh * 2, (uint64_t)sb * 2, (uint64_t)ss * 2};
    uint32_t box[4] = {64, 1, 1, (uint32_t)FB};
    return make_tmap_nd(tm, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 4, dims, str, box);
  };
  int rc = mk(&p.tmQ, q, sq, nq, q_ss, q_sb, q_sh); if (rc) return rc;
  rc = mk(&p.tmK, k, sk, nkv, k_ss, k_sb, k_sh); if (rc) return rc;
  rc = mk(&p.tmV, v, sk, nkv, v_ss, v_sb, v_sh); if (rc) return rc;
  p.O = (__nv_bfloat16*)o; p.lse = lse;
  p.sq = sq; p.sk = sk; p.b = b; p.nq = nq; p.nkv = nkv; p.causal = causal; p.q_offset = q_offset;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashSmem::TOTAL);
    if (e != cudaSuccess) { msb_set_error("flash_fwd: cannot set dynamic shared memory: %s", cudaGetErrorString(e)); return 1; }
    attr = true;
  }
  dim3 grid((sq + FB - 1) / FB, nq, b);
  flash_fwd_sm100_kernel<<<grid, 192, FlashSmem::TOTAL, s>>>(p);
  MSB_CHECK_LAUNCH("flash_fwd_sm100");
  return 0;
}
