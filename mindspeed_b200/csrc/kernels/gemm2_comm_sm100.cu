// Fused GEMM + collective on CTA pairs (tcgen05 cta_group::2) over NVLink peer memory, sm_100a.
//
//   MODE_AG   Y[M,N] = allgather(x)[M,K] * B        (column-parallel forward, row-parallel data gradient)
//   MODE_RS   Y[M/W,N] = reduce_scatter(x[M,K] * B)  (row-parallel forward, column-parallel data gradient)
//             optionally followed, in the same kernel, by the all-gather of the reduced rows (= all-reduce)
//
// Everything that crosses NVLink is a TMA bulk STORE into a peer's memory (posted writes; no remote loads):
//
// MODE_AG  Rank r owns rows [r*R, (r+1)*R) of the gathered operand and has written them into slab r of its OWN gathered
//   buffer (symmetric heap) before the launch.  A copy warp in every CTA pushes this rank's slab to the peers in W-1
//   phases: in phase s all of it goes to rank (r - s), which is the order in which that peer consumes slabs (its own
//   first, then r+1, r+2, ...), and in every phase each GPU sends to exactly one peer and receives from exactly one.  A
//   push is an 8 KB bulk load from local memory into a shared-memory ring followed by a bulk store to the peer; when
//   the store has completed the copy warp adds one to the peer's arrival counter of that 256-row tile.  The TMA
//   producer of a tile whose rows are remote waits (bounded) for the counter to reach the tile's chunk count, then
//   loads A from LOCAL memory.  A remote row therefore crosses NVLink once and the filled buffer is the gathered input
//   that backward needs.
//
// MODE_RS  Tiles are visited owner by owner, own rows first, then rank+1, rank+2, ...  The epilogue stages each
//   32 x 64 piece in shared memory and TMA-stores it straight into slab `rank` of the OWNER's staging area
//   [W][R, N] (the own slab is a local store): no partial buffer, no re-read.  Per owner a counter on the sending GPU
//   counts finished epilogue warps; the warp that completes an owner's tiles raises this rank's flag at the owner.
//   When all tiles are done every CTA waits (bounded) for the W flags of its own staging area and the whole grid sums
//   the W slabs in rank order in fp32 (+ optional residual) into the output: deterministic.  With `ar_out` set the
//   reduced rows are also written to every peer's output (all-reduce) and a final flag round makes them visible.
//
// Both modes start with an all-to-all epoch handshake: every peer has entered this call, so its previous use of the
// shared buffers is over and its inputs are in place.  Every wait is bounded; a time-out sets the status word and all
// roles fall through to the teardown.
//
// reference semantics being replaced: the fused vendor ops npu_all_gather_base_mm / npu_mm_reduce_scatter_base /
// npu_mm_all_reduce_base (mindspeed/core/tensor_parallel/mc2_feature/linear_function.py:40,169;
// mindspeed/ops/csrc/atb/lcal_coc.cpp:39-183).
#include "msb_common.cuh"
#include "msb_sm100.cuh"

using namespace msb;
using namespace msb::sm100;

namespace {

constexpr int BM = 128;          // rows per CTA; the pair covers 256
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int MAX_R = 8;
constexpr int NSTAGE = 5;
constexpr int RING = 4;          // copy ring slots
constexpr int CHUNK = 8192;      // bytes per pushed chunk

enum CommMode : int { MODE_AG = 1, MODE_RS = 2 };

// flag words in each rank's symmetric heap (u32 index)
constexpr int F_ENTRY = 0;       // [W] entry flags, written by peers
constexpr int F_DONE = 8;        // [W] RS: "rank r has stored everything it owes me"; AG: unused
constexpr int F_ARRIVE = 16;     // local CTA arrival counter
constexpr int F_PHASE = 24;      // [W] RS: local count of finished epilogue warps per owner
constexpr int F_AR = 32;         // [W] all-reduce: "rank r has written its reduced rows into my output"
constexpr int F_READY = 64;      // AG: per-256-row-tile arrival counters

struct Comm2Params {
  CUtensorMap tmA, tmB;
  CUtensorMap tmD[MAX_R];        // AG: [0] = local output [M, N]; RS: [o] = slab `rank` of owner o's staging [R, N]
  int M, N, K;
  int world, rank;
  int rows_per_rank;             // R
  int group_m;                   // 256-row tiles per L2 group (divides R / 256)
  unsigned int epoch;
  unsigned int* flag_local;
  unsigned int* flag_peer[MAX_R];
  unsigned int* status;
  unsigned long long wait_ns;    // limit of every cross-GPU wait
  // AG
  const uint8_t* ag_local;       // this rank's gathered buffer [M, K]
  uint8_t* ag_peer[MAX_R];       // every rank's gathered buffer
  unsigned int ready_target;     // chunks per 256-row tile
  // RS tail
  const uint4* stage_local;      // own staging [W][R, N]
  uint4* out;                    // [R, N]
  const uint4* residual;         // optional [R, N]
  uint4* ar_out[MAX_R];          // optional: every rank's all-reduce output [M, N]
  unsigned long long* timeline;  // optional [8]: %globaltimer stamps written by CTA 0 (entry, handshake done, copy / producer /
                                 // epilogue loops done, RS flags in, RS sum done); for the micro-benchmark's breakdown
};

struct Smem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;            // 32 KB
  static constexpr int EPI_BUF = 4096;                             // 32 rows x 64 bf16
  static constexpr int EPI_OFFSET = NSTAGE * STAGE_BYTES;          // 160 KB
  static constexpr int RING_OFFSET = EPI_OFFSET + 4 * 2 * EPI_BUF; // + 32 KB
  static constexpr int BAR_OFFSET = RING_OFFSET + RING * CHUNK;    // + 32 KB
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
  static_assert(TOTAL <= 232448, "exceeds the 227 KB of shared memory a CTA may use");
};

__device__ __forceinline__ bool wait_flag_ge(const unsigned int* flag, unsigned int value, unsigned int* status,
                                             unsigned int code, uint64_t limit_ns) {
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int)(v - value) >= 0) return true;
    if (globaltimer_ns() - t0 > limit_ns) { atomicCAS(status, 0u, code); return false; }
    if (*((volatile unsigned int*)status) != 0u) return false;
    __nanosleep(100);
  }
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// untiled bulk copies: global -> shared (mbarrier byte count) and shared -> global (bulk group)
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Tile order.
// MODE_AG: m-tiles (256 rows) grouped so that a group never straddles two ranks' rows, groups visited starting at this
//   rank's rows (the order in which slabs arrive); inside a group n-major so CTA pairs running together share A and B panels.
// MODE_RS: consecutive tiles belong to consecutive owners (rank+1, rank+2, ..., own rows last in every round of W tiles), so at
//   any moment the pairs of this GPU store to all peers at once and NVLink is busy for the whole kernel instead of idling
//   while the own rows are computed.  Tiles are grouped (about 8 m-tiles, the same number from every owner) and swept n-major
//   inside a group, so the group's A panels stay in L2 while the B panels stream.
template <int MODE>
__device__ __forceinline__ void tile_mn(int t, int num_m, int num_n, int group_m, int rot, int world, int rank, int tiles_per_rank,
                                        int& m, int& n) {
  if (MODE == MODE_RS) {
    // group = `group_m` m-tiles of EVERY owner; inside a group n is the slow index and owners alternate fastest
    const int gw = group_m * world;
    const int per_group = gw * num_n;
    const int g = t / per_group;
    const int r = t - g * per_group;
    n = r / gw;
    const int mm = r - n * gw;
    const int owner = (rank + 1 + mm % world) % world;
    m = owner * tiles_per_rank + g * group_m + mm / world;
    return;
  }
  const int per_group = group_m * num_n;
  const int g = t / per_group;
  const int r = t - g * per_group;
  m = g * group_m + (r % group_m);
  n = r / group_m;
  m = (m + rot) % num_m;
}

template <int MODE, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(224, 1) gemm2_comm_kernel(const __grid_constant__ Comm2Params p) {
  using L = Smem;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (NSTAGE + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + 2 + a); };
  auto ring_bar = [&](int i) { return bar_base + 8u * (2 * NSTAGE + 4 + i); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * NSTAGE + 4 + RING);
  uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  __shared__ int s_ok;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int num_m = p.M / (2 * BM), num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int tiles_per_rank = p.rows_per_rank / (2 * BM);
  const int rot = (MODE == MODE_AG ? p.rank : p.rank) * tiles_per_rank;     // both modes start at the own rows
  constexpr uint32_t TMEM_COLS = 512u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 8); }
    for (int i = 0; i < RING; ++i) mbar_init(ring_bar(i), 1);
    mbar_fence_init();
    s_ok = 1;
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  auto stamp = [&](int i) { if (p.timeline && blockIdx.x == 0) p.timeline[i] = globaltimer_ns(); };
  if (threadIdx.x == 0) stamp(0);
  // ---- entry handshake: every peer has entered this call ----
  bool alive = true;
  {
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
      __threadfence_system();
      st_release_sys(p.flag_peer[threadIdx.x] + F_ENTRY + p.rank, p.epoch);
    }
    if (threadIdx.x < p.world)
      alive = wait_flag_ge(p.flag_local + F_ENTRY + threadIdx.x, p.epoch, p.status, 0x100u + threadIdx.x, p.wait_ns);
    alive = __syncthreads_and(alive);
  }
  if (threadIdx.x == 0) stamp(1);

  if (alive) {
    if (warp == 0) {
      // ===================== TMA producer (both CTAs) =====================
      if (lane == 0) {
        int stage = 0; uint32_t phase = 0;
        for (int t = pair; t < num_tiles && alive; t += npairs) {
          int m_blk, n_blk;
          tile_mn<MODE>(t, num_m, num_n, p.group_m, rot, p.world, p.rank, tiles_per_rank, m_blk, n_blk);
          if (MODE == MODE_AG && (m_blk / tiles_per_rank) != p.rank) {
            if (!wait_flag_ge(p.flag_local + F_READY + m_blk, p.ready_target, p.status, 0x40u, p.wait_ns)) { alive = false; break; }
            asm volatile("fence.proxy.async.global;" ::: "memory");   // peers' writes -> this thread's TMA (async proxy) reads
          }
          const int m0 = m_blk * (2 * BM) + (int)cta * BM;
          const int n0 = n_blk * BN + (int)cta * (BN / 2);
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 0x10u)) { alive = false; break; }
            const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
            const uint32_t sb = sa + L::A_BYTES;
            if (cta == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
            const uint32_t lead_full = mapa_u32(full_bar(stage), 0);
            const int k0 = kb * BK;
            tma_load_2d_pair(sa, &p.tmA, lead_full, k0, m0);
            if (!B_MN) {
              tma_load_2d_pair(sb, &p.tmB, lead_full, k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j) tma_load_2d_pair(sb + j * (BK * 128), &p.tmB, lead_full, n0 + j * 64, k0);
            }
            if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
          }
        }
        stamp(3);
        for (int i = 0; i < NSTAGE && alive; ++i) {      // tail: all commits aimed at this CTA have landed
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, 0x11u)) { alive = false; break; }
          if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
        }
      }
    } else if (warp == 1) {
      // ===================== MMA issuer (leader CTA) =====================
      if (lane == 0 && cta == 0) {
        constexpr uint32_t idesc = make_idesc_f16(2 * BM, BN, 1, 0, B_MN ? 1 : 0);
        int stage = 0; uint32_t phase = 0;
        int acc = 0; uint32_t acc_phase = 0;
        for (int t = pair; t < num_tiles && alive; t += npairs) {
          if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, p.status, 0x20u, p.wait_ns)) { alive = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, p.status, 0x21u, p.wait_ns)) { alive = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_base + stage * L::STAGE_BYTES;
            const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t adesc = make_smem_desc(sa + k * (UMMA_K * 2), 0, 1024);
              const uint64_t bdesc = B_MN ? make_smem_desc(sb + k * (UMMA_K * 128), BK * 128, 1024)
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
    } else if (warp < 6) {
      // ===================== epilogue (warps 2..5, both CTAs) =====================
      const int q = warp & 3;
      const uint32_t buf_base = smem_base + L::EPI_OFFSET + (uint32_t)q * 2u * L::EPI_BUF;
      const uint32_t lead_tempty[2] = {mapa_u32(tempty_bar(0), 0), mapa_u32(tempty_bar(1), 0)};
      const unsigned int owner_target = (unsigned int)(tiles_per_rank * num_n * 8);   // epilogue warps per owner
      int acc = 0; uint32_t acc_phase = 0;
      uint32_t chunk = 0;
      unsigned int owner_count[MAX_R];                     // RS: tiles of each owner this warp has stored
#pragma unroll
      for (int o = 0; o < MAX_R; ++o) owner_count[o] = 0;
      // RS: this warp's tiles are in the owners' staging once its stores have completed; it then adds its counts to this
      // GPU's per-owner counters and, for every owner whose last warp-tile is in, raises this rank's flag at that owner.
      // One full-completion wait per warp, not per tile: stores of consecutive tiles stay in flight.
      auto finish_owners = [&]() {
        if (MODE != MODE_RS || lane != 0) return;
        tma_store_wait<0>();
        __threadfence_system();
#pragma unroll
        for (int o = 0; o < MAX_R; ++o) {
          if (o >= p.world) break;
          // every warp reports to every owner's counter (possibly with 0) so the last reporter can be recognised
          const unsigned int prev = atomicAdd(p.flag_local + F_PHASE + o, owner_count[o] + 0x10000u);
          if ((prev >> 16) + 1u == (unsigned int)(gridDim.x * 4) && (prev & 0xffffu) + owner_count[o] == owner_target) {
            p.flag_local[F_PHASE + o] = 0u;                             // ready for the next call
            __threadfence_system();
            st_release_sys(p.flag_peer[o] + F_DONE + p.rank, p.epoch);
          }
        }
      };
      for (int t = pair; t < num_tiles && alive; t += npairs) {
        int m_blk, n_blk;
        tile_mn<MODE>(t, num_m, num_n, p.group_m, rot, p.world, p.rank, tiles_per_rank, m_blk, n_blk);
        if (!mbar_wait_warp(tfull_bar(acc), acc_phase, p.status, 0x30u, p.wait_ns)) { alive = false; break; }
        tc_fence_after();
        const int owner = m_blk / tiles_per_rank;
        if (MODE == MODE_RS) {
#pragma unroll
          for (int o = 0; o < MAX_R; ++o) if (o == owner) ++owner_count[o];
        }
        const int row0 = m_blk * (2 * BM) + (int)cta * BM + q * 32;
        const int drow = (MODE == MODE_RS) ? row0 - owner * p.rows_per_rank : row0;
        const CUtensorMap* tmD = (MODE == MODE_RS) ? &p.tmD[owner] : &p.tmD[0];
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
          const uint32_t buf = buf_base + (chunk & 1u) * L::EPI_BUF;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          const uint32_t row_addr = buf + (uint32_t)lane * 128u;
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
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(tmD, buf, col0, drow);
            tma_store_commit();
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_tempty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      if (alive) finish_owners();
      if (lane == 0) tma_store_wait<0>();
      if (warp == 2 && lane == 0) stamp(4);
    } else if (MODE == MODE_AG) {
      // ===================== copy warp (warp 6): push this rank's slab to the peers =====================
      if (lane == 0) {
        const uint32_t ring = smem_base + L::RING_OFFSET;
        const size_t slab_bytes = (size_t)p.rows_per_rank * (size_t)p.K * 2;
        const size_t slab_off = (size_t)p.rank * slab_bytes;
        const int chunks_per_slab = (int)(slab_bytes / CHUNK);
        const size_t tile_bytes = (size_t)(2 * BM) * (size_t)p.K * 2;
        const int per_phase = (chunks_per_slab - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // my chunks per phase
        const int total = per_phase * (p.world - 1);
        // item i -> (phase s = i / per_phase, chunk c = blockIdx.x + (i % per_phase) * gridDim.x)
        auto item = [&](int i, int& dst, size_t& off) {
          const int s = i / per_phase + 1;
          dst = (p.rank - s + p.world) % p.world;
          off = slab_off + (size_t)(blockIdx.x + (i - (s - 1) * per_phase) * gridDim.x) * CHUNK;
        };
        // Pipeline per CTA: loads (local memory -> ring) run LAG items ahead of stores (ring -> peer); a ring slot is
        // reused as soon as its store has READ it, so the number of stores in flight is not bounded by the ring.  Items
        // are signalled in batches once their stores have fully completed (checked SIG_LAG stores later, without
        // draining the pipeline): one system-scope fence per batch, then one relaxed add per (peer, tile) run.
        constexpr int LAG = 2;
        constexpr int SIG_LAG = 4;
        constexpr int SIG_BATCH = 8;
        int stored = 0, signalled = 0;
        auto signal_upto = [&](int upto) {
          if (upto <= signalled) return;
          __threadfence_system();
          int run_dst = -1, run_tile = -1; unsigned int run = 0;
          auto emit = [&]() {
            if (run) asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p.flag_peer[run_dst] + F_READY + run_tile), "r"(run) : "memory");
          };
          for (; signalled < upto; ++signalled) {
            int dst; size_t off;
            item(signalled, dst, off);
            const int tile = (int)(off / tile_bytes);
            if (dst != run_dst || tile != run_tile) { emit(); run_dst = dst; run_tile = tile; run = 0; }
            ++run;
          }
          emit();
        };
        uint32_t ring_phase = 0;   // bit i = parity of slot i's barrier
        auto store_item = [&](int k) -> bool {
          const int slot = k % RING;
          if (!mbar_wait(ring_bar(slot), (ring_phase >> slot) & 1u, p.status, 0x60u, p.wait_ns)) return false;
          ring_phase ^= 1u << slot;
          int dst; size_t off;
          item(k, dst, off);
          bulk_s2g(p.ag_peer[dst] + off, ring + slot * CHUNK, CHUNK);
          tma_store_commit();
          ++stored;
          if (stored - SIG_LAG - signalled >= SIG_BATCH) {
            tma_store_wait<SIG_LAG>();                 // all but the SIG_LAG most recent stores are complete
            signal_upto(stored - SIG_LAG);
          }
          return true;
        };
        for (int j = 0; j < total && alive; ++j) {
          if (j >= RING) tma_store_wait_read<RING - LAG - 1>();   // the store of item j - RING no longer reads its slot
          int dst; size_t off;
          item(j, dst, off);
          const int slot = j % RING;
          mbar_arrive_expect_tx(ring_bar(slot), CHUNK);
          bulk_g2s(ring + slot * CHUNK, p.ag_local + off, CHUNK, ring_bar(slot));
          if (j >= LAG && !store_item(j - LAG)) { alive = false; break; }
        }
        for (int k = max(total - LAG, 0); k < total && alive; ++k)
          if (!store_item(k)) alive = false;
        tma_store_wait<0>();
        if (alive) signal_upto(stored);
        stamp(2);
      }
    }
  }

  // ---- RS tail: wait for every rank's slab of my rows, sum them ----
  if (MODE == MODE_RS) {
    __syncthreads();
    if (threadIdx.x < p.world) {
      if (!wait_flag_ge(p.flag_local + F_DONE + threadIdx.x, p.epoch, p.status, 0x200u + threadIdx.x, p.wait_ns)) s_ok = 0;
    }
    if (threadIdx.x == 0 && *((volatile unsigned int*)p.status) != 0u) s_ok = 0;
    __syncthreads();
    if (threadIdx.x == 0) stamp(5);
    if (s_ok) {
      const long long n_v4 = (long long)p.rows_per_rank * p.N / 8;
      const long long ar_off = (long long)p.rank * n_v4;
      for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_v4; i += (long long)gridDim.x * blockDim.x) {
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = 0.f;
        for (int r = 0; r < p.world; ++r) {
          const uint4 v = ld_cg_v4(p.stage_local + (long long)r * n_v4 + i);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); a[2 * j] += f.x; a[2 * j + 1] += f.y; }
        }
        if (p.residual) {
          const uint4 v = p.residual[i];
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); a[2 * j] += f.x; a[2 * j + 1] += f.y; }
        }
        uint4 o;
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ho[j] = __floats2bfloat162_rn(a[2 * j], a[2 * j + 1]);
        if (p.out) p.out[i] = o;
        if (p.ar_out[0]) {
#pragma unroll 1
          for (int r = 0; r < p.world; ++r) p.ar_out[r][ar_off + i] = o;     // coalesced 16-byte stores, local and over NVLink
        }
      }
    }
    if (p.ar_out[0]) {
      // all-reduce: tell every peer that my rows are in its output, then wait for everybody's rows in mine
      __shared__ unsigned int last_cta;
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(p.flag_local + F_ARRIVE, 1u);
        last_cta = (prev == gridDim.x - 1) ? 1u : 0u;
      }
      __syncthreads();
      if (last_cta && threadIdx.x < p.world) {
        if (threadIdx.x == 0) p.flag_local[F_ARRIVE] = 0u;
        __threadfence_system();
        st_release_sys(p.flag_peer[threadIdx.x] + F_AR + p.rank, p.epoch);
      }
      if (threadIdx.x < p.world && s_ok)
        wait_flag_ge(p.flag_local + F_AR + threadIdx.x, p.epoch, p.status, 0x300u + threadIdx.x, p.wait_ns);
    }
  }

  // ---- teardown ----
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();
  if (threadIdx.x == 0) stamp(6);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int MODE, bool B_MN>
int launch_comm2(const Comm2Params& p, int pairs, cudaStream_t s) {
  auto kern = gemm2_comm_kernel<MODE, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::TOTAL);
    if (e != cudaSuccess) { msb_set_error("gemm2_comm: cannot set %d bytes of dynamic shared memory: %s", Smem::TOTAL, cudaGetErrorString(e)); return 1; }
    attr_set = true;
  }
  kern<<<2 * pairs, 224, Smem::TOTAL, s>>>(p);
  MSB_CHECK_LAUNCH("gemm2_comm");
  return 0;
}

}  // namespace

// Arguments shared by both fused launchers.  All symmetric buffers are given as per-rank base pointers.
struct MsbComm2Args {
  const void* A;                 // AG: this rank's gathered buffer [M, K] (own slab filled); RS: local activation [M, K]
  const void* B;                 // weight, K-major [N, K] (b_mn_major = 0) or MN-major [K, N] (1)
  void* D;                       // AG: output [M, N]; RS: output [M / world, N]
  const void* peer_buf[MAX_R];   // AG: every rank's gathered buffer; RS: every rank's staging [world][M / world, N]
  const void* residual;          // RS: optional bf16 [M / world, N] added in the final sum
  void* ar_out[MAX_R];           // RS: optional, every rank's all-reduce output [M, N] (symmetric); D may then be null
  int M, N, K;
  int b_mn_major;
  int world, rank;
  unsigned int epoch;
  unsigned int* flag_local;
  unsigned int* flag_peer[MAX_R];
  unsigned int* status;
  int wait_limit_ms;             // 0: default (10 s)
  int max_ctas;                  // 0: all SMs
  unsigned long long* timeline;  // optional [8] device words for CTA 0's time stamps
};

static int fill_comm2(Comm2Params& p, const MsbComm2Args* a, int mode) {
  memset(&p, 0, sizeof(p));
  int rc = make_tmap_2d(&p.tmA, a->A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->M, a->K, a->K, BM, BK);
  if (rc) return rc;
  if (!a->b_mn_major) rc = make_tmap_2d(&p.tmB, a->B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->N, a->K, a->K, BN / 2, BK);
  else rc = make_tmap_2d(&p.tmB, a->B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->K, a->N, a->N, BK, 64);
  if (rc) return rc;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.world = a->world; p.rank = a->rank; p.epoch = a->epoch;
  p.rows_per_rank = a->M / a->world;
  p.flag_local = a->flag_local;
  for (int i = 0; i < MAX_R; ++i) p.flag_peer[i] = a->flag_peer[i];
  p.status = a->status;
  p.timeline = a->timeline;
  p.wait_ns = (a->wait_limit_ms > 0 ? (unsigned long long)a->wait_limit_ms : 10000ull) * 1000000ull;
  const int tiles_per_rank = p.rows_per_rank / (2 * BM);
  p.group_m = 8;
  if (mode == MODE_RS) p.group_m = 8 / a->world > 0 ? 8 / a->world : 1;   // per owner; a group holds group_m * world m-tiles
  while (tiles_per_rank % p.group_m != 0) p.group_m >>= 1;
  if (mode == MODE_AG) {
    rc = make_tmap_2d(&p.tmD[0], a->D, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->M, a->N, a->N, 32, 64);
    if (rc) return rc;
    p.ag_local = reinterpret_cast<const uint8_t*>(a->A);
    for (int i = 0; i < a->world; ++i) p.ag_peer[i] = reinterpret_cast<uint8_t*>(const_cast<void*>(a->peer_buf[i]));
    p.ready_target = (unsigned int)(((size_t)(2 * BM) * a->K * 2) / CHUNK);
  } else {
    const size_t slab = (size_t)p.rows_per_rank * a->N * 2;
    for (int o = 0; o < a->world; ++o) {
      const uint8_t* base = reinterpret_cast<const uint8_t*>(a->peer_buf[o]) + (size_t)a->rank * slab;
      rc = make_tmap_2d(&p.tmD[o], base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.rows_per_rank, a->N, a->N, 32, 64);
      if (rc) return rc;
    }
    p.stage_local = reinterpret_cast<const uint4*>(a->peer_buf[a->rank]);
    p.out = reinterpret_cast<uint4*>(a->D);
    p.residual = reinterpret_cast<const uint4*>(a->residual);
    for (int i = 0; i < a->world; ++i) p.ar_out[i] = reinterpret_cast<uint4*>(a->ar_out[i]);
  }
  return 0;
}

static int check_comm2(const MsbComm2Args* a, const char* what) {
  MSB_REQUIRE(a->world >= 2 && a->world <= MAX_R, "%s: world size %d not in [2, %d]", what, a->world, MAX_R);
  MSB_REQUIRE(a->M % (a->world * 2 * BM) == 0, "%s: M=%d must be a multiple of world*256", what, a->M);
  MSB_REQUIRE(a->N % 8 == 0 && a->K % 8 == 0, "%s: N=%d and K=%d must be multiples of 8", what, a->N, a->K);
  MSB_REQUIRE(a->status && a->flag_local, "%s: status and flags are required", what);
  return 0;
}

static int pairs_for(const MsbComm2Args* a) {
  int pairs = msb::num_sms() / 2;
  if (a->max_ctas > 0 && pairs > a->max_ctas / 2) pairs = a->max_ctas / 2;
  return pairs < 1 ? 1 : pairs;
}

// True when the pair kernels cover this problem (else the caller uses the one-CTA fused kernels).
MSB_API int msb_gemm2_comm_supported(int M, int N, int K, int world, int mode) {
  if (world < 2 || world > MAX_R || M % (world * 2 * BM) != 0 || N % 8 != 0 || K % 8 != 0) return 0;
  if (mode == MODE_AG) {
    const size_t slab = (size_t)(M / world) * K * 2, tile = (size_t)(2 * BM) * K * 2;
    if (slab % CHUNK != 0 || tile % CHUNK != 0) return 0;
    if (M / (2 * BM) > 1024) return 0;            // arrival counters available in the flag area
  }
  return 1;
}

// Y[M, N] = allgather(x)[M, K] * B.  Every rank has already stored its rows into slab `rank` of its own gathered buffer.
MSB_API int msb_gemm2_allgather(const MsbComm2Args* a, cudaStream_t s) {
  int rc = check_comm2(a, "gemm2_allgather");
  if (rc) return rc;
  MSB_REQUIRE(msb_gemm2_comm_supported(a->M, a->N, a->K, a->world, MODE_AG), "gemm2_allgather: unsupported shape %dx%dx%d", a->M, a->N, a->K);
  Comm2Params p;
  rc = fill_comm2(p, a, MODE_AG);
  if (rc) return rc;
  if (cudaMemsetAsync(a->flag_local + F_READY, 0, sizeof(unsigned int) * (a->M / (2 * BM)), s) != cudaSuccess) {
    msb_set_error("gemm2_allgather: memset failed");
    return 1;
  }
  const int pairs = pairs_for(a);
  return a->b_mn_major ? launch_comm2<MODE_AG, true>(p, pairs, s) : launch_comm2<MODE_AG, false>(p, pairs, s);
}

// out[M/world, N] = reduce_scatter(x[M, K] * B) (+ residual); with ar_out set, every rank's ar_out receives all reduced rows.
MSB_API int msb_gemm2_reduce_scatter(const MsbComm2Args* a, cudaStream_t s) {
  int rc = check_comm2(a, "gemm2_reduce_scatter");
  if (rc) return rc;
  Comm2Params p;
  rc = fill_comm2(p, a, MODE_RS);
  if (rc) return rc;
  const int pairs = pairs_for(a);
  return a->b_mn_major ? launch_comm2<MODE_RS, true>(p, pairs, s) : launch_comm2<MODE_RS, false>(p, pairs, s);
}
