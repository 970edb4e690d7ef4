// Host algorithms of adaptive context parallelism for arbitrary attention masks:
//   coarsen_mask      reduce a [S, S] boolean mask to [S/b, S/b] blocks (a block is "on" if any element is), threaded
//   search_kmeans     group sequence blocks with similar mask columns so that each rank needs few remote KV blocks
//   schedule_rounds   greedy assignment of the needed (q-rank, kv-rank) block exchanges to rounds, at most
//                     `comm_limit` sends and receives per rank per round
// reference: mindspeed/ops/csrc/algorithm/adaptive_cp/adaptive_cp.cpp:47-454,
// mindspeed/core/context_parallel/utils.py:362-708.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <random>
#include <thread>
#include <vector>

#define MSB_HOST_API extern "C" __attribute__((visibility("default")))

MSB_HOST_API void msb_coarsen_mask(const uint8_t* mask, int64_t S, int64_t block, uint8_t* out, int threads) {
  const int64_t nb = S / block;
  if (threads < 1) threads = 1;
  auto work = [&](int64_t lo, int64_t hi) {
    for (int64_t bi = lo; bi < hi; ++bi)
      for (int64_t bj = 0; bj < nb; ++bj) {
        uint8_t any = 0;
        for (int64_t i = 0; i < block && !any; ++i) {
          const uint8_t* row = mask + (bi * block + i) * S + bj * block;
          for (int64_t j = 0; j < block; ++j) if (row[j]) { any = 1; break; }
        }
        out[bi * nb + bj] = any;
      }
  };
  std::vector<std::thread> pool;
  const int64_t per = (nb + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    int64_t lo = t * per, hi = std::min<int64_t>(nb, lo + per);
    if (lo < hi) pool.emplace_back(work, lo, hi);
  }
  for (auto& th : pool) th.join();
}

// k-means over the rows of a coarse mask [nb, nb] (as 0/1 vectors) into `k` equal-sized clusters (balanced:
// every rank must hold nb/k blocks).  Returns the permutation `order` (cluster-major) of the nb blocks.
MSB_HOST_API void msb_search_kmeans(const uint8_t* coarse, int64_t nb, int k, int iters, uint64_t seed, int64_t* order) {
  const int64_t per = nb / k;
  std::vector<double> cent((size_t)k * nb, 0.0);
  std::mt19937_64 rng(seed);
  std::vector<int64_t> idx(nb);
  for (int64_t i = 0; i < nb; ++i) idx[i] = i;
  // initial centroids: evenly spaced rows (deterministic, good for banded masks)
  for (int c = 0; c < k; ++c)
    for (int64_t j = 0; j < nb; ++j) cent[(size_t)c * nb + j] = coarse[(c * per + per / 2) * nb + j];
  std::vector<int> assign(nb, 0);
  for (int it = 0; it < iters; ++it) {
    // balanced assignment: sort (distance, row, cluster) and fill clusters up to `per`
    struct Cand { double d; int64_t row; int c; };
    std::vector<Cand> cands;
    cands.reserve((size_t)nb * k);
    for (int64_t r = 0; r < nb; ++r)
      for (int c = 0; c < k; ++c) {
        double d = 0;
        for (int64_t j = 0; j < nb; ++j) { double t = coarse[r * nb + j] - cent[(size_t)c * nb + j]; d += t * t; }
        cands.push_back({d, r, c});
      }
    std::stable_sort(cands.begin(), cands.end(), [](const Cand& a, const Cand& b) { return a.d < b.d; });
    std::vector<int64_t> fill(k, 0);
    std::vector<char> done(nb, 0);
    for (auto& cd : cands) {
      if (done[cd.row] || fill[cd.c] >= per) continue;
      assign[cd.row] = cd.c; done[cd.row] = 1; fill[cd.c]++;
    }
    std::fill(cent.begin(), cent.end(), 0.0);
    for (int64_t r = 0; r < nb; ++r)
      for (int64_t j = 0; j < nb; ++j) cent[(size_t)assign[r] * nb + j] += coarse[r * nb + j] / (double)per;
  }
  int64_t pos = 0;
  for (int c = 0; c < k; ++c)
    for (int64_t r = 0; r < nb; ++r) if (assign[r] == c) order[pos++] = r;
}

// need[q * cp + kv] != 0 when rank q needs the KV block of rank kv (q != kv).  Assign each needed pair a round so that in
// every round each rank sends at most `comm_limit` blocks and receives at most `comm_limit` blocks.
// round_of[q * cp + kv] = round index (or -1); returns the number of rounds.
MSB_HOST_API int msb_schedule_rounds(const uint8_t* need, int cp, int comm_limit, int* round_of) {
  std::vector<std::pair<int, int>> pairs;
  for (int q = 0; q < cp; ++q)
    for (int kv = 0; kv < cp; ++kv) {
      round_of[q * cp + kv] = -1;
      if (q != kv && need[q * cp + kv]) pairs.push_back({q, kv});
    }
  int rounds = 0;
  std::vector<char> placed(pairs.size(), 0);
  size_t left = pairs.size();
  while (left > 0) {
    std::vector<int> sends(cp, 0), recvs(cp, 0);
    for (size_t i = 0; i < pairs.size(); ++i) {
      if (placed[i]) continue;
      int q = pairs[i].first, kv = pairs[i].second;
      if (recvs[q] < comm_limit && sends[kv] < comm_limit) {
        recvs[q]++; sends[kv]++;
        round_of[q * cp + kv] = rounds;
        placed[i] = 1; left--;
      }
    }
    rounds++;
  }
  return rounds;
}
