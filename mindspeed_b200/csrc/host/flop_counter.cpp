// FLOP formulas and a process-wide counter for MFU / HFU accounting.
// Op wrappers add their FLOPs while the counter is running; it is paused during recompute so that the "model"
// (MFU) and "hardware" (HFU) totals can be told apart
// (reference: mindspeed/ops/csrc/flop_counter/flop_counter.h:27-40, flop_counter.cpp:22-362;
// pause/resume semantics mindspeed/functional/tflops_calculate/tflops_utils.py:37-60).
#include <atomic>
#include <cstdint>

#define MSB_HOST_API extern "C" __attribute__((visibility("default")))

namespace {
std::atomic<long long> g_model{0}, g_hardware{0};
std::atomic<int> g_running{0}, g_recompute{0};
}

MSB_HOST_API long long msb_mm_flop(long long m, long long n, long long k) { return 2 * m * n * k; }
MSB_HOST_API long long msb_bmm_flop(long long b, long long m, long long n, long long k) { return 2 * b * m * n * k; }
// fused GEMM + collective: the GEMM of the full (gathered / unreduced) problem on this rank
MSB_HOST_API long long msb_coc_flop(long long m, long long n, long long k, int world, int gathers_m) {
  return 2 * (gathers_m ? m * world : m) * n * k;
}
// attention: QK^T and PV, sparse = fraction of the score matrix actually computed (0.5 for causal)
MSB_HOST_API long long msb_flash_attention_forward_flop(long long b, long long heads, long long sq, long long sk, long long d,
                                                        long long dv, double sparse) {
  return (long long)((2.0 * b * heads * sq * sk * d + 2.0 * b * heads * sq * sk * dv) * sparse);
}
MSB_HOST_API long long msb_flash_attention_backward_flop(long long b, long long heads, long long sq, long long sk, long long d,
                                                         long long dv, double sparse) {
  // recomputed S, dP, dV, dK, dQ: 2.5x the forward
  return (long long)(2.5 * (2.0 * b * heads * sq * sk * d + 2.0 * b * heads * sq * sk * dv) * sparse);
}
MSB_HOST_API long long msb_gmm_flop(const long long* group_rows, int groups, long long k, long long n) {
  long long rows = 0;
  for (int i = 0; i < groups; ++i) rows += group_rows[i];
  return 2 * rows * k * n;
}
MSB_HOST_API long long msb_gmm_add_flop(const long long* group_rows, int groups, long long k, long long n) {
  return msb_gmm_flop(group_rows, groups, k, n);
}

MSB_HOST_API void msb_flops_start() { g_model = 0; g_hardware = 0; g_running = 1; g_recompute = 0; }
MSB_HOST_API void msb_flops_stop() { g_running = 0; }
MSB_HOST_API void msb_flops_enter_recompute() { g_recompute.fetch_add(1); }
MSB_HOST_API void msb_flops_exit_recompute() { g_recompute.fetch_sub(1); }
MSB_HOST_API void msb_flops_add(long long f) {
  if (!g_running.load()) return;
  g_hardware.fetch_add(f);
  if (g_recompute.load() == 0) g_model.fetch_add(f);
}
MSB_HOST_API long long msb_flops_model() { return g_model.load(); }
MSB_HOST_API long long msb_flops_hardware() { return g_hardware.load(); }
