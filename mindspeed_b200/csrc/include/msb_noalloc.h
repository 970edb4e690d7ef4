/* Entry points of libmsb200_kernels.so that never allocate.
 *
 * This header has no counterpart in the reference framework; it exists for embedders of this library.
 *
 * Who needs it: code that runs where device memory may not be requested. Examples are a training or serving
 * process that hands its whole memory budget to one pool at start-up and forbids later cudaMalloc calls, a
 * callback running inside a caching allocator (allocating there would re-enter the allocator), and plain C or
 * C++ hosts that link this library without PyTorch and therefore have no tensor allocator to borrow scratch
 * from. The regular msb_rmsnorm_bwd() asks such callers for a scratch buffer they cannot supply.
 *
 * msb_rmsnorm_bwd_noalloc() computes exactly what msb_rmsnorm_bwd() computes:
 *     dx     = rstd * (dy*gamma - xhat * mean(dy*gamma*xhat)),   xhat = x * rstd
 *     dgamma = sum over rows of dy * xhat        (added to the existing dgamma when accumulate_dgamma != 0)
 * The caller passes only inputs and outputs. The partial sums that the two-stage dgamma reduction needs live in
 * a 2 MiB array compiled into the library; every GPU that loads the library keeps that array until the process
 * exits.
 *
 * Limits and rules:
 *   - cols must be a multiple of 8 and at most msb_rmsnorm_bwd_noalloc_max_cols() (8192). Anything else is
 *     refused with return code 2 and a message in msb_last_error(); nothing is launched.
 *   - The function calls no cudaMalloc, cudaFree or other allocating routine, on any call.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current) and remembers it. Make that first call during normal set-up, before any stream capture begins
 *     on that device. The remembered address is kept in a plain per-device table without a lock: two host threads
 *     that make their first call on the same device at the same time both look the address up and store the same
 *     value, which is harmless.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left in it. This
 *     function needs no clearing (it overwrites every slot it later reads), but two calls whose kernels can
 *     overlap on the GPU, for instance on two streams without an ordering between them, would race on the
 *     array. Order such calls on one stream or with events.
 *   - dtype codes: 0 = float32, 1 = bfloat16, 2 = float16; x, dy, gamma, dx and dgamma share the dtype,
 *     rstd is float32 with one value per row (as written by msb_rmsnorm_fwd).
 *
 * Returns 0 on success, 1 on a CUDA error, 2 on a refused argument.
 */
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

size_t msb_rmsnorm_bwd_noalloc_max_cols(void);

int msb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx,
                            void* dgamma, int rows, int cols, int zero_centered, int accumulate_dgamma, int dtype,
                            cudaStream_t stream);

#ifdef __cplusplus
}
#endif
