/* Exact-fp32 two-sided product  P = L * G * R  for one block, and an entry point for callers
 * that must not allocate device memory.
 *
 * `two_sided_apply` is the fp32 (CUDA-core) form of the preconditioner application
 * P = L^(-1/p) G R^(-1/p).  It runs two chained GEMM launches and needs an m x n intermediate
 * T = G R between them; the regular entry point (bound to Python as `two_sided_apply`) gets that
 * scratch from the caller's allocator.
 *
 * ob200_two_sided_apply_noalloc has no counterpart in the reference library.  It exists for
 * callers that cannot call cudaMalloc or any allocating routine at the point where they need
 * the product: code running inside a memory-frozen region (for example between a framework's
 * "no more allocations" checkpoint and the end of a step), plug-ins loaded into a host process
 * that owns the whole device heap, or real-time loops where an allocation's latency and its
 * implicit synchronisation are not acceptable.  The intermediate T lives in a file-scope
 * `static __device__` array inside the library instead.
 *
 * Contract
 *   - L is m x m, G is m x n, R is n x n, P is m x n; all row-major contiguous fp32 device
 *     pointers on the current device.  P may not alias the inputs.
 *   - m * n must not exceed OB200_NOALLOC_MAX_ELEMS (1 Mi elements = 4 MiB); larger products are
 *     rejected with OB200_NOALLOC_ERR_TOO_LARGE and nothing is launched.  Every GPU that loads
 *     the library holds this 4 MiB array until the process exits.
 *   - The function calls no cudaMalloc, cudaFree or other allocating routine (no torch allocator
 *     either).  The first call on each device resolves the device address of the scratch array
 *     (cudaGetSymbolAddress, with that device current) and caches it; make that first call
 *     outside of any stream capture.
 *   - All calls on a device share the one scratch array, which keeps the previous call's
 *     contents.  Nothing in it has to start at zero: each call overwrites the m x n region it
 *     later reads.  Two calls that overlap on the GPU (different streams without an ordering
 *     between them) race on the array; serialise them on one stream or with events.
 *   - The work is enqueued on `stream` and the function returns without synchronising.
 *   - The function may be called from several host threads.  Threads that make the first call on
 *     a device at the same time each resolve the scratch address (the same value) themselves.
 *   - The return code reports this call's own launches: a launch error left pending by an earlier,
 *     unrelated CUDA call of the process is cleared, not reported; errors that only show when the
 *     kernels execute surface at the caller's next synchronisation, as with any launch.
 *
 * Returns 0 on success or one of the negative codes below; ob200_noalloc_strerror gives a text.
 */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OB200_NOALLOC_MAX_ELEMS (1 << 20)

#define OB200_NOALLOC_OK 0
#define OB200_NOALLOC_ERR_BAD_ARGUMENT (-1)
#define OB200_NOALLOC_ERR_TOO_LARGE (-2)
#define OB200_NOALLOC_ERR_CUDA (-3)

int ob200_two_sided_apply_noalloc(const float* L, const float* G, const float* R, float* P, int m, int n,
                                  cudaStream_t stream);

const char* ob200_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
namespace ob200 {
/* The regular entry point: same kernels, intermediate supplied by the caller (m x n fp32). */
void launch_two_sided_apply(const float* L, const float* G, const float* R, float* P, float* scratch, int m, int n,
                            cudaStream_t stream);
}  // namespace ob200
#endif
