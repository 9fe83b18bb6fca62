// See two_sided_apply.h.
#include "two_sided_apply.h"

#include <atomic>
#include <cstdio>

namespace ob200 {

namespace {

constexpr int kT = 32;

// C[M,N] = A[M,K] * B[K,N], row-major fp32, shared-memory tiled, fp32 FMA accumulation.
__global__ void __launch_bounds__(kT* kT) sgemm_nn_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                         float* __restrict__ C, int M, int N, int K) {
  __shared__ float As[kT][kT + 1];
  __shared__ float Bs[kT][kT + 1];
  const int tx = threadIdx.x % kT, ty = threadIdx.x / kT;
  const int row = blockIdx.y * kT + ty, col = blockIdx.x * kT + tx;
  float acc = 0.f;
  for (int k0 = 0; k0 < K; k0 += kT) {
    As[ty][tx] = (row < M && k0 + tx < K) ? A[static_cast<long long>(row) * K + k0 + tx] : 0.f;
    Bs[ty][tx] = (k0 + ty < K && col < N) ? B[static_cast<long long>(k0 + ty) * N + col] : 0.f;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kT; ++k) acc = fmaf(As[ty][k], Bs[k][tx], acc);
    __syncthreads();
  }
  if (row < M && col < N) C[static_cast<long long>(row) * N + col] = acc;
}

void sgemm_nn(const float* A, const float* B, float* C, int M, int N, int K, cudaStream_t stream) {
  dim3 grid((N + kT - 1) / kT, (M + kT - 1) / kT);
  sgemm_nn_kernel<<<grid, kT * kT, 0, stream>>>(A, B, C, M, N, K);
}

// Intermediate of the no-allocation entry point.  In host code this name is only a stand-in
// for the symbol; its device address is obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[OB200_NOALLOC_MAX_ELEMS];

constexpr int kMaxDevices = 64;
// Device address of the scratch array, per device.  Threads that race on the first call of a
// device all resolve the same address; the atomic only makes the publication well defined.
std::atomic<float*> g_scratch_addr[kMaxDevices];

}  // namespace

void launch_two_sided_apply(const float* L, const float* G, const float* R, float* P, float* scratch, int m, int n,
                            cudaStream_t stream) {
  sgemm_nn(G, R, scratch, m, n, n, stream);  // T = G R
  sgemm_nn(L, scratch, P, m, n, m, stream);  // P = L T
}

}  // namespace ob200

extern "C" int ob200_two_sided_apply_noalloc(const float* L, const float* G, const float* R, float* P, int m, int n,
                                             cudaStream_t stream) {
  using namespace ob200;
  if (L == nullptr || G == nullptr || R == nullptr || P == nullptr || m <= 0 || n <= 0) {
    return OB200_NOALLOC_ERR_BAD_ARGUMENT;
  }
  if (static_cast<long long>(m) * n > OB200_NOALLOC_MAX_ELEMS) {
    std::fprintf(stderr,
                 "ob200_two_sided_apply_noalloc: m*n = %lld exceeds the built-in scratch of %d elements; "
                 "use the allocating entry point for this size\n",
                 static_cast<long long>(m) * n, OB200_NOALLOC_MAX_ELEMS);
    return OB200_NOALLOC_ERR_TOO_LARGE;
  }
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return OB200_NOALLOC_ERR_CUDA;
  float* scratch = g_scratch_addr[device].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // Once per device, with that device current: the symbol's address on *this* device.
    const cudaError_t err = cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_noalloc_scratch);
    if (err != cudaSuccess || scratch == nullptr) {
      std::fprintf(stderr, "ob200_two_sided_apply_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(err));
      return OB200_NOALLOC_ERR_CUDA;
    }
    g_scratch_addr[device].store(scratch, std::memory_order_release);
  }
  // The return code speaks for this call's two launches only: an error that some earlier,
  // unrelated call left pending is taken off first, and each launch is checked right after it.
  (void)cudaGetLastError();
  sgemm_nn(G, R, scratch, m, n, n, stream);  // T = G R
  cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess) {
    sgemm_nn(L, scratch, P, m, n, m, stream);  // P = L T
    err = cudaGetLastError();
  }
  if (err != cudaSuccess) {
    std::fprintf(stderr, "ob200_two_sided_apply_noalloc: kernel launch failed: %s\n", cudaGetErrorString(err));
    return OB200_NOALLOC_ERR_CUDA;
  }
  return OB200_NOALLOC_OK;
}

extern "C" const char* ob200_noalloc_strerror(int code) {
  switch (code) {
    case OB200_NOALLOC_OK:
      return "success";
    case OB200_NOALLOC_ERR_BAD_ARGUMENT:
      return "null pointer or non-positive dimension";
    case OB200_NOALLOC_ERR_TOO_LARGE:
      return "m * n exceeds OB200_NOALLOC_MAX_ELEMS (the built-in scratch holds 1 Mi fp32 elements)";
    case OB200_NOALLOC_ERR_CUDA:
      return "a CUDA runtime call failed";
    default:
      return "unknown code";
  }
}
