// Kernels over flat (contiguous) tensors: the tf32 (hi, lo) operand split, and the fused
// GPA-AdamW update and train/eval interpolation as single multi-tensor launches.
//
// gpa_adamw: one read and one write of p, z, m, v and one read of g per element, instead of the
// nine-plus pointwise launches and three temporaries per parameter of the reference loop
// (gpa/gpa_adamw.py:455-497); gpa_lerp replaces the per-parameter lerp_ of train()/eval()
// (gpa/gpa_adamw.py:307-357).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace ob200 {

constexpr int kGpaChunk = 4096;  // elements handled by one CTA iteration

struct GpaTensorDesc {
  void* param;       // fp32 / bf16 / fp16
  const void* grad;  // same dtype as param; null when the parameter has no gradient
  float* z;
  float* m;
  float* v;
  long long numel;
  int dtype;  // 0 fp32, 1 bf16, 2 fp16
  int pad_;
};

// One contiguous copy of a grouped scatter / gather over local and peer memory.
struct CopyDesc {
  const void* src;
  void* dst;
  long long bytes;  // multiple of 4
};

constexpr int kCopyChunkBytes = 64 * 1024;  // bytes handled by one CTA iteration

// peer_copy: every (src, dst, bytes) entry of the table in one launch; either side may be another
// GPU's memory (plain loads / stores over NVLink).  This is the data movement of the lossless
// fully-shard exchange: gradient shards pushed straight from the local shard tensors into the
// owners' receive buffers, updated parameter chunks pushed from the owners' full copies into the
// shard holders' receive buffers; packing into a send buffer and the collective call are gone
// (reference: distributed_shampoo/distributor/_shampoo_fully_shard_utils.py:519-588, :806-835).
void launch_peer_copy(const CopyDesc* table, const int2* chunks, int num_chunks, cudaStream_t stream);

// One symmetric matrix of a batched eigendecomposition.
struct JacobiDesc {
  const float* a;  // n x n, row pitch lda (symmetric)
  float* q;        // n x n, row pitch ldq: eigenvectors as columns, ascending eigenvalue order
  float* lam;      // n eigenvalues, ascending
  int n, lda, ldq;
  int transposed;     // 1: eigenvectors are written as the rows of q instead
  float shift_scale;  // s > 0: the kernel works on A + s ||A||_F I (same eigenvectors, every eigenvalue at least
                      // (s - 1) ||A||_F) and subtracts the shift from the eigenvalues at the end.  One-sided Jacobi
                      // orthogonalises the columns of A V; on a singular or indefinite matrix the columns that
                      // belong to eigenvalues near zero are rounding noise and never pass the relative test.
  int pad_;
};

constexpr int kJacobiMaxN = 128;

// jacobi_eigh: eigendecomposition of many small symmetric matrices (n <= 128), one CTA per
// matrix, entirely in shared memory: one-sided (Hestenes) Jacobi on the columns of A with a
// round-robin pair schedule (n/2 disjoint pairs per round, one warp per pair), V accumulated
// alongside; at convergence the columns of A V are lambda_j v_j.  Sweeps stop when no pair of a
// sweep exceeded the relative threshold, or after `max_sweeps`.  It replaces the per-matrix library
// eigensolver calls (torch.linalg.eigh -> syevd, reference matrix_functions.py:754) for the small
// factors, where launch and workspace overhead dominates; `sweeps` (one int per matrix) reports the
// number of sweeps used, max_sweeps + 1 meaning not converged.
void launch_jacobi_eigh(const JacobiDesc* descs, int count, int max_sweeps, float tol, int* sweeps,
                        cudaStream_t stream);

// One square matrix of a grouped pointwise pass over many matrices of different sizes.
struct MatOp {
  const float* src;  // d x d, row pitch ld_src
  float* dst_hi;     // d x d, row pitch ld_dst (tf32-rounded part, or the plain result when dst_lo is null)
  float* dst_lo;     // residual part, may be null
  float* err;        // one float per matrix (identity_error)
  int d, ld_src, ld_dst, pad_;
};

constexpr int kMatRowsPerChunk = 8;

// dst = a * src + b * I for every matrix of the table, written as a (hi, lo) tf32 pair: the
// M_p = (1 - alpha) I + alpha M step of the coupled Newton iteration (reference:
// distributed_shampoo/preconditioner/matrix_functions.py:423-428), fused with the operand split.
void launch_affine_identity_split(const MatOp* ops, const int2* chunks, int num_chunks, float a, float b,
                                  cudaStream_t stream);

// err = max |src - I| per matrix (err must be zeroed first): the convergence measure of the
// coupled iterations, kept on the device (reference: torch.dist(M, I, p=inf) read by the host every
// iteration, matrix_functions.py:423).
void launch_identity_error(const MatOp* ops, const int2* chunks, int num_chunks, cudaStream_t stream);

void launch_tf32_split(const float* src, long long src_pitch, float* hi, float* lo, long long dst_pitch, int rows,
                       int cols, cudaStream_t stream);

void launch_gpa_adamw(const GpaTensorDesc* table, const int2* chunks, int num_chunks, float lr, float beta1,
                      float beta2, float eps, float bias_correction1, float bias_correction2, float weight_decay,
                      bool wd_on_y, float avg_coeff, float train_interp_coeff, cudaStream_t stream);

void launch_gpa_lerp(const GpaTensorDesc* table, const int2* chunks, int num_chunks, float weight,
                     cudaStream_t stream);

}  // namespace ob200
