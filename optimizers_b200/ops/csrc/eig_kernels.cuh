// Kernels of the batched eigensolver and of the QR eigenbasis refresh that are not matrix products:
//
//   householder_panel   Householder factorisation of one panel (up to 16 columns) of every matrix
//                       of a batch, one CTA per matrix, the panel resident in shared memory; emits
//                       the compact-WY operands (V, T^T V^T, T V^T as tf32 (hi, lo) pairs) with
//                       which the grouped tensor-core GEMM applies the block reflector to the
//                       trailing columns and accumulates Q.  Replaces cuSOLVER geqrf / orgqr behind
//                       torch.linalg.qr (reference: distributed_shampoo/preconditioner/
//                       matrix_functions.py:843).
//   sym_measure         trace / n and ||A - (trace / n) I||_F of every matrix of a batch
//   shift_scale_split   X = a A + b I per matrix (a, b per matrix), written as a (hi, lo) pair
//   sq_offdiag          ||B||_F^2 and ||diag B||_F^2 per matrix: the convergence criterion of the QR
//                       iteration (matrix_functions.py:772-797) without a host round trip per factor
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace ob200 {

constexpr int kQrPanel = 16;            // columns per Householder panel
constexpr int kQrThreads = 512;
constexpr int kQrSmemFloats = 3072 * kQrPanel;  // panels up to this many floats live in shared memory

// One panel of one matrix.  The matrix is stored transposed: row c of `ct` (pitch ld) is column c
// of the matrix being factored, a vector of length n.  The panel covers columns c0 .. c1-1
// (c1 - c0 <= kQrPanel, c0 a multiple of kQrPanel); entries [0, c0) of its rows are finished R
// entries and are not touched.  On return rows c0..c1-1 hold R on and before the diagonal position
// and the reflector below it (LAPACK geqrf layout), and, for i in [c0, n):
//   v       [(i - c0) * kQrPanel + j]      = V[i, j]          (n - c0) x kQrPanel, zero padded
//   ttv     [j * ldw + (i - c0)]           = (T^T V^T)[j, i]  operand of the trailing update
//   tv      [j * ldw + (i - c0)]           = (T V^T)[j, i]    operand of the accumulation of Q
// (the caller points ttv_* / tv_* at the entry of panel row 0 and column c0 of a larger array)
// each as a tf32 (hi, lo) pair.  H_c0 ... H_{c1-1} = I - V T V^T with T upper triangular.
struct QrPanelDesc {
  float* ct;
  float* v_hi;
  float* v_lo;
  float* ttv_hi;
  float* ttv_lo;
  float* tv_hi;
  float* tv_lo;
  int ld, n, c0, c1;
  int ldw;  // row pitch of tt_v / t_v (>= n - c0, multiple of 4)
  int pad_[3];
};

void launch_householder_panel(const QrPanelDesc* descs, int count, cudaStream_t stream);

// One square matrix of a batched pass.
struct SymOp {
  const float* src;  // n x n, row pitch ld_src
  float* dst_hi;     // n x n, row pitch ld_dst
  float* dst_lo;     // may be null: dst_hi then receives the plain result
  float* stats;      // sym_measure: [trace / n, ||A - (trace / n) I||_F]; sq_offdiag: [||B||_F^2, ||diag B||_F^2]
  float a, b;        // shift_scale_split: dst = a * src + b * I
  int n, ld_src, ld_dst, pad_;
};

constexpr int kSymRowsPerChunk = 8;

// One CTA per matrix.
void launch_sym_measure(const SymOp* ops, int count, cudaStream_t stream);
void launch_sq_offdiag(const SymOp* ops, int count, cudaStream_t stream);
// Chunked over (matrix, 8-row band) pairs.
void launch_shift_scale_split(const SymOp* ops, const int2* chunks, int num_chunks, cudaStream_t stream);

// Transposed copy of a rows x cols matrix (pitch ld_src) into dst (cols x rows, pitch ld_dst),
// optionally also as a (hi, lo) pair.  One launch covers a table of matrices.
struct TransposeOp {
  const float* src;
  float* dst;     // plain transposed copy (may be null)
  float* dst_hi;  // may be null
  float* dst_lo;
  int rows, cols, ld_src, ld_dst;
};
void launch_transpose_split(const TransposeOp* ops, const int4* tiles, int num_tiles, cudaStream_t stream);

}  // namespace ob200
