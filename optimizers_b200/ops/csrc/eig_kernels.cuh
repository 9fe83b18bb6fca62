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
// and the reflector below it (LAPACK geqrf layout), and three kQrPanel x (n - c0) arrays of common
// row pitch ldw (rows beyond the panel's columns are zero) hold, for i in [c0, n):
//   vt  [j * ldw + (i - c0)] = V[i, j]            the reflectors
//   ttv [j * ldw + (i - c0)] = (T^T V^T)[j, i]    left factor of the trailing update
//   tv  [j * ldw + (i - c0)] = (T V^T)[j, i]      left factor of the accumulation of Q
// with H_c0 ... H_{c1-1} = I - V T V^T and T upper triangular.  (The caller points vt / ttv / tv at
// the entry of panel row 0 and column c0 of larger arrays.)
struct QrPanelDesc {
  float* ct;
  float* vt;
  float* ttv;
  float* tv;
  int ld, n, c0, c1;
  int ldw;
  int pad_[3];
};

void launch_householder_panel(const QrPanelDesc* descs, int count, cudaStream_t stream);

// Application of a block reflector to a block of rows:  X <- X - (X W^T) Vt  with X rows x L
// (pitch ldx), W and Vt kQrPanel x L (pitch ldw a multiple of 4, 16-byte aligned rows, and at least
// kReflectChunk columns of addressable slack after column L of every row: chunks are copied whole).  In the transposed storage of the QR this is
// C <- (I - V T V^T)^T C on trailing columns (W = T^T V^T) and Z <- Z (I - V T^T V^T) on the
// accumulated Q^T (W = T V^T).  A rank-16 update moves 8 bytes per element for 64 flops: it is
// bound by HBM, so it runs on the CUDA cores in exact fp32, each CTA holding a tile of whole rows in
// shared memory between the two passes (inner products, update); x_hi / x_lo, when given, also
// receive the tf32 (hi, lo) pair of the updated block (same pitch).
struct ReflectDesc {
  float* x;
  float* x_hi;  // may be null
  float* x_lo;
  const float* w;
  const float* vt;
  int ldx, ldw, rows, L;
  int rows_per_tile;  // whole rows held by one CTA: at most kReflectMaxRows, rows_per_tile * L <= kReflectSmemFloats
  int pad_[3];
};

constexpr int kReflectMaxRows = 8;
constexpr int kReflectSmemFloats = 16384;  // row tile: 64 KB, two CTAs per SM
constexpr int kReflectChunk = 256;         // columns of W / Vt staged per step

void launch_apply_block_reflector(const ReflectDesc* descs, const int2* tiles, int num_tiles, cudaStream_t stream);

// Q^T of a factored matrix (all of its panels) in one pass over its rows; see accumulate_q_kernel.
// vt / tv are the [npan * kQrPanel, ldw] arrays the panel kernel filled (row 16 j + m = reflector m of
// panel j, indexed by absolute column), zt / zt_hi / zt_lo the n x n outputs of pitch ldz.
struct AccumulateDesc {
  float* zt;
  float* zt_hi;
  float* zt_lo;
  const float* vt;
  const float* tv;
  int ldz, ldw, n, npan;
  int rows_per_tile;
  int q_rows;  // only rows [0, q_rows) of Q^T are produced (the first q_rows columns of Q)
  int pad_[2];
};

void launch_accumulate_q(const AccumulateDesc* descs, const int2* tiles, int num_tiles, cudaStream_t stream);

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

// dst = the symmetric d x d matrix held in `src`, either as its row-major packed upper triangle
// (packed = 1; the checkpoint layout of the factor and inverse-root state) or in full (pitch ld_src),
// written as a tf32 (hi, lo) pair, or plain into dst_hi when dst_lo is null.  One launch rebuilds
// the GEMM operand mirrors of every factor of a parameter group from the state, instead of an
// index_put and two copies per factor.
struct UnpackOp {
  const float* src;
  float* dst_hi;
  float* dst_lo;
  int d, ld_src, ld_dst, packed;
};
void launch_unpack_split(const UnpackOp* ops, const int2* chunks, int num_chunks, cudaStream_t stream);
// The reverse for the checkpoint state: dst_hi (packed = 1: the packed upper triangle, else a full
// d x d array of pitch ld_dst) = the d x d matrix at src (pitch ld_src); dst_lo is not used.
void launch_pack_upper(const UnpackOp* ops, const int2* chunks, int num_chunks, cudaStream_t stream);

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
