// Grouped "TN" GEMM on the 5th-generation tensor cores:  C_g = beta * C_g + alpha * A_g * B_g^T
// for a table of independent problems, where A_g is [M,K] and B_g is [N,K], both K-major fp32.
//
// Two accuracy modes.  kSplit == 1: each operand arrives as a (hi, lo) pair with
// hi = tf32_round(x), lo = x - hi, and every K step issues three tf32 products
// (hi*hi + hi*lo + lo*hi) into the same fp32 TMEM accumulator, which restores fp32-grade
// accuracy.  kSplit == 0: one tf32 product on the raw fp32 operands.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of 128 x 32 fp32 with 128-byte swizzle
//   warp 1      MMA issuer: tcgen05.mma 128x128x8 kind::tf32, accumulators in TMEM, two
//               accumulator buffers so the epilogue of one tile overlaps the next tile's MMAs
//   warps 2..5  epilogue: tcgen05.ld, transpose through shared memory, then coalesced global
//               access with the fused options below.
//
// Epilogue options per problem (flags):
//   kFlagPackedC    C is the row-major packed upper triangle of a symmetric N x N matrix; only
//                   entries with col >= row are touched (the tile list then holds only tiles
//                   on or above the diagonal)
//   kFlagSplitOut   additionally write the result as a (hi, lo) tf32 pair into d_hi/d_lo
//                   (row pitch ldd) so it can feed the next GEMM of a chain
//   kFlagSumSq      add the sum of squares of the results to *sumsq (Frobenius norm partials)
//   kFlagNoC        do not write C (only the split / sumsq outputs)
//   kFlagPeerPush   the result is also stored, in the communication dtype, into every rank's gather
//                   buffer over NVLink (fused all-gather of the search directions)
//   kFlagSquareAcc  the accumulator is squared before alpha/beta are applied: with C the running
//                   second moment V this is V <- beta2 V + w (Q_L^T G Q_R)^2 fused into the projection
//   kFlagMirror     the result is symmetric (products of commuting symmetric matrices, Grams): the
//                   tile list holds only tiles on or above the diagonal and every tile strictly
//                   above it is also stored transposed (C, d_hi, d_lo), so the full matrix is an
//                   operand of the next product at half the tensor-core work; sumsq counts such
//                   a tile twice
//   kFlagAddDiag    gamma (a launch scalar) is added to the diagonal entries: C = alpha A B^T +
//                   beta C + gamma I, the polynomial steps of the matrix sign iteration
//   kFlagTrace      add the diagonal entries of the result to sumsq[1] (trace)
#pragma once

#include <cstdint>
#include <cuda.h>

namespace ob200 {

constexpr int kFlagPackedC = 1;
constexpr int kFlagSplitOut = 2;
constexpr int kFlagSumSq = 4;
constexpr int kFlagNoC = 8;
constexpr int kFlagSquareAcc = 16;  // C = beta * C + alpha * acc^2 (second moment in the eigenbasis)
constexpr int kFlagMirror = 64;     // symmetric result: upper tiles computed, mirrored into the lower triangle
constexpr int kFlagAddDiag = 128;   // + gamma on the diagonal
constexpr int kFlagTrace = 256;     // sumsq[1] += trace of the result
constexpr int kFlagPeerPush = 32;   // also store the result, cast to the communication dtype, into the
                                    // problem's slot of every rank's gather buffer (PeerPush): the
                                    // all-gather of the search directions happens tile by tile from
                                    // the epilogue of the GEMM that produces them

constexpr int kErrPipelineTimeout = 1;  // a bounded mbarrier wait expired

struct alignas(128) GemmProblem {
  // 2-D tensor maps (dim0 = K, contiguous; dim1 = rows) of the arrays the operands are views of.
  // They live in device memory next to the problem table; several problems (the panels of a
  // blocked factorisation) may share one map and differ only in the view origin below.
  const CUtensorMap* a_hi;
  const CUtensorMap* a_lo;
  const CUtensorMap* b_hi;
  const CUtensorMap* b_lo;
  int a_row0, a_k0;  // origin of the A view inside its array (a_k0 a multiple of 4: TMA alignment)
  int b_row0, b_k0;  // a view that does not end where its array ends along K must have K % kBK == 0
  float* c;
  float* d_hi;
  float* d_lo;
  float* sumsq;
  int M, N, K;
  int ldc;  // row pitch of C in elements (full mode); N in packed mode
  int ldd;  // row pitch of d_hi / d_lo
  int flags;
  int pad_[2];
  long long push_offset;  // byte offset of the problem's slot inside the gather buffers (kFlagPeerPush)
};

// Destination of kFlagPeerPush stores: the gather buffer of every rank of the group (this rank
// included), all laid out identically.  Plain stores over NVLink; no TMA touches peer memory.
struct PeerPush {
  unsigned long long base[8];
  int num_peers;  // 0: no problem of the launch pushes
  int dtype;      // 0 fp32, 1 bf16, 2 fp16
};

struct GemmTile {
  int problem;
  int m0;  // first row of the tile
  int n0;  // first column of the tile
  int pad_;
};

constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kBK = 32;  // fp32 elements = 128 bytes = one swizzle row

// Host-side launch.  `status` is a device int the kernel writes a non-zero error code to.
void launch_grouped_gemm(const GemmProblem* problems, const GemmTile* tiles, int num_tiles, float alpha, float beta,
                         bool split, int* status, int max_ctas, cudaStream_t stream, const PeerPush* push = nullptr,
                         float gamma = 0.f);

}  // namespace ob200
