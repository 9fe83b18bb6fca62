// Grouped TN GEMM kernel for sm_100a (tcgen05 + TMEM + TMA).  See grouped_gemm.cuh for the
// contract.  Replaces, as one launch over a problem table, the per-block cuBLAS calls behind
// torch.tensordot in the reference (distributed_shampoo/preconditioner/
// shampoo_preconditioner_list.py:1499-1507 factor Gram matrices, :1563-1578 preconditioner
// application) together with the packing / EMA / norm kernels around them (:1525-1539).
#include "grouped_gemm.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace ob200 {

namespace {

constexpr int kThreads = 192;
constexpr int kEpilogueWarps = 4;
constexpr int kTileBytesA = kBM * kBK * 4;  // 16 KiB
constexpr int kTileBytesB = kBN * kBK * 4;  // 16 KiB
constexpr int kStagePitch = 33;             // floats per staged row: conflict-free transposition
constexpr int kAccumCols = 2 * kBN;         // two accumulator buffers
constexpr uint32_t kIdesc = make_idesc(/*tf32*/ 2, kBM, kBN);

template <int kSplit>
struct Cfg {
  static constexpr int kStageBytes = (kTileBytesA + kTileBytesB) * (kSplit ? 2 : 1);
  static constexpr int kStages = kSplit ? 3 : 6;
  static constexpr int kStagingBytes = kEpilogueWarps * 32 * kStagePitch * 4;
  static constexpr int kBarrierBytes = 256;
  // 1024 B of slack so the stage buffers can be aligned for the 128-byte swizzle.
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kStagingBytes + kBarrierBytes;
};

// kPush: instantiation whose epilogue also stores into the peers' gather buffers; kept apart so
// that the store loop of the common instantiation is not burdened with it.
template <int kSplit, bool kPush>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const GemmProblem* __restrict__ problems, const GemmTile* __restrict__ tiles, int num_tiles,
                    float alpha, float beta, float gamma, int* __restrict__ status, const PeerPush push) {
  using C = Cfg<kSplit>;
  constexpr int kStages = C::kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  float* staging = reinterpret_cast<float*>(smem + kStages * C::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * C::kStageBytes + C::kStagingBytes);
  uint64_t* full_bar = bars;                 // [kStages]
  uint64_t* empty_bar = bars + kStages;      // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], kEpilogueWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kAccumCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const GemmTile tile = tiles[t];
        const GemmProblem* p = &problems[tile.problem];
        const int num_kb = (p->K + kBK - 1) / kBK;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* s = stage_base + stage * C::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], C::kStageBytes);
          const int ak = p->a_k0 + kb * kBK, bk = p->b_k0 + kb * kBK;
          const int ar = p->a_row0 + tile.m0, br = p->b_row0 + tile.n0;
          tma_load_2d(s, p->a_hi, &full_bar[stage], ak, ar);
          tma_load_2d(s + kTileBytesA, p->b_hi, &full_bar[stage], bk, br);
          if (kSplit) {
            tma_load_2d(s + kTileBytesA + kTileBytesB, p->a_lo, &full_bar[stage], ak, ar);
            tma_load_2d(s + 2 * kTileBytesA + kTileBytesB, p->b_lo, &full_bar[stage], bk, br);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const GemmTile tile = tiles[t];
        const int num_kb = (problems[tile.problem].K + kBK - 1) / kBK;
        const int buf = it & 1;
        if (!mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kBN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t s = smem_u32(stage_base + stage * C::kStageBytes);
          const uint64_t a_hi = make_kmajor_sw128_desc(s);
          const uint64_t b_hi = make_kmajor_sw128_desc(s + kTileBytesA);
          const uint64_t a_lo = make_kmajor_sw128_desc(s + kTileBytesA + kTileBytesB);
          const uint64_t b_lo = make_kmajor_sw128_desc(s + 2 * kTileBytesA + kTileBytesB);
#pragma unroll
          for (int k = 0; k < kBK / 8; ++k) {
            // Advancing the start address by 32 bytes (encoded >> 4) walks the K steps inside
            // the 128-byte swizzle row.
            const uint64_t koff = static_cast<uint64_t>(k * 2);
            if (kSplit) {
              // Consecutive products share one operand descriptor (b_hi, then a_hi).
              umma_tf32(d_tmem, a_lo + koff, b_hi + koff, kIdesc, (kb | k) != 0);
              umma_tf32(d_tmem, a_hi + koff, b_hi + koff, kIdesc, 1);
              umma_tf32(d_tmem, a_hi + koff, b_lo + koff, kIdesc, 1);
            } else {
              umma_tf32(d_tmem, a_hi + koff, b_hi + koff, kIdesc, (kb | k) != 0);
            }
          }
          umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    float* st = staging + (warp - 2) * 32 * kStagePitch;
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      const GemmTile tile = tiles[t];
      const GemmProblem* p = &problems[tile.problem];
      const int M = p->M, N = p->N, flags = p->flags;
      float* __restrict__ Cp = p->c;
      float* __restrict__ Dhi = p->d_hi;
      float* __restrict__ Dlo = p->d_lo;
      const int ldc = p->ldc, ldd = p->ldd;
      const bool do_push = kPush && (flags & kFlagPeerPush) && push.num_peers > 0;
      const long long push_offset = p->push_offset;
      const int buf = it & 1;
      if (!mbar_wait(&acc_full[buf], (it >> 1) & 1, abort_flag)) break;
      tc_fence_after_sync();
      const int row0 = tile.m0 + q * 32;
      float sq = 0.f, tr = 0.f;
      // Symmetric result (kFlagMirror): only entries on or above the diagonal are taken from the
      // accumulator; every 32 x 32 chunk strictly above the diagonal is also stored transposed and
      // the chunks on the diagonal are symmetrised, so the stored matrix is symmetric bit for bit
      // (an antisymmetric rounding residue would be amplified by the polynomial iterations that
      // consume these products).
      const bool sym = (flags & kFlagMirror) != 0;
      const bool diag_tile = sym && tile.n0 == tile.m0;
      if (row0 < M) {
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
          const int col0 = tile.n0 + c * 32;
          if (col0 >= N) break;
          if ((flags & kFlagPackedC) && col0 + 31 < row0) continue;  // chunk strictly below the diagonal
          if (diag_tile && c < q) continue;  // written as the transpose of chunk (c, q)
          const bool mirror = sym && (!diag_tile || c > q);
          const bool diag_chunk = diag_tile && c == q;
          float v[32];
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kBN + c * 32, v);
          float sq_chunk = 0.f;
          // Fast path: the thread that holds row (row0 + lane) of the accumulator stores its 32
          // consecutive columns itself with 16-byte accesses (C, then the (hi, lo) pair), and
          // stores the transposed copy of a symmetric result one column at a time, where the 32
          // lanes are 32 consecutive addresses.  No staging through shared memory.  It needs a full
          // chunk, 16-byte alignment of every row segment and none of the per-element layouts
          // (packed triangle, peer push, the symmetrised diagonal chunk).
          const bool fast_c = (flags & kFlagNoC) || ((ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(Cp) & 15) == 0);
          const bool fast_d = !(flags & kFlagSplitOut) ||
                              ((ldd & 3) == 0 && ((reinterpret_cast<uintptr_t>(Dhi) | reinterpret_cast<uintptr_t>(Dlo)) & 15) == 0);
          if (col0 + 32 <= N && !(flags & kFlagPackedC) && !do_push && !diag_chunk && fast_c && fast_d) {
            const int row = row0 + lane;
            if (row < M) {
              const bool write_c = !(flags & kFlagNoC);
              if (flags & kFlagSquareAcc) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] *= v[j];
              }
              if (write_c && beta != 0.f) {
                const float4* src = reinterpret_cast<const float4*>(Cp + static_cast<long long>(row) * ldc + col0);
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                  const float4 o = src[j4];
                  v[4 * j4 + 0] = alpha * v[4 * j4 + 0] + beta * o.x;
                  v[4 * j4 + 1] = alpha * v[4 * j4 + 1] + beta * o.y;
                  v[4 * j4 + 2] = alpha * v[4 * j4 + 2] + beta * o.z;
                  v[4 * j4 + 3] = alpha * v[4 * j4 + 3] + beta * o.w;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] *= alpha;
              }
              if (flags & (kFlagAddDiag | kFlagTrace)) {
                const int dj = row - col0;  // position of the diagonal entry in this segment, if any
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (j == dj) {
                    if (flags & kFlagAddDiag) v[j] += gamma;
                    if (flags & kFlagTrace) tr += v[j];
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < 32; ++j) sq_chunk = fmaf(v[j], v[j], sq_chunk);
              if (write_c) {
                float4* dst = reinterpret_cast<float4*>(Cp + static_cast<long long>(row) * ldc + col0);
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) dst[j4] = make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
              }
              if (flags & kFlagSplitOut) {
                float4* dh = reinterpret_cast<float4*>(Dhi + static_cast<long long>(row) * ldd + col0);
                float4* dl = reinterpret_cast<float4*>(Dlo + static_cast<long long>(row) * ldd + col0);
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                  float h[4], l[4];
#pragma unroll
                  for (int k = 0; k < 4; ++k) {
                    h[k] = tf32_round(v[4 * j4 + k]);
                    l[k] = v[4 * j4 + k] - h[k];
                  }
                  dh[j4] = make_float4(h[0], h[1], h[2], h[3]);
                  dl[j4] = make_float4(l[0], l[1], l[2], l[3]);
                }
              }
              if (mirror) {
                // (row, col0 + j) -> (col0 + j, row): for a fixed j the warp writes 32 consecutive floats
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const long long oc = static_cast<long long>(col0 + j) * ldc + row;
                  if (write_c) Cp[oc] = v[j];
                  if (flags & kFlagSplitOut) {
                    const long long od = static_cast<long long>(col0 + j) * ldd + row;
                    const float hi = tf32_round(v[j]);
                    Dhi[od] = hi;
                    Dlo[od] = v[j] - hi;
                  }
                }
                sq_chunk *= 2.f;
              }
            }
            sq += sq_chunk;
            continue;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) st[lane * kStagePitch + j] = v[j];
          __syncwarp();
          const int col = col0 + lane;
          if (col < N) {
            const int rows = min(32, M - row0);
            const bool packed = (flags & kFlagPackedC) != 0;
            const bool write_c = packed || !(flags & kFlagNoC);
            // All loads of the old values first, then the stores: the loads are independent
            // and overlap instead of each waiting behind the previous store.  Offsets advance
            // incrementally: one row down is +ldc, or +(N - row - 1) in the packed triangle.
            const long long off0 =
                packed ? static_cast<long long>(row0) * N - (static_cast<long long>(row0) * (row0 - 1)) / 2 + (col - row0)
                       : static_cast<long long>(row0) * ldc + col;
            float old[32];
            if (write_c && beta != 0.f) {
              long long o = off0;
#pragma unroll
              for (int rr = 0; rr < 32; ++rr) {
                const int row = row0 + rr;
                const bool live = rr < rows && (!packed || col >= row);
                old[rr] = live ? Cp[o] : 0.f;
                o += packed ? (N - row - 1) : ldc;
              }
            } else {
#pragma unroll
              for (int rr = 0; rr < 32; ++rr) old[rr] = 0.f;
            }
            long long o = off0;
#pragma unroll
            for (int rr = 0; rr < 32; ++rr) {
              const int row = row0 + rr;
              const bool live = rr < rows && (!packed || col >= row);
              if (live) {
                float acc = st[rr * kStagePitch + lane];
                if (flags & kFlagSquareAcc) acc *= acc;
                float val = alpha * acc + beta * old[rr];
                if ((flags & kFlagAddDiag) && row == col) val += gamma;
                if (sym) st[rr * kStagePitch + lane] = val;  // read back transposed below
                if (!diag_chunk) {
                  if ((flags & kFlagTrace) && row == col) tr += val;
                  if (write_c) Cp[o] = val;
                  if (flags & kFlagSplitOut) {
                    const long long od = static_cast<long long>(row) * ldd + col;
                    const float hi = tf32_round(val);
                    Dhi[od] = hi;
                    Dlo[od] = val - hi;
                  }
                  if (kPush && do_push) {
                    // A warp stores 32 consecutive elements of one row into each rank's slot.
                    const long long e = static_cast<long long>(row) * N + col;
                    for (int r = 0; r < push.num_peers; ++r) {
                      void* dst = reinterpret_cast<void*>(push.base[r] + push_offset);
                      if (push.dtype == 1) {
                        static_cast<__nv_bfloat16*>(dst)[e] = __float2bfloat16_rn(val);
                      } else if (push.dtype == 2) {
                        static_cast<__half*>(dst)[e] = __float2half_rn(val);
                      } else {
                        static_cast<float*>(dst)[e] = val;
                      }
                    }
                  }
                  sq_chunk += val * val;
                }
              }
              o += packed ? (N - row - 1) : ldc;
            }
          }
          __syncwarp();
          if (diag_chunk) {
            // Entry (row0 + rr, col0 + lane) takes the value computed for whichever of it and its
            // transpose lies on or above the diagonal.
            if (col < N) {
              const int rows = min(32, M - row0);
              const bool write_c = !(flags & kFlagNoC);
              for (int rr = 0; rr < rows; ++rr) {
                const float val = lane >= rr ? st[rr * kStagePitch + lane] : st[lane * kStagePitch + rr];
                const int row = row0 + rr;
                if ((flags & kFlagTrace) && rr == lane) tr += val;
                if (write_c) Cp[static_cast<long long>(row) * ldc + col] = val;
                if (flags & kFlagSplitOut) {
                  const long long od = static_cast<long long>(row) * ldd + col;
                  const float hi = tf32_round(val);
                  Dhi[od] = hi;
                  Dlo[od] = val - hi;
                }
                sq_chunk += val * val;
              }
            }
            __syncwarp();
          } else if (mirror) {
            // Element (row0 + lane, col0 + j) goes to (col0 + j, row0 + lane): lanes run along the
            // destination row, and the odd staging pitch keeps the column read conflict-free.
            const int rows = min(32, M - row0), cols = min(32, N - col0);
            if (lane < rows) {
              const bool write_c = !(flags & kFlagNoC);
              for (int j = 0; j < cols; ++j) {
                const float val = st[lane * kStagePitch + j];
                const int drow = col0 + j, dcol = row0 + lane;
                if (write_c) Cp[static_cast<long long>(drow) * ldc + dcol] = val;
                if (flags & kFlagSplitOut) {
                  const long long od = static_cast<long long>(drow) * ldd + dcol;
                  const float hi = tf32_round(val);
                  Dhi[od] = hi;
                  Dlo[od] = val - hi;
                }
              }
            }
            __syncwarp();
            sq_chunk *= 2.f;
          }
          sq += sq_chunk;
        }
      }
      tc_fence_before_sync();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      if (flags & kFlagSumSq) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0 && sq != 0.f) atomicAdd(p->sumsq, sq);
      }
      if (flags & kFlagTrace) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tr += __shfl_xor_sync(0xffffffffu, tr, o);
        if (lane == 0 && tr != 0.f) atomicAdd(p->sumsq + 1, tr);
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, kErrPipelineTimeout);
    // Give copies that are still in flight time to land before the CTA's shared memory goes away.
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kAccumCols);
  }
}

template <int kSplit, bool kPush>
void launch_impl(const GemmProblem* problems, const GemmTile* tiles, int num_tiles, float alpha, float beta,
                 float gamma, int* status, int max_ctas, cudaStream_t stream, const PeerPush& push) {
  using C = Cfg<kSplit>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(grouped_gemm_kernel<kSplit, kPush>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    configured = true;
  }
  const int grid = num_tiles < max_ctas ? num_tiles : max_ctas;
  grouped_gemm_kernel<kSplit, kPush><<<grid, kThreads, C::kSmemBytes, stream>>>(problems, tiles, num_tiles, alpha,
                                                                               beta, gamma, status, push);
}

}  // namespace

void launch_grouped_gemm(const GemmProblem* problems, const GemmTile* tiles, int num_tiles, float alpha, float beta,
                         bool split, int* status, int max_ctas, cudaStream_t stream, const PeerPush* push, float gamma) {
  if (num_tiles <= 0) return;
  PeerPush none{};
  const PeerPush& pp = push != nullptr ? *push : none;
  const bool pushing = pp.num_peers > 0;
  if (split) {
    if (pushing) launch_impl<1, true>(problems, tiles, num_tiles, alpha, beta, gamma, status, max_ctas, stream, pp);
    else launch_impl<1, false>(problems, tiles, num_tiles, alpha, beta, gamma, status, max_ctas, stream, pp);
  } else {
    if (pushing) launch_impl<0, true>(problems, tiles, num_tiles, alpha, beta, gamma, status, max_ctas, stream, pp);
    else launch_impl<0, false>(problems, tiles, num_tiles, alpha, beta, gamma, status, max_ctas, stream, pp);
  }
}

}  // namespace ob200
