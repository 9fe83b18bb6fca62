// See eig_kernels.cuh.
#include "eig_kernels.cuh"
#include "ptx.cuh"

namespace ob200 {

namespace {

constexpr int kQrWarps = kQrThreads / 32;

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__device__ __forceinline__ void store_split(float* __restrict__ hi, float* __restrict__ lo, long long o, float x) {
  const float h = tf32_round(x);
  hi[o] = h;
  lo[o] = x - h;
}

// Householder QR of one panel.  P[j * pitch + i] is entry i (counted from row c0) of panel column
// j; it lives in shared memory when the panel fits there and is worked on in place in global
// memory otherwise (the same code runs on a generic pointer).
//
// Column step j needs, for every other panel column j', the inner product of the part of column j
// below the pivot with the same part of column j' (one block-wide reduction of up to 16 values):
//   j' = j   sum of squares -> the reflector's beta, tau and scaling
//   j' > j   w_j' = P[j'][j] + scale * dot: the coefficient of the update of a column still to factor
//   j' < j   z_j' = the same expression on a stored reflector: (V^T v_j)[j'], the input of T's column j
__global__ void __launch_bounds__(kQrThreads, 1) householder_panel_kernel(const QrPanelDesc* __restrict__ descs) {
  extern __shared__ float qsm[];
  __shared__ float red[kQrWarps][kQrPanel];
  __shared__ float wsh[kQrPanel];
  __shared__ float scal[4];
  __shared__ float taus[kQrPanel];
  __shared__ float zmat[kQrPanel][kQrPanel];  // zmat[j][m] = (V^T v_j)[m], m < j
  __shared__ float tmat[kQrPanel][kQrPanel];  // T, upper triangular

  const QrPanelDesc d = descs[blockIdx.x];
  const int nb = d.c1 - d.c0;
  const int L = d.n - d.c0;
  if (nb <= 0 || L <= 0) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool in_smem = static_cast<long long>(L) * kQrPanel <= kQrSmemFloats;
  float* gpanel = d.ct + static_cast<long long>(d.c0) * d.ld + d.c0;
  float* P = in_smem ? qsm : gpanel;
  const long long pitch = in_smem ? L : d.ld;

  if (in_smem) {
    for (int j = 0; j < nb; ++j)
      for (int i = tid; i < L; i += kQrThreads) P[j * pitch + i] = gpanel[static_cast<long long>(j) * d.ld + i];
  }
  for (int e = tid; e < kQrPanel * kQrPanel; e += kQrThreads) {
    zmat[e / kQrPanel][e % kQrPanel] = 0.f;
    tmat[e / kQrPanel][e % kQrPanel] = 0.f;
  }
  __syncthreads();

  for (int j = 0; j < nb; ++j) {
    float acc[kQrPanel];
#pragma unroll
    for (int jj = 0; jj < kQrPanel; ++jj) acc[jj] = 0.f;
    for (int i = tid; i < L; i += kQrThreads) {
      if (i > j) {
        const float x = P[j * pitch + i];
#pragma unroll
        for (int jj = 0; jj < kQrPanel; ++jj)
          if (jj < nb) acc[jj] = fmaf(x, P[jj * pitch + i], acc[jj]);
      }
    }
#pragma unroll
    for (int jj = 0; jj < kQrPanel; ++jj) {
      const float s = warp_sum(acc[jj]);
      if (lane == 0) red[warp][jj] = s;
    }
    __syncthreads();
    if (warp == 0) {
      float t = 0.f;
      if (lane < kQrPanel)
        for (int w = 0; w < kQrWarps; ++w) t += red[w][lane];
      const float ssq = __shfl_sync(0xffffffffu, t, j);
      const float alpha = P[j * pitch + j];
      float beta = alpha, tau = 0.f, scale = 0.f;
      if (ssq > 0.f) {
        beta = -copysignf(sqrtf(alpha * alpha + ssq), alpha);
        tau = (beta - alpha) / beta;
        scale = 1.f / (alpha - beta);
      }
      float wv = 0.f;
      if (lane < nb && lane != j) wv = P[lane * pitch + j] + scale * t;
      if (lane < kQrPanel) wsh[lane] = wv;
      if (lane < j) zmat[j][lane] = wv;
      if (lane == 0) {
        scal[0] = tau;
        scal[1] = scale;
        scal[2] = beta;
        taus[j] = tau;
      }
    }
    __syncthreads();
    const float tau = scal[0], scale = scal[1], beta = scal[2];
    for (int i = tid; i < L; i += kQrThreads) {
      if (i > j) {
        const float vi = P[j * pitch + i] * scale;
        for (int jj = j + 1; jj < nb; ++jj) P[jj * pitch + i] -= tau * wsh[jj] * vi;
        P[j * pitch + i] = vi;
      } else if (i == j) {
        for (int jj = j + 1; jj < nb; ++jj) P[jj * pitch + j] -= tau * wsh[jj];
        P[j * pitch + j] = beta;
      }
    }
    // The next step's reads of other threads' entries (pivot entries, by warp 0) come after its
    // first barrier, which every writer of this step has then passed.
  }
  __syncthreads();

  // T: T[j][j] = tau_j, T[0:j, j] = -tau_j T[0:j, 0:j] z_j (one warp, lane = row).
  if (warp == 0) {
    for (int j = 0; j < nb; ++j) {
      if (lane < j) {
        float s = 0.f;
        for (int m = lane; m < j; ++m) s = fmaf(tmat[lane][m], zmat[j][m], s);
        tmat[lane][j] = -taus[j] * s;
      } else if (lane == j) {
        tmat[j][j] = taus[j];
      }
      __syncwarp();
    }
  }
  __syncthreads();

  for (int i = tid; i < L; i += kQrThreads) {
    float v[kQrPanel];
#pragma unroll
    for (int jj = 0; jj < kQrPanel; ++jj) {
      float x = 0.f;
      if (jj < nb) x = (i == jj) ? 1.f : (i > jj ? P[jj * pitch + i] : 0.f);
      v[jj] = x;
    }
#pragma unroll
    for (int jj = 0; jj < kQrPanel; ++jj) {
      float ttv = 0.f, tv = 0.f;
      if (jj < nb) {
#pragma unroll
        for (int m = 0; m < kQrPanel; ++m) {
          if (m <= jj) ttv = fmaf(tmat[m][jj], v[m], ttv);
          if (m >= jj) tv = fmaf(tmat[jj][m], v[m], tv);
        }
      }
      const long long o = static_cast<long long>(jj) * d.ldw + i;  // all kQrPanel rows are written
      d.vt[o] = v[jj];
      d.ttv[o] = ttv;
      d.tv[o] = tv;
    }
  }
  if (in_smem) {
    for (int j = 0; j < nb; ++j)
      for (int i = tid; i < L; i += kQrThreads) gpanel[static_cast<long long>(j) * d.ld + i] = P[j * pitch + i];
  }
}

constexpr int kReflectThreads = 256;
constexpr int kReflectGroupRows = 4;                                   // rows whose sums one thread keeps in registers
constexpr int kReflectGroups = kReflectMaxRows / kReflectGroupRows;    // row groups of a tile
constexpr int kReflectGroupThreads = kReflectThreads / kReflectGroups;
constexpr int kReflectGroupWarps = kReflectGroupThreads / 32;
static_assert(kReflectChunk % kReflectGroupThreads == 0, "every thread of a group owns whole columns of a chunk");

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

// Stage columns [c0, c0 + kReflectChunk) of the kQrPanel rows of `src` (pitch ldw) into `dst`.  The
// arrays are allocated with kReflectChunk columns of slack per row, so a chunk never leaves its
// row's storage; entries beyond L are garbage that no thread uses.
__device__ __forceinline__ void stage_chunk(float* dst, const float* __restrict__ src, int ldw, int c0) {
  constexpr int kVecs = kReflectChunk / 4;
  for (int e = threadIdx.x; e < kQrPanel * kVecs; e += blockDim.x) {
    const int j = e / kVecs, i4 = e % kVecs;
    cp_async16(dst + j * kReflectChunk + 4 * i4, src + static_cast<long long>(j) * ldw + c0 + 4 * i4);
  }
  cp_async_commit();
}

// One block reflector applied to a tile of rows resident in shared memory:
//   xs[r][i] -= sum_j (sum_i' xs[r][i'] W[j][i']) Vt[j][i],   r < R, i < L  (xs row pitch `pitch`).
// The threads are split into row groups of four rows; a thread owns columns i = t, t + 128, ... of
// its group, keeps the 16 entries W[:, i] (then Vt[:, i]) in registers and runs them against its
// four rows, so a shared-memory load feeds 16 multiply-adds instead of one.  The chunks of W and Vt
// are double buffered with cp.async: the next chunk travels while the current one is consumed.
// Chunk 0 of W must already have been staged into ws (and committed) by the caller, so that its
// latency overlaps whatever the caller does before (loading the rows).  Ends with a barrier.
struct ReflectScratch {
  float part[kReflectGroups][kReflectGroupWarps][kReflectGroupRows * kQrPanel];
  float us[kReflectGroups][kReflectGroupRows * kQrPanel];
};

__device__ __forceinline__ void reflect_tile(float* ws, float* xs, int pitch, int R, int L, const float* __restrict__ w,
                                             const float* __restrict__ vt, int ldw, ReflectScratch& sc) {
  constexpr int kBuf = kQrPanel * kReflectChunk;
  const int lane = threadIdx.x & 31;
  const int g = threadIdx.x / kReflectGroupThreads, t = threadIdx.x % kReflectGroupThreads;
  const int gw = t >> 5;  // warp inside the group
  const int num_chunks = (L + kReflectChunk - 1) / kReflectChunk;
  const int rbase = g * kReflectGroupRows;  // first row of this thread's group inside the tile
  // ---- pass 1: u[r][j] = sum_i X[r][i] W[j][i]
  float acc[kReflectGroupRows][kQrPanel];
#pragma unroll
  for (int q = 0; q < kReflectGroupRows; ++q)
#pragma unroll
    for (int j = 0; j < kQrPanel; ++j) acc[q][j] = 0.f;
  for (int c = 0; c < num_chunks; ++c) {
    const int c0 = c * kReflectChunk;
    const int cw = min(kReflectChunk, L - c0);
    const float* wb = ws + (c & 1) * kBuf;
    // next chunk of W, or the first chunk of Vt for the second pass
    if (c + 1 < num_chunks) stage_chunk(ws + ((c + 1) & 1) * kBuf, w, ldw, c0 + kReflectChunk);
    else stage_chunk(ws + ((c + 1) & 1) * kBuf, vt, ldw, 0);
    cp_async_wait<1>();
    __syncthreads();  // chunk c (and, at c = 0, the rows) visible to all threads
    if (rbase < R) {
      for (int i = t; i < cw; i += kReflectGroupThreads) {
        float wv[kQrPanel];
#pragma unroll
        for (int j = 0; j < kQrPanel; ++j) wv[j] = wb[j * kReflectChunk + i];
#pragma unroll
        for (int q = 0; q < kReflectGroupRows; ++q) {
          const float x = rbase + q < R ? xs[(rbase + q) * pitch + c0 + i] : 0.f;
#pragma unroll
          for (int j = 0; j < kQrPanel; ++j) acc[q][j] = fmaf(x, wv[j], acc[q][j]);
        }
      }
    }
    __syncthreads();  // buffer (c & 1) may be refilled by the next iteration's prefetch
  }
  // sums over the threads of the group: inside each warp, then across the group's warps
#pragma unroll
  for (int q = 0; q < kReflectGroupRows; ++q)
#pragma unroll
    for (int j = 0; j < kQrPanel; ++j) {
      const float sum = warp_sum(acc[q][j]);
      if (lane == 0) sc.part[g][gw][q * kQrPanel + j] = sum;
    }
  __syncthreads();
  if (t < kReflectGroupRows * kQrPanel) {
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < kReflectGroupWarps; ++k) sum += sc.part[g][k][t];
    sc.us[g][t] = sum;
  }
  __syncthreads();
  float u[kReflectGroupRows][kQrPanel];
#pragma unroll
  for (int q = 0; q < kReflectGroupRows; ++q)
#pragma unroll
    for (int j = 0; j < kQrPanel; ++j) u[q][j] = sc.us[g][q * kQrPanel + j];
  // ---- pass 2: X[r][i] -= sum_j u[r][j] Vt[j][i]; chunk c of Vt sits in buffer (num_chunks + c) & 1
  for (int c = 0; c < num_chunks; ++c) {
    const int c0 = c * kReflectChunk;
    const int cw = min(kReflectChunk, L - c0);
    const float* vb = ws + ((num_chunks + c) & 1) * kBuf;
    if (c + 1 < num_chunks) {
      stage_chunk(ws + ((num_chunks + c + 1) & 1) * kBuf, vt, ldw, c0 + kReflectChunk);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (rbase < R) {
      for (int i = t; i < cw; i += kReflectGroupThreads) {
        float v[kQrPanel];
#pragma unroll
        for (int j = 0; j < kQrPanel; ++j) v[j] = vb[j * kReflectChunk + i];
#pragma unroll
        for (int q = 0; q < kReflectGroupRows; ++q) {
          if (rbase + q < R) {
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < kQrPanel; ++j) sum = fmaf(u[q][j], v[j], sum);
            xs[(rbase + q) * pitch + c0 + i] -= sum;
          }
        }
      }
    }
    __syncthreads();
  }
}

// Rows of a resident tile back to global memory, optionally also as the tf32 (hi, lo) pair.
__device__ __forceinline__ void store_tile(const float* xs, int R, int L, float* xg, float* hg, float* lg, int ldx) {
  const bool split = hg != nullptr;
  const bool vec = (L & 3) == 0 && (ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(xg) & 15) == 0 &&
                   (!split || (((reinterpret_cast<uintptr_t>(hg) | reinterpret_cast<uintptr_t>(lg)) & 15) == 0));
  if (vec) {
    const int L4 = L >> 2;
    for (int e = threadIdx.x; e < R * L4; e += kReflectThreads) {
      const int r = e / L4, i4 = e % L4;
      const float4 x = reinterpret_cast<const float4*>(xs + r * L)[i4];
      reinterpret_cast<float4*>(xg + static_cast<long long>(r) * ldx)[i4] = x;
      if (split) {
        float4 h, l;
        h.x = tf32_round(x.x); h.y = tf32_round(x.y); h.z = tf32_round(x.z); h.w = tf32_round(x.w);
        l.x = x.x - h.x; l.y = x.y - h.y; l.z = x.z - h.z; l.w = x.w - h.w;
        reinterpret_cast<float4*>(hg + static_cast<long long>(r) * ldx)[i4] = h;
        reinterpret_cast<float4*>(lg + static_cast<long long>(r) * ldx)[i4] = l;
      }
    }
  } else {
    for (int e = threadIdx.x; e < R * L; e += kReflectThreads) {
      const int r = e / L, i = e % L;
      const float x = xs[r * L + i];
      const long long o = static_cast<long long>(r) * ldx + i;
      xg[o] = x;
      if (split) store_split(hg, lg, o, x);
    }
  }
}

// A tile of up to kReflectMaxRows whole rows stays in shared memory between the two passes.
__global__ void __launch_bounds__(kReflectThreads, 2) apply_block_reflector_kernel(const ReflectDesc* __restrict__ descs,
                                                                                  const int2* __restrict__ tiles,
                                                                                  int num_tiles) {
  extern __shared__ float rsm[];
  float* ws = rsm;                                 // [2][kQrPanel][kReflectChunk] chunks of W, then of Vt
  float* xs = rsm + 2 * kQrPanel * kReflectChunk;  // [rows_per_tile][L]
  __shared__ ReflectScratch sc;
  for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
    const int2 ref = tiles[tile];
    const ReflectDesc d = descs[ref.x];
    const int row0 = ref.y;
    const int R = min(d.rows_per_tile, d.rows - row0);
    const int L = d.L;
    float* xg = d.x + static_cast<long long>(row0) * d.ldx;
    stage_chunk(ws, d.w, d.ldw, 0);
    const bool vec = (L & 3) == 0 && (d.ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(xg) & 15) == 0;
    if (vec) {
      const int L4 = L >> 2;
      for (int e = threadIdx.x; e < R * L4; e += kReflectThreads) {
        const int r = e / L4, i4 = e % L4;
        reinterpret_cast<float4*>(xs + r * L)[i4] = reinterpret_cast<const float4*>(xg + static_cast<long long>(r) * d.ldx)[i4];
      }
    } else {
      for (int e = threadIdx.x; e < R * L; e += kReflectThreads) {
        const int r = e / L, i = e % L;
        xs[r * L + i] = xg[static_cast<long long>(r) * d.ldx + i];
      }
    }
    reflect_tile(ws, xs, L, R, L, d.w, d.vt, d.ldw, sc);
    const bool split = d.x_hi != nullptr;
    store_tile(xs, R, L, xg, split ? d.x_hi + static_cast<long long>(row0) * d.ldx : nullptr,
               split ? d.x_lo + static_cast<long long>(row0) * d.ldx : nullptr, d.ldx);
    __syncthreads();  // xs is reused by the next tile
  }
}

// Accumulation of Q^T in one launch: Z = I (I - V_last T_last^T V_last^T) ... (I - V_0 T_0^T V_0^T).
// Every row of Z is transformed independently of the others, so a CTA keeps a tile of rows in
// shared memory, starts it as rows of the identity and applies every panel's reflector in turn
// (last panel first); Z is never read and written once, and the panels' W / Vt operands are shared
// by all tiles of a matrix through the L2.  Panel j only acts on columns >= 16 j, and rows above
// 16 j are still rows of the identity there, so a tile starts at the last panel that reaches it.
__global__ void __launch_bounds__(kReflectThreads, 2) accumulate_q_kernel(const AccumulateDesc* __restrict__ descs,
                                                                         const int2* __restrict__ tiles, int num_tiles) {
  extern __shared__ float rsm[];
  float* ws = rsm;
  float* xs = rsm + 2 * kQrPanel * kReflectChunk;  // [rows_per_tile][n]
  __shared__ ReflectScratch sc;
  for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
    const int2 ref = tiles[tile];
    const AccumulateDesc d = descs[ref.x];
    const int row0 = ref.y, n = d.n;
    const int R = min(d.rows_per_tile, d.q_rows - row0);
    const int first = min(d.npan - 1, (row0 + R - 1) / kQrPanel);  // last panel whose columns reach the tile's rows
    {
      const long long off = static_cast<long long>(first) * kQrPanel * d.ldw + first * kQrPanel;
      stage_chunk(ws, d.tv + off, d.ldw, 0);
    }
    for (int e = threadIdx.x; e < R * n; e += kReflectThreads) {
      const int r = e / n, i = e % n;
      xs[e] = (i == row0 + r) ? 1.f : 0.f;
    }
    for (int j = first; j >= 0; --j) {
      const int c0 = j * kQrPanel;
      const long long off = static_cast<long long>(c0) * d.ldw + c0;  // panel row 0, column c0
      reflect_tile(ws, xs + c0, n, R, n - c0, d.tv + off, d.vt + off, d.ldw, sc);
      if (j > 0) {
        const long long next = static_cast<long long>(c0 - kQrPanel) * d.ldw + (c0 - kQrPanel);
        stage_chunk(ws, d.tv + next, d.ldw, 0);  // reflect_tile left both chunk buffers free
      }
    }
    float* zg = d.zt + static_cast<long long>(row0) * d.ldz;
    store_tile(xs, R, n, zg, d.zt_hi + static_cast<long long>(row0) * d.ldz, d.zt_lo + static_cast<long long>(row0) * d.ldz, d.ldz);
    __syncthreads();
  }
}

constexpr int kSymThreads = 512;

__device__ __forceinline__ float block_sum(float x, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  x = warp_sum(x);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  float t = 0.f;
  const int warps = blockDim.x >> 5;
  for (int w = 0; w < warps; ++w) t += scratch[w];
  return t;
}

__global__ void __launch_bounds__(kSymThreads) sym_measure_kernel(const SymOp* __restrict__ ops) {
  __shared__ float scratch[kSymThreads / 32];
  const SymOp op = ops[blockIdx.x];
  const int n = op.n;
  float tr = 0.f;
  for (int i = threadIdx.x; i < n; i += kSymThreads) tr += op.src[static_cast<long long>(i) * op.ld_src + i];
  const float sigma = block_sum(tr, scratch) / static_cast<float>(n);
  float ss = 0.f;
  for (int i = threadIdx.x / 32; i < n; i += kSymThreads / 32) {
    const float* row = op.src + static_cast<long long>(i) * op.ld_src;
    float part = 0.f;
    for (int j = threadIdx.x & 31; j < n; j += 32) {
      const float x = row[j] - (i == j ? sigma : 0.f);
      part = fmaf(x, x, part);
    }
    ss += part;
  }
  const float total = block_sum(ss, scratch);
  if (threadIdx.x == 0) {
    op.stats[0] = sigma;
    op.stats[1] = sqrtf(total);
  }
}

__global__ void __launch_bounds__(kSymThreads) sq_offdiag_kernel(const SymOp* __restrict__ ops) {
  __shared__ float scratch[kSymThreads / 32];
  const SymOp op = ops[blockIdx.x];
  const int n = op.n;
  float all = 0.f, diag = 0.f;
  for (int i = threadIdx.x / 32; i < n; i += kSymThreads / 32) {
    const float* row = op.src + static_cast<long long>(i) * op.ld_src;
    float part = 0.f;
    for (int j = threadIdx.x & 31; j < n; j += 32) {
      const float x = row[j];
      part = fmaf(x, x, part);
      if (i == j) diag = fmaf(x, x, diag);
    }
    all += part;
  }
  const float a = block_sum(all, scratch);
  const float dg = block_sum(diag, scratch);
  if (threadIdx.x == 0) {
    op.stats[0] = a;
    op.stats[1] = dg;
  }
}

__global__ void __launch_bounds__(256) shift_scale_split_kernel(const SymOp* __restrict__ ops,
                                                                const int2* __restrict__ chunks, int num_chunks) {
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ref = chunks[c];
    const SymOp op = ops[ref.x];
    const int row0 = ref.y * kSymRowsPerChunk;
    const int rows = min(kSymRowsPerChunk, op.n - row0);
    for (int e = threadIdx.x; e < rows * op.n; e += blockDim.x) {
      const int i = row0 + e / op.n, j = e % op.n;
      float x = op.a != 0.f ? op.a * op.src[static_cast<long long>(i) * op.ld_src + j] : 0.f;  // a == 0: src is not read
      if (i == j) x += op.b;
      const long long o = static_cast<long long>(i) * op.ld_dst + j;
      if (op.dst_lo != nullptr) {
        store_split(op.dst_hi, op.dst_lo, o, x);
      } else {
        op.dst_hi[o] = x;
      }
    }
  }
}

__global__ void __launch_bounds__(256) unpack_split_kernel(const UnpackOp* __restrict__ ops, const int2* __restrict__ chunks,
                                                           int num_chunks) {
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ref = chunks[c];
    const UnpackOp op = ops[ref.x];
    const int row0 = ref.y * kSymRowsPerChunk;
    const int rows = min(kSymRowsPerChunk, op.d - row0);
    for (int e = threadIdx.x; e < rows * op.d; e += blockDim.x) {
      const int i = row0 + e / op.d, j = e % op.d;
      float x;
      if (op.packed) {
        const long long a = i < j ? i : j, b = i < j ? j : i;  // (a, b) with a <= b lies in the stored triangle
        x = op.src[a * op.d - a * (a - 1) / 2 + (b - a)];
      } else {
        x = op.src[static_cast<long long>(i) * op.ld_src + j];
      }
      const long long o = static_cast<long long>(i) * op.ld_dst + j;
      if (op.dst_lo != nullptr) {
        store_split(op.dst_hi, op.dst_lo, o, x);
      } else {
        op.dst_hi[o] = x;
      }
    }
  }
}

__global__ void __launch_bounds__(256) pack_upper_kernel(const UnpackOp* __restrict__ ops, const int2* __restrict__ chunks,
                                                         int num_chunks) {
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ref = chunks[c];
    const UnpackOp op = ops[ref.x];
    const int row0 = ref.y * kSymRowsPerChunk;
    const int rows = min(kSymRowsPerChunk, op.d - row0);
    for (int e = threadIdx.x; e < rows * op.d; e += blockDim.x) {
      const int i = row0 + e / op.d, j = e % op.d;
      const float x = op.src[static_cast<long long>(i) * op.ld_src + j];
      if (op.packed) {
        if (j >= i) op.dst_hi[static_cast<long long>(i) * op.d - static_cast<long long>(i) * (i - 1) / 2 + (j - i)] = x;
      } else {
        op.dst_hi[static_cast<long long>(i) * op.ld_dst + j] = x;
      }
    }
  }
}

__global__ void __launch_bounds__(256) transpose_split_kernel(const TransposeOp* __restrict__ ops,
                                                              const int4* __restrict__ tiles, int num_tiles) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const int4 ref = tiles[t];
    const TransposeOp op = ops[ref.x];
    const int r0 = ref.y * 32, c0 = ref.z * 32;
    for (int k = ty; k < 32; k += 8) {
      const int r = r0 + k, c = c0 + tx;
      tile[k][tx] = (r < op.rows && c < op.cols) ? op.src[static_cast<long long>(r) * op.ld_src + c] : 0.f;
    }
    __syncthreads();
    for (int k = ty; k < 32; k += 8) {
      const int c = c0 + k, r = r0 + tx;  // destination row c, destination column r
      if (c < op.cols && r < op.rows) {
        const float x = tile[tx][k];
        const long long o = static_cast<long long>(c) * op.ld_dst + r;
        if (op.dst != nullptr) op.dst[o] = x;
        if (op.dst_hi != nullptr) store_split(op.dst_hi, op.dst_lo, o, x);
      }
    }
    __syncthreads();
  }
}

}  // namespace

void launch_householder_panel(const QrPanelDesc* descs, int count, cudaStream_t stream) {
  if (count <= 0) return;
  static bool configured = false;
  constexpr int kBytes = kQrSmemFloats * 4;
  if (!configured) {
    cudaFuncSetAttribute(householder_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
    configured = true;
  }
  householder_panel_kernel<<<count, kQrThreads, kBytes, stream>>>(descs);
}

void launch_apply_block_reflector(const ReflectDesc* descs, const int2* tiles, int num_tiles, cudaStream_t stream) {
  if (num_tiles <= 0) return;
  static bool configured = false;
  constexpr int kBytes = (2 * kQrPanel * kReflectChunk + kReflectSmemFloats) * 4;
  if (!configured) {
    cudaFuncSetAttribute(apply_block_reflector_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
    configured = true;
  }
  const int cap = 2 * sm_count();  // two CTAs per SM: one loads or stores its rows while the other computes
  apply_block_reflector_kernel<<<num_tiles < cap ? num_tiles : cap, kReflectThreads, kBytes, stream>>>(descs, tiles, num_tiles);
}

void launch_accumulate_q(const AccumulateDesc* descs, const int2* tiles, int num_tiles, cudaStream_t stream) {
  if (num_tiles <= 0) return;
  static bool configured = false;
  constexpr int kBytes = (2 * kQrPanel * kReflectChunk + kReflectSmemFloats) * 4;
  if (!configured) {
    cudaFuncSetAttribute(accumulate_q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
    configured = true;
  }
  const int cap = 2 * sm_count();
  accumulate_q_kernel<<<num_tiles < cap ? num_tiles : cap, kReflectThreads, kBytes, stream>>>(descs, tiles, num_tiles);
}

void launch_sym_measure(const SymOp* ops, int count, cudaStream_t stream) {
  if (count <= 0) return;
  sym_measure_kernel<<<count, kSymThreads, 0, stream>>>(ops);
}

void launch_sq_offdiag(const SymOp* ops, int count, cudaStream_t stream) {
  if (count <= 0) return;
  sq_offdiag_kernel<<<count, kSymThreads, 0, stream>>>(ops);
}

void launch_shift_scale_split(const SymOp* ops, const int2* chunks, int num_chunks, cudaStream_t stream) {
  if (num_chunks <= 0) return;
  const int cap = sm_count() * 8;
  shift_scale_split_kernel<<<num_chunks < cap ? num_chunks : cap, 256, 0, stream>>>(ops, chunks, num_chunks);
}

void launch_unpack_split(const UnpackOp* ops, const int2* chunks, int num_chunks, cudaStream_t stream) {
  if (num_chunks <= 0) return;
  const int cap = sm_count() * 8;
  unpack_split_kernel<<<num_chunks < cap ? num_chunks : cap, 256, 0, stream>>>(ops, chunks, num_chunks);
}

void launch_pack_upper(const UnpackOp* ops, const int2* chunks, int num_chunks, cudaStream_t stream) {
  if (num_chunks <= 0) return;
  const int cap = sm_count() * 8;
  pack_upper_kernel<<<num_chunks < cap ? num_chunks : cap, 256, 0, stream>>>(ops, chunks, num_chunks);
}

void launch_transpose_split(const TransposeOp* ops, const int4* tiles, int num_tiles, cudaStream_t stream) {
  if (num_tiles <= 0) return;
  const int cap = sm_count() * 16;
  transpose_split_kernel<<<num_tiles < cap ? num_tiles : cap, 256, 0, stream>>>(ops, tiles, num_tiles);
}

}  // namespace ob200
