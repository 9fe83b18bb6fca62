// Fused kernels of the example transformer models (GPT-2, Llama): the memory-bound pieces around
// the library GEMMs of a training step.
//
//   xent_fwd_bwd      softmax cross-entropy over a [rows, ld] bf16 logits matrix of which the first
//                     V columns are valid: writes the per-row loss and overwrites the logits with
//                     softmax - onehot (the unscaled gradient); padding columns become zero.  One
//                     read and one write of the matrix from HBM instead of the five passes of the
//                     log_softmax / nll_loss / upcast chain.
//   norm_fwd / bwd    LayerNorm or RMSNorm over the last dim with fp32 statistics, input fp32 or
//                     bf16, output directly in the dtype the following GEMM consumes; the backward
//                     produces dx and per-CTA partial sums of dgamma / dbeta.
//
// No reference counterpart: the reference's examples use stock torch modules.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <torch/extension.h>

namespace ob200 {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Combine two (max, sum of exp(x - max)) partial softmax states.
__device__ __forceinline__ void softmax_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  const float a = (m == mm) ? s : s * __expf(m - mm);
  const float b = (m2 == mm) ? s2 : s2 * __expf(m2 - mm);
  m = mm;
  s = a + b;
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 t = __bfloat1622float2(h[k]);
    f[2 * k] = t.x;
    f[2 * k + 1] = t.y;
  }
}

constexpr int kXentThreads = 256;

// One CTA per row.  Pass 1: running max / sum-exp with 16-byte loads.  Pass 2 re-reads the row,
// which is still in L2 (a row is ~100 KB), and overwrites it with the gradient.
__global__ void __launch_bounds__(kXentThreads)
xent_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long ld, int V, const long long* __restrict__ targets,
                    float* __restrict__ loss_rows, long long ignore_index) {
  __shared__ float red_m[kXentThreads / 32], red_s[kXentThreads / 32];
  __shared__ float row_m, row_inv, row_logsum;
  const long long row = blockIdx.x;
  __nv_bfloat16* x = logits + row * ld;
  const long long tgt = targets[row];
  const bool ignored = tgt == ignore_index || tgt < 0 || tgt >= V;
  const int nvec = V / 8;
  const int ldvec = static_cast<int>(ld / 8);  // ld is a multiple of 8 (checked on the host)
  uint4* xv = reinterpret_cast<uint4*>(x);
  float x_tgt = 0.f;
  if (threadIdx.x == 0 && !ignored) x_tgt = __bfloat162float(x[tgt]);

  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += kXentThreads) {
    float f[8];
    unpack8(xv[i], f);
    float lm = f[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) lm = fmaxf(lm, f[k]);
    if (lm > m) {
      s *= __expf(m - lm);  // m == -inf gives 0 * 0
      m = lm;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) s += __expf(f[k] - m);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += kXentThreads) softmax_merge(m, s, __bfloat162float(x[i]), 1.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    softmax_merge(m, s, m2, s2);
  }
  if ((threadIdx.x & 31) == 0) {
    red_m[threadIdx.x >> 5] = m;
    red_s[threadIdx.x >> 5] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bm = red_m[0], bs = red_s[0];
    for (int w = 1; w < kXentThreads / 32; ++w) softmax_merge(bm, bs, red_m[w], red_s[w]);
    row_m = bm;
    row_inv = 1.f / bs;
    row_logsum = __logf(bs);
    loss_rows[row] = ignored ? 0.f : (row_logsum + bm - x_tgt);
  }
  __syncthreads();
  const float bm = row_m, inv = ignored ? 0.f : row_inv;
  const int tvec = ignored ? -1 : static_cast<int>(tgt / 8), tk = static_cast<int>(tgt % 8);
  for (int i = threadIdx.x; i < ldvec; i += kXentThreads) {
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (i < nvec) {
      float f[8];
      unpack8(xv[i], f);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = __expf(f[k] - bm) * inv;
      if (i == tvec) f[tk] -= 1.f;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
    } else if (i == nvec && (V & 7)) {
      // The vector that straddles V: valid scalars first, zeros after.
      __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(&out);
      for (int k = 0; k < (V & 7); ++k) {
        float p = __expf(__bfloat162float(x[i * 8 + k]) - bm) * inv;
        if (!ignored && i * 8 + k == tgt) p -= 1.f;
        h[k] = __float2bfloat16_rn(p);
      }
    }
    xv[i] = out;
  }
}

// ------------------------------------------------------------------------------------------------
// LayerNorm / RMSNorm.  One warp per row; C = kVecs * 128, each lane owns kVecs float4 groups.
// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float4& v) {
  uint2 u;
  *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = u;
}

constexpr int kNormThreads = 256;

template <int kVecs, bool kRms, typename InT, typename OutT>
__global__ void __launch_bounds__(kNormThreads)
norm_fwd_kernel(const InT* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                OutT* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, long long rows, float eps) {
  constexpr int C = kVecs * 128;
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * kNormThreads + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * kNormThreads) >> 5;
  for (long long r = warp; r < rows; r += nwarps) {
    float4 e[kVecs];
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      e[v] = load4(x + r * C + (v * 32 + lane) * 4);
      sum += (e[v].x + e[v].y) + (e[v].z + e[v].w);
    }
    const float mu = kRms ? 0.f : warp_sum(sum) * (1.f / C);
    float var = 0.f;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const float a = e[v].x - mu, bb = e[v].y - mu, c = e[v].z - mu, d = e[v].w - mu;
      var += (a * a + bb * bb) + (c * c + d * d);
    }
    const float rs = rsqrtf(warp_sum(var) * (1.f / C) + eps);
    if (lane == 0) {
      if (!kRms) mean[r] = mu;
      rstd[r] = rs;
    }
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      // gamma / beta stay in L1 across rows; holding them in registers would spill for wide rows.
      const float4 g = load4(gamma + (v * 32 + lane) * 4);
      const float4 b = kRms ? make_float4(0.f, 0.f, 0.f, 0.f) : load4(beta + (v * 32 + lane) * 4);
      float4 o;
      o.x = (e[v].x - mu) * rs * g.x + b.x;
      o.y = (e[v].y - mu) * rs * g.y + b.y;
      o.z = (e[v].z - mu) * rs * g.z + b.z;
      o.w = (e[v].w - mu) * rs * g.w + b.w;
      store4(y + r * C + (v * 32 + lane) * 4, o);
    }
  }
}

// kSmemAcc: wide rows keep no per-lane dgamma / dbeta accumulators (they would spill); every row adds
// its contributions to the shared-memory sums directly.
template <int kVecs, bool kRms, bool kSmemAcc, typename InT, typename GradT>
__global__ void __launch_bounds__(kNormThreads, 2)
norm_bwd_kernel(const GradT* __restrict__ dy, const InT* __restrict__ x, const float* __restrict__ gamma,
                const float* __restrict__ mean, const float* __restrict__ rstd, InT* __restrict__ dx,
                float* __restrict__ partial, long long rows) {
  constexpr int C = kVecs * 128;
  __shared__ float acc[2][C];
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * kNormThreads + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * kNormThreads) >> 5;
  for (int i = threadIdx.x; i < 2 * C; i += kNormThreads) (&acc[0][0])[i] = 0.f;
  constexpr int kAcc = kSmemAcc ? 1 : kVecs;
  float4 dg[kAcc], db[kAcc];
#pragma unroll
  for (int v = 0; v < kAcc; ++v) {
    dg[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    db[v] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();
  for (long long r = warp; r < rows; r += nwarps) {
    const float mu = kRms ? 0.f : mean[r], rs = rstd[r];
    float4 xh[kVecs], d[kVecs];
    float s1 = 0.f, s2 = 0.f;  // sum(dy*gamma), sum(dy*gamma*xhat)
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const float4 e = load4(x + r * C + (v * 32 + lane) * 4);
      const float4 t = load4(dy + r * C + (v * 32 + lane) * 4);
      const float4 g = load4(gamma + (v * 32 + lane) * 4);
      xh[v] = make_float4((e.x - mu) * rs, (e.y - mu) * rs, (e.z - mu) * rs, (e.w - mu) * rs);
      if constexpr (kSmemAcc) {
        const int c = (v * 32 + lane) * 4;
        atomicAdd(&acc[0][c], t.x * xh[v].x); atomicAdd(&acc[0][c + 1], t.y * xh[v].y);
        atomicAdd(&acc[0][c + 2], t.z * xh[v].z); atomicAdd(&acc[0][c + 3], t.w * xh[v].w);
        if (!kRms) {
          atomicAdd(&acc[1][c], t.x); atomicAdd(&acc[1][c + 1], t.y);
          atomicAdd(&acc[1][c + 2], t.z); atomicAdd(&acc[1][c + 3], t.w);
        }
      } else {
        dg[v].x += t.x * xh[v].x; dg[v].y += t.y * xh[v].y; dg[v].z += t.z * xh[v].z; dg[v].w += t.w * xh[v].w;
        db[v].x += t.x; db[v].y += t.y; db[v].z += t.z; db[v].w += t.w;
      }
      d[v] = make_float4(t.x * g.x, t.y * g.y, t.z * g.z, t.w * g.w);
      s1 += (d[v].x + d[v].y) + (d[v].z + d[v].w);
      s2 += (d[v].x * xh[v].x + d[v].y * xh[v].y) + (d[v].z * xh[v].z + d[v].w * xh[v].w);
    }
    const float m1 = kRms ? 0.f : warp_sum(s1) * (1.f / C);
    const float m2 = warp_sum(s2) * (1.f / C);
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      float4 o;
      o.x = (d[v].x - m1 - xh[v].x * m2) * rs;
      o.y = (d[v].y - m1 - xh[v].y * m2) * rs;
      o.z = (d[v].z - m1 - xh[v].z * m2) * rs;
      o.w = (d[v].w - m1 - xh[v].w * m2) * rs;
      store4(dx + r * C + (v * 32 + lane) * 4, o);
    }
  }
#pragma unroll
  for (int v = 0; v < kAcc; ++v) {
    if (kSmemAcc) break;
    const int c = (v * 32 + lane) * 4;
    atomicAdd(&acc[0][c], dg[v].x); atomicAdd(&acc[0][c + 1], dg[v].y);
    atomicAdd(&acc[0][c + 2], dg[v].z); atomicAdd(&acc[0][c + 3], dg[v].w);
    if (!kRms) {
      atomicAdd(&acc[1][c], db[v].x); atomicAdd(&acc[1][c + 1], db[v].y);
      atomicAdd(&acc[1][c + 2], db[v].z); atomicAdd(&acc[1][c + 3], db[v].w);
    }
  }
  __syncthreads();
  float* out = partial + static_cast<long long>(blockIdx.x) * 2 * C;
  for (int i = threadIdx.x; i < 2 * C; i += kNormThreads) out[i] = (&acc[0][0])[i];
}

// ------------------------------------------------------------------------------------------------
// Column sums of a [rows, N] matrix (bias gradient of a linear layer).  A lane owns four
// consecutive columns (8- or 16-byte loads), the eight warps of a CTA interleave the rows of one
// row slice with four loads in flight each, shared memory combines them into partial[slice][n];
// the CTA that finishes last for a column block then adds the slices in index order (a fixed order:
// the result does not depend on scheduling) and writes out[n], so no second launch is needed.
// ------------------------------------------------------------------------------------------------
constexpr int kColsumThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kColsumThreads)
colsum_kernel(const T* __restrict__ x, float* __restrict__ partial, float* __restrict__ out, int* __restrict__ counters,
              long long rows, int N, int rows_per_slice) {
  __shared__ float acc[kColsumThreads / 32][128];
  __shared__ int is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 128 + lane * 4;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_slice;
  const long long r1 = r0 + rows_per_slice < rows ? r0 + rows_per_slice : rows;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  if (col < N) {
    long long r = r0 + warp;
    for (; r + 24 < r1; r += 32) {
      const float4 a = load4(x + r * N + col), b = load4(x + (r + 8) * N + col);
      const float4 c = load4(x + (r + 16) * N + col), d = load4(x + (r + 24) * N + col);
      sum.x += (a.x + b.x) + (c.x + d.x); sum.y += (a.y + b.y) + (c.y + d.y);
      sum.z += (a.z + b.z) + (c.z + d.z); sum.w += (a.w + b.w) + (c.w + d.w);
    }
    for (; r < r1; r += 8) {
      const float4 a = load4(x + r * N + col);
      sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
    }
  }
  acc[warp][lane * 4] = sum.x; acc[warp][lane * 4 + 1] = sum.y;
  acc[warp][lane * 4 + 2] = sum.z; acc[warp][lane * 4 + 3] = sum.w;
  __syncthreads();
  const int c = blockIdx.x * 128 + (threadIdx.x & 127);
  if (threadIdx.x < 128 && c < N) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kColsumThreads / 32; ++w) t += acc[w][threadIdx.x];
    partial[static_cast<long long>(blockIdx.y) * N + c] = t;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&counters[blockIdx.x], 1) == static_cast<int>(gridDim.y) - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // Two halves of the slices by the two halves of the CTA, each in ascending slice order.
  const int half = threadIdx.x >> 7;
  float t = 0.f;
  if (c < N)
    for (int sl = half; sl < static_cast<int>(gridDim.y); sl += 2) t += __ldcg(partial + static_cast<long long>(sl) * N + c);
  if (half == 1) acc[0][threadIdx.x & 127] = t;
  __syncthreads();
  if (half == 0 && c < N) out[c] = t + acc[0][threadIdx.x];
}

int norm_grid(long long rows) {
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const long long need = (rows + kNormThreads / 32 - 1) / (kNormThreads / 32);
  return static_cast<int>(std::max<long long>(1, std::min<long long>(need, 4LL * sms)));
}

template <int kVecs, bool kRms>
void norm_fwd_launch(const torch::Tensor& x, const torch::Tensor& gamma, const torch::Tensor& beta, torch::Tensor& y,
                     torch::Tensor& mean, torch::Tensor& rstd, long long rows, float eps, cudaStream_t st) {
  const int grid = norm_grid(rows);
  const float* bp = kRms ? nullptr : beta.data_ptr<float>();
  float* mp = kRms ? nullptr : mean.data_ptr<float>();
  auto go = [&](auto* xp, auto* yp) {
    using InT = std::remove_cv_t<std::remove_pointer_t<decltype(xp)>>;
    using OutT = std::remove_pointer_t<decltype(yp)>;
    norm_fwd_kernel<kVecs, kRms, InT, OutT><<<grid, kNormThreads, 0, st>>>(xp, gamma.data_ptr<float>(), bp, yp, mp,
                                                                        rstd.data_ptr<float>(), rows, eps);
  };
  using bf = __nv_bfloat16;
  const bool xin_f = x.scalar_type() == torch::kFloat32, yout_f = y.scalar_type() == torch::kFloat32;
  if (xin_f && yout_f) go(x.data_ptr<float>(), y.data_ptr<float>());
  else if (xin_f) go(x.data_ptr<float>(), reinterpret_cast<bf*>(y.data_ptr()));
  else if (yout_f) go(reinterpret_cast<const bf*>(x.data_ptr()), y.data_ptr<float>());
  else go(reinterpret_cast<const bf*>(x.data_ptr()), reinterpret_cast<bf*>(y.data_ptr()));
}

template <int kVecs, bool kRms>
void norm_bwd_launch(const torch::Tensor& dy, const torch::Tensor& x, const torch::Tensor& gamma,
                     const torch::Tensor& mean, const torch::Tensor& rstd, torch::Tensor& dx, torch::Tensor& partial,
                     long long rows, int grid, cudaStream_t st) {
  const float* mp = kRms ? nullptr : mean.data_ptr<float>();
  auto go = [&](auto* dyp, auto* xp, auto* dxp) {
    using GradT = std::remove_cv_t<std::remove_pointer_t<decltype(dyp)>>;
    using InT = std::remove_pointer_t<decltype(dxp)>;
    norm_bwd_kernel<kVecs, kRms, (kVecs > 8), InT, GradT><<<grid, kNormThreads, 0, st>>>(
        dyp, xp, gamma.data_ptr<float>(), mp, rstd.data_ptr<float>(), dxp, partial.data_ptr<float>(), rows);
  };
  using bf = __nv_bfloat16;
  const bool x_f = x.scalar_type() == torch::kFloat32, dy_f = dy.scalar_type() == torch::kFloat32;
  if (x_f && dy_f) go(dy.data_ptr<float>(), x.data_ptr<float>(), dx.data_ptr<float>());
  else if (x_f) go(reinterpret_cast<const bf*>(dy.data_ptr()), x.data_ptr<float>(), dx.data_ptr<float>());
  else if (dy_f) go(dy.data_ptr<float>(), reinterpret_cast<const bf*>(x.data_ptr()), reinterpret_cast<bf*>(dx.data_ptr()));
  else go(reinterpret_cast<const bf*>(dy.data_ptr()), reinterpret_cast<const bf*>(x.data_ptr()), reinterpret_cast<bf*>(dx.data_ptr()));
}

#define OB200_NORM_DISPATCH(VECS, CALL)                                   \
  switch (VECS) {                                                         \
    case 2: { constexpr int kV = 2; CALL; break; }                        \
    case 4: { constexpr int kV = 4; CALL; break; }                        \
    case 6: { constexpr int kV = 6; CALL; break; }                        \
    case 8: { constexpr int kV = 8; CALL; break; }                        \
    case 16: { constexpr int kV = 16; CALL; break; }                      \
    default: TORCH_CHECK(false, "norm: unsupported feature size");        \
  }

bool check_float_like(const torch::Tensor& t) {
  return t.scalar_type() == torch::kFloat32 || t.scalar_type() == torch::kBFloat16;
}

}  // namespace

bool norm_supported(int64_t C) {
  const int64_t v = C / 128;
  return C % 128 == 0 && (v == 2 || v == 4 || v == 6 || v == 8 || v == 16);
}

// logits [rows, ld] bf16 (modified in place), targets [rows] int64 -> loss_rows [rows] fp32
torch::Tensor xent_fwd_bwd(torch::Tensor logits, int64_t V, const torch::Tensor& targets, int64_t ignore_index) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == torch::kBFloat16 && logits.stride(1) == 1,
              "xent: logits must be a 2-D bf16 CUDA tensor with unit inner stride");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == torch::kInt64 && targets.is_contiguous() &&
                  targets.numel() == logits.size(0), "xent: targets must be int64 [rows]");
  const int64_t ld = logits.stride(0);
  TORCH_CHECK(ld % 8 == 0 && V <= logits.size(1) && logits.size(1) <= ld && V > 0 && V < (1LL << 31),
              "xent: row pitch must be a multiple of 8 elements and cover V");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(logits.data_ptr()) % 16 == 0, "xent: logits must be 16-byte aligned");
  TORCH_CHECK(logits.size(1) == ld, "xent: the padded width must equal the row pitch");
  c10::cuda::CUDAGuard guard(logits.device());
  auto loss = torch::empty({logits.size(0)}, logits.options().dtype(torch::kFloat32));
  if (logits.size(0) == 0) return loss;
  xent_fwd_bwd_kernel<<<static_cast<unsigned>(logits.size(0)), kXentThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<__nv_bfloat16*>(logits.data_ptr()), ld, static_cast<int>(V), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
      loss.data_ptr<float>(), ignore_index);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return loss;
}

// x [rows, C] -> (y in out_dtype, mean, rstd).  rms: no mean / beta.
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> norm_fwd(const torch::Tensor& x, const torch::Tensor& gamma,
                                                                 const std::optional<torch::Tensor>& beta, double eps,
                                                                 bool rms, bool out_bf16) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && check_float_like(x), "norm: x must be [rows, C] fp32/bf16");
  const int64_t rows = x.size(0), C = x.size(1);
  TORCH_CHECK(norm_supported(C), "norm: unsupported feature size ", C);
  TORCH_CHECK(gamma.scalar_type() == torch::kFloat32 && gamma.is_contiguous() && gamma.numel() == C, "norm: gamma fp32 [C]");
  TORCH_CHECK(rms || (beta.has_value() && beta->scalar_type() == torch::kFloat32 && beta->is_contiguous() && beta->numel() == C),
              "norm: beta fp32 [C]");
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty({rows, C}, x.options().dtype(out_bf16 ? torch::kBFloat16 : torch::kFloat32));
  auto stats = x.options().dtype(torch::kFloat32);
  auto mean = torch::empty({rms ? 0 : rows}, stats), rstd = torch::empty({rows}, stats);
  if (rows == 0) return {y, mean, rstd};
  auto st = at::cuda::getCurrentCUDAStream();
  const torch::Tensor b = rms ? gamma : *beta;
  if (rms) {
    OB200_NORM_DISPATCH(C / 128, (norm_fwd_launch<kV, true>(x, gamma, b, y, mean, rstd, rows, static_cast<float>(eps), st)));
  } else {
    OB200_NORM_DISPATCH(C / 128, (norm_fwd_launch<kV, false>(x, gamma, b, y, mean, rstd, rows, static_cast<float>(eps), st)));
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, mean, rstd};
}

// -> (dx in x's dtype, partial [grid, 2, C] whose sum over dim 0 is (dgamma, dbeta))
std::tuple<torch::Tensor, torch::Tensor> norm_bwd(const torch::Tensor& dy, const torch::Tensor& x,
                                                  const torch::Tensor& gamma, const torch::Tensor& mean,
                                                  const torch::Tensor& rstd, bool rms) {
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && dy.sizes() == x.sizes() && check_float_like(dy), "norm: dy like x");
  TORCH_CHECK(x.is_contiguous() && check_float_like(x) && x.dim() == 2, "norm: x must be [rows, C]");
  const int64_t rows = x.size(0), C = x.size(1);
  TORCH_CHECK(norm_supported(C), "norm: unsupported feature size ", C);
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = torch::empty_like(x);
  const int grid = norm_grid(rows);
  auto partial = torch::empty({grid, 2, C}, x.options().dtype(torch::kFloat32));
  if (rows == 0) return {dx, partial.zero_()};
  auto st = at::cuda::getCurrentCUDAStream();
  if (rms) {
    OB200_NORM_DISPATCH(C / 128, (norm_bwd_launch<kV, true>(dy, x, gamma, mean, rstd, dx, partial, rows, grid, st)));
  } else {
    OB200_NORM_DISPATCH(C / 128, (norm_bwd_launch<kV, false>(dy, x, gamma, mean, rstd, dx, partial, rows, grid, st)));
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dx, partial};
}

// x [rows, N] fp32 / bf16 (N % 4 == 0) -> column sums [N] fp32
torch::Tensor colsum(const torch::Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && check_float_like(x), "colsum: x must be [rows, N] fp32/bf16");
  const int64_t rows = x.size(0), N = x.size(1);
  TORCH_CHECK(N % 4 == 0 && N < (1LL << 31), "colsum: N must be a multiple of 4");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "colsum: x must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(x.device());
  auto f32 = x.options().dtype(torch::kFloat32);
  if (rows == 0) return torch::zeros({N}, f32);
  const int col_blocks = static_cast<int>((N + 127) / 128);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  int slices = std::max<int>(1, std::min<int64_t>((4 * sms + col_blocks - 1) / col_blocks, (rows + 63) / 64));
  const int rows_per_slice = static_cast<int>((rows + slices - 1) / slices);
  slices = static_cast<int>((rows + rows_per_slice - 1) / rows_per_slice);
  auto partial = torch::empty({slices, N}, f32);
  auto out = torch::empty({N}, f32);
  auto counters = torch::zeros({col_blocks}, x.options().dtype(torch::kInt32));
  dim3 grid(col_blocks, slices);
  auto st = at::cuda::getCurrentCUDAStream();
  if (x.scalar_type() == torch::kFloat32) {
    colsum_kernel<float><<<grid, kColsumThreads, 0, st>>>(x.data_ptr<float>(), partial.data_ptr<float>(),
                                                          out.data_ptr<float>(), counters.data_ptr<int>(), rows,
                                                          static_cast<int>(N), rows_per_slice);
  } else {
    colsum_kernel<__nv_bfloat16><<<grid, kColsumThreads, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), partial.data_ptr<float>(), out.data_ptr<float>(),
        counters.data_ptr<int>(), rows, static_cast<int>(N), rows_per_slice);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

void register_model_ops(pybind11::module_& m) {
  m.def("colsum", &colsum);
  m.def("xent_fwd_bwd", &xent_fwd_bwd);
  m.def("norm_fwd", &norm_fwd);
  m.def("norm_bwd", &norm_bwd);
  m.def("norm_supported", &norm_supported);
}

}  // namespace ob200
