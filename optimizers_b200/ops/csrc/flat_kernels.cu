// See flat_kernels.cuh.
#include "flat_kernels.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace ob200 {

namespace {

// torch.lerp semantics: the formula switches at weight 0.5 to stay monotone.
__device__ __forceinline__ float lerpf(float a, float b, float w) {
  const float d = b - a;
  return w < 0.5f ? a + w * d : b - d * (1.f - w);
}

template <typename T>
__device__ __forceinline__ float load_as_float(const void* base, long long i);
template <>
__device__ __forceinline__ float load_as_float<float>(const void* base, long long i) {
  return static_cast<const float*>(base)[i];
}
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const void* base, long long i) {
  return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]);
}
template <>
__device__ __forceinline__ float load_as_float<__half>(const void* base, long long i) {
  return __half2float(static_cast<const __half*>(base)[i]);
}
template <typename T>
__device__ __forceinline__ void store_from_float(void* base, long long i, float x);
template <>
__device__ __forceinline__ void store_from_float<float>(void* base, long long i, float x) {
  static_cast<float*>(base)[i] = x;
}
template <>
__device__ __forceinline__ void store_from_float<__nv_bfloat16>(void* base, long long i, float x) {
  static_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(x);
}
template <>
__device__ __forceinline__ void store_from_float<__half>(void* base, long long i, float x) {
  static_cast<__half*>(base)[i] = __float2half_rn(x);
}

__global__ void __launch_bounds__(256) tf32_split_kernel(const float* __restrict__ src, long long src_pitch,
                                                         float* __restrict__ hi, float* __restrict__ lo,
                                                         long long dst_pitch, int rows, int cols) {
  const long long total = static_cast<long long>(rows) * cols;
  for (long long e = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; e < total;
       e += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(e / cols), j = static_cast<int>(e % cols);
    const float x = src[i * src_pitch + j];
    const float h = tf32_round(x);
    hi[i * dst_pitch + j] = h;
    lo[i * dst_pitch + j] = x - h;
  }
}

__global__ void __launch_bounds__(256) affine_identity_split_kernel(const MatOp* __restrict__ ops,
                                                                    const int2* __restrict__ chunks, int num_chunks,
                                                                    float a, float b) {
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ref = chunks[c];
    const MatOp op = ops[ref.x];
    const int row0 = ref.y * kMatRowsPerChunk;
    const int rows = min(kMatRowsPerChunk, op.d - row0);
    const bool vec = ((op.d | op.ld_src | op.ld_dst) & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(op.src) | reinterpret_cast<uintptr_t>(op.dst_hi) |
                       reinterpret_cast<uintptr_t>(op.dst_lo)) & 15) == 0;
    if (vec) {
      // 16-byte accesses: a thread owns four consecutive columns of a row.
      const int d4 = op.d >> 2;
      for (int e = threadIdx.x; e < rows * d4; e += blockDim.x) {
        const int i = row0 + e / d4, j = (e % d4) * 4;
        const float4 v = *reinterpret_cast<const float4*>(op.src + static_cast<long long>(i) * op.ld_src + j);
        float x[4] = {a * v.x, a * v.y, a * v.z, a * v.w};
        if (i >= j && i < j + 4) x[i - j] += b;
        const long long o = static_cast<long long>(i) * op.ld_dst + j;
        if (op.dst_lo != nullptr) {
          float h[4], l[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            h[k] = tf32_round(x[k]);
            l[k] = x[k] - h[k];
          }
          *reinterpret_cast<float4*>(op.dst_hi + o) = make_float4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<float4*>(op.dst_lo + o) = make_float4(l[0], l[1], l[2], l[3]);
        } else {
          *reinterpret_cast<float4*>(op.dst_hi + o) = make_float4(x[0], x[1], x[2], x[3]);
        }
      }
      continue;
    }
    for (int e = threadIdx.x; e < rows * op.d; e += blockDim.x) {
      const int i = row0 + e / op.d, j = e % op.d;
      float x = a * op.src[static_cast<long long>(i) * op.ld_src + j];
      if (i == j) x += b;
      const long long o = static_cast<long long>(i) * op.ld_dst + j;
      if (op.dst_lo != nullptr) {
        const float h = tf32_round(x);
        op.dst_hi[o] = h;
        op.dst_lo[o] = x - h;
      } else {
        op.dst_hi[o] = x;
      }
    }
  }
}

__global__ void __launch_bounds__(256) identity_error_kernel(const MatOp* __restrict__ ops,
                                                             const int2* __restrict__ chunks, int num_chunks) {
  __shared__ float red[8];
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ref = chunks[c];
    const MatOp op = ops[ref.x];
    const int row0 = ref.y * kMatRowsPerChunk;
    const int rows = min(kMatRowsPerChunk, op.d - row0);
    float worst = 0.f;
    for (int e = threadIdx.x; e < rows * op.d; e += blockDim.x) {
      const int i = row0 + e / op.d, j = e % op.d;
      const float x = op.src[static_cast<long long>(i) * op.ld_src + j] - (i == j ? 1.f : 0.f);
      const float ax = fabsf(x);
      worst = (ax > worst || ax != ax) ? ax : worst;  // NaN propagates
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, worst, o);
      worst = (other > worst || other != other) ? other : worst;
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = worst;
    __syncthreads();
    if (threadIdx.x == 0) {
      float w = 0.f;
      for (int k = 0; k < 8; ++k) w = (red[k] > w || red[k] != red[k]) ? red[k] : w;
      // Non-negative floats (and +NaN, which has the largest bit pattern) order like their bits.
      atomicMax(reinterpret_cast<int*>(op.err), __float_as_int(w));
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256) peer_copy_kernel(const CopyDesc* __restrict__ table,
                                                        const int2* __restrict__ chunks, int num_chunks) {
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ref = chunks[c];
    const CopyDesc d = table[ref.x];
    const long long begin = static_cast<long long>(ref.y) * kCopyChunkBytes;
    const long long left = d.bytes - begin;
    const int n = static_cast<int>(left < kCopyChunkBytes ? left : kCopyChunkBytes);
    const char* src = static_cast<const char*>(d.src) + begin;
    char* dst = static_cast<char*>(d.dst) + begin;
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
      const int nv = n / 16;
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      // Four independent 16-byte loads per thread before the first store.
      int i = threadIdx.x;
      for (; i + 3 * 256 < nv; i += 4 * 256) {
        const uint4 a = s4[i], b = s4[i + 256], e = s4[i + 512], f = s4[i + 768];
        d4[i] = a; d4[i + 256] = b; d4[i + 512] = e; d4[i + 768] = f;
      }
      for (; i < nv; i += 256) d4[i] = s4[i];
      for (int k = nv * 16 / 4 + threadIdx.x; k < n / 4; k += 256)
        reinterpret_cast<uint32_t*>(dst)[k] = reinterpret_cast<const uint32_t*>(src)[k];
    } else {
      for (int k = threadIdx.x; k < n / 4; k += 256)
        reinterpret_cast<uint32_t*>(dst)[k] = reinterpret_cast<const uint32_t*>(src)[k];
    }
  }
}

constexpr int kJacobiThreads = 1024;  // 32 warps: two column pairs per warp and round at n = 128
constexpr int kJacobiPitch = kJacobiMaxN + 1;  // odd: column reads and row (transposed) reads are both conflict-free

__global__ void __launch_bounds__(kJacobiThreads) jacobi_eigh_kernel(const JacobiDesc* __restrict__ descs,
                                                                     int max_sweeps, float tol,
                                                                     int* __restrict__ sweeps_out) {
  extern __shared__ float jsm[];
  float* a = jsm;                                // column j of A V at a + j * pitch
  float* v = jsm + kJacobiMaxN * kJacobiPitch;   // column j of V
  __shared__ int rotated;
  __shared__ int significant;  // a rotation of the current sweep was well above the tolerance
  __shared__ float lam_s[kJacobiMaxN];
  const JacobiDesc d = descs[blockIdx.x];
  const int n = d.n;
  const int np = n + (n & 1);  // even number of players; the extra one is a zero column
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int kWarps = kJacobiThreads / 32;

  // A is symmetric: row j read contiguously is column j.
  for (int j = warp; j < np; j += kWarps) {
    for (int i = lane; i < np; i += 32) {
      a[j * kJacobiPitch + i] = (i < n && j < n) ? d.a[static_cast<long long>(j) * d.lda + i] : 0.f;
      v[j * kJacobiPitch + i] = (i == j) ? 1.f : 0.f;
    }
  }
  __syncthreads();
  float shift = 0.f;
  if (d.shift_scale > 0.f) {
    __shared__ float fro_parts[kWarps];
    __shared__ float shift_s;
    float ss = 0.f;
    for (int e = threadIdx.x; e < n * n; e += kJacobiThreads) {
      const float x = a[(e / n) * kJacobiPitch + (e % n)];
      ss = fmaf(x, x, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) fro_parts[warp] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float total = 0.f;
      for (int w = 0; w < kWarps; ++w) total += fro_parts[w];
      shift_s = d.shift_scale * sqrtf(total);
    }
    __syncthreads();
    shift = shift_s;
    for (int j = threadIdx.x; j < n; j += kJacobiThreads) a[j * kJacobiPitch + j] += shift;
    __syncthreads();
  }

  int sweep = 0;
  bool converged = false, settled = false;
  for (; sweep < max_sweeps && !converged; ++sweep) {
    if (threadIdx.x == 0) rotated = significant = 0;
    __syncthreads();
    for (int r = 0; r < np - 1; ++r) {
      // Round r of the round-robin tournament: player np-1 stays, the others rotate.
      for (int k = warp; k < np / 2; k += kWarps) {
        int p, q;
        if (k == 0) {
          p = np - 1;
          q = r;
        } else {
          p = (r + k) % (np - 1);
          q = (r - k + (np - 1)) % (np - 1);
        }
        float* ap = a + p * kJacobiPitch;
        float* aq = a + q * kJacobiPitch;
        float alpha = 0.f, beta = 0.f, gamma = 0.f;
        for (int i = lane; i < n; i += 32) {
          const float x = ap[i], y = aq[i];
          alpha += x * x;
          beta += y * y;
          gamma += x * y;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          alpha += __shfl_xor_sync(0xffffffffu, alpha, o);
          beta += __shfl_xor_sync(0xffffffffu, beta, o);
          gamma += __shfl_xor_sync(0xffffffffu, gamma, o);
        }
        // sqrt(alpha) * sqrt(beta), not sqrt(alpha * beta): for a leaf with entries of 1e-12 the
        // product of the squared norms underflows to zero and every pair would rotate for ever.
        const float scale = sqrtf(alpha) * sqrtf(beta);
        if (fabsf(gamma) > tol * scale && fabsf(gamma) > 1e-37f) {
          const float zeta = (beta - alpha) / (2.f * gamma);
          const float t = copysignf(1.f, zeta) / (fabsf(zeta) + sqrtf(1.f + zeta * zeta));
          const float c = rsqrtf(1.f + t * t), s = c * t;
          float* vp = v + p * kJacobiPitch;
          float* vq = v + q * kJacobiPitch;
          for (int i = lane; i < n; i += 32) {
            const float x = ap[i], y = aq[i];
            ap[i] = c * x - s * y;
            aq[i] = s * x + c * y;
            const float vx = vp[i], vy = vq[i];
            vp[i] = c * vx - s * vy;
            vq[i] = s * vx + c * vy;
          }
          if (lane == 0) {
            rotated = 1;
            if (fabsf(gamma) > 8.f * tol * scale) significant = 1;
          }
        }
      }
      __syncthreads();
    }
    converged = rotated == 0;
    // Inner products of fp32 columns carry rounding noise of the order of the tolerance itself: a
    // pair can hover around it for ever.  A last sweep all of whose rotations were within 8 times
    // the tolerance has nothing left to remove.
    settled = converged || significant == 0;
    __syncthreads();
  }

  // lambda_j = v_j . (A v_j); ascending order by rank (ties broken by index).
  for (int j = warp; j < n; j += kWarps) {
    float dot = 0.f;
    for (int i = lane; i < n; i += 32) dot += v[j * kJacobiPitch + i] * a[j * kJacobiPitch + i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) lam_s[j] = dot;
  }
  __syncthreads();
  // Thousands of fp32 rotations leave V orthogonal only to ~3e-5; one Newton-Schulz step
  // V <- V (3 I - V^T V) / 2 squares that error.  M = 1.5 I - 0.5 V^T V goes where A V was.
  for (int j = warp; j < n; j += kWarps) {
    for (int k = 0; k <= j; ++k) {
      float dot = 0.f;
      for (int i = lane; i < n; i += 32) dot += v[j * kJacobiPitch + i] * v[k * kJacobiPitch + i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (lane == 0) {
        const float m = (j == k ? 1.5f : 0.f) - 0.5f * dot;
        a[j * kJacobiPitch + k] = m;
        a[k * kJacobiPitch + j] = m;
      }
    }
  }
  __syncthreads();
  for (int i = warp; i < n; i += kWarps) {  // row i of V (component i of every eigenvector) is owned by one warp
    float acc[kJacobiMaxN / 32];
#pragma unroll
    for (int u = 0; u < kJacobiMaxN / 32; ++u) acc[u] = 0.f;
    for (int k = 0; k < n; ++k) {
      const float x = v[k * kJacobiPitch + i];
#pragma unroll
      for (int u = 0; u < kJacobiMaxN / 32; ++u) {
        const int j = lane + 32 * u;
        if (j < n) acc[u] += x * a[k * kJacobiPitch + j];
      }
    }
    __syncwarp();
#pragma unroll
    for (int u = 0; u < kJacobiMaxN / 32; ++u) {
      const int j = lane + 32 * u;
      if (j < n) v[j * kJacobiPitch + i] = acc[u];
    }
  }
  __syncthreads();
  int* rank_of = reinterpret_cast<int*>(a);  // M is no longer needed
  for (int j = threadIdx.x; j < n; j += kJacobiThreads) {
    const float x = lam_s[j];
    int rank = 0;
    for (int k = 0; k < n; ++k) rank += (lam_s[k] < x) || (lam_s[k] == x && k < j);
    rank_of[j] = rank;
    d.lam[rank] = x - shift;
  }
  __syncthreads();
  // Q[i][rank(j)] = v_j[i]; lanes run over j so that the scattered destination stays within a row.
  if (d.transposed) {
    // Row rank(j) of q is eigenvector j: lanes run over its components.
    for (int j = warp; j < n; j += kWarps)
      for (int i = lane; i < n; i += 32) d.q[static_cast<long long>(rank_of[j]) * d.ldq + i] = v[j * kJacobiPitch + i];
  } else {
    for (int i = warp; i < n; i += kWarps)
      for (int j = lane; j < n; j += 32) d.q[static_cast<long long>(i) * d.ldq + rank_of[j]] = v[j * kJacobiPitch + i];
  }
  if (threadIdx.x == 0) sweeps_out[blockIdx.x] = settled ? sweep : max_sweeps + 1;
}

struct GpaScalars {
  float lr, beta1, beta2, eps, bc1, bc2, wd, avg_coeff, mu_y;
  int wd_on_y;
};

template <typename T>
__device__ __forceinline__ void gpa_chunk(const GpaTensorDesc& d, long long begin, long long end, const GpaScalars& s) {
  const float y_step = s.lr * (s.mu_y * (1.f - s.avg_coeff) - 1.f);
  const float shrink = 1.f - s.lr * s.wd;
  for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float g = load_as_float<T>(d.grad, i);
    float y = load_as_float<T>(d.param, i);
    float z = d.z[i];
    const float m = lerpf(d.m[i], g, 1.f - s.beta1);
    const float v = s.beta2 * d.v[i] + (1.f - s.beta2) * g * g;
    d.m[i] = m;
    d.v[i] = v;
    const float gn = (m / s.bc1) / (sqrtf(v / s.bc2) + s.eps);
    if (s.wd != 0.f) {
      if (s.wd_on_y) {
        y *= shrink;
      } else {
        z *= shrink;
      }
    }
    y = lerpf(y, z, s.avg_coeff);
    y += y_step * gn;
    z -= s.lr * gn;
    store_from_float<T>(d.param, i, y);
    d.z[i] = z;
  }
}

__device__ __forceinline__ void gpa_element(float g, float& y, float& z, float& m, float& v, const GpaScalars& s,
                                            float y_step, float shrink) {
  m = lerpf(m, g, 1.f - s.beta1);
  v = s.beta2 * v + (1.f - s.beta2) * g * g;
  const float gn = (m / s.bc1) / (sqrtf(v / s.bc2) + s.eps);
  if (s.wd != 0.f) {
    if (s.wd_on_y) {
      y *= shrink;
    } else {
      z *= shrink;
    }
  }
  y = lerpf(y, z, s.avg_coeff);
  y += y_step * gn;
  z -= s.lr * gn;
}

// fp32 parameters with 16-byte aligned arrays: two 16-byte groups per thread and array are loaded
// before anything is stored, twice per 4096-element chunk.
__device__ __forceinline__ void gpa_chunk_vec4(const GpaTensorDesc& d, long long begin, long long end,
                                               const GpaScalars& s) {
  const float y_step = s.lr * (s.mu_y * (1.f - s.avg_coeff) - 1.f);
  const float shrink = 1.f - s.lr * s.wd;
  const float4* g4 = reinterpret_cast<const float4*>(static_cast<const float*>(d.grad) + begin);
  float4* y4 = reinterpret_cast<float4*>(static_cast<float*>(d.param) + begin);
  float4* z4 = reinterpret_cast<float4*>(d.z + begin);
  float4* m4 = reinterpret_cast<float4*>(d.m + begin);
  float4* v4 = reinterpret_cast<float4*>(d.v + begin);
  const int nvec = static_cast<int>((end - begin) / 4);
  for (int base = 0; base < nvec; base += 512) {
    float4 g[2], y[2], z[2], m[2], v[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = base + u * 256 + threadIdx.x;
      if (i < nvec) {
        g[u] = g4[i]; y[u] = y4[i]; z[u] = z4[i]; m[u] = m4[i]; v[u] = v4[i];
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = base + u * 256 + threadIdx.x;
      if (i < nvec) {
        gpa_element(g[u].x, y[u].x, z[u].x, m[u].x, v[u].x, s, y_step, shrink);
        gpa_element(g[u].y, y[u].y, z[u].y, m[u].y, v[u].y, s, y_step, shrink);
        gpa_element(g[u].z, y[u].z, z[u].z, m[u].z, v[u].z, s, y_step, shrink);
        gpa_element(g[u].w, y[u].w, z[u].w, m[u].w, v[u].w, s, y_step, shrink);
        y4[i] = y[u]; z4[i] = z[u]; m4[i] = m[u]; v4[i] = v[u];
      }
    }
  }
  // ragged tail of the last chunk
  for (long long i = begin + 4LL * nvec + threadIdx.x; i < end; i += blockDim.x) {
    float y = static_cast<float*>(d.param)[i], z = d.z[i], m = d.m[i], v = d.v[i];
    gpa_element(static_cast<const float*>(d.grad)[i], y, z, m, v, s, y_step, shrink);
    static_cast<float*>(d.param)[i] = y; d.z[i] = z; d.m[i] = m; d.v[i] = v;
  }
}

__device__ __forceinline__ bool gpa_aligned16(const GpaTensorDesc& d) {
  return ((reinterpret_cast<uintptr_t>(d.param) | reinterpret_cast<uintptr_t>(d.grad) | reinterpret_cast<uintptr_t>(d.z) |
           reinterpret_cast<uintptr_t>(d.m) | reinterpret_cast<uintptr_t>(d.v)) & 15) == 0;
}

__global__ void __launch_bounds__(256, 3) gpa_adamw_kernel(const GpaTensorDesc* __restrict__ table,
                                                        const int2* __restrict__ chunks, int num_chunks, GpaScalars s) {
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ref = chunks[c];
    const GpaTensorDesc d = table[ref.x];
    if (d.grad == nullptr) continue;
    const long long begin = static_cast<long long>(ref.y) * kGpaChunk;
    const long long end = begin + kGpaChunk < d.numel ? begin + kGpaChunk : d.numel;
    if (d.dtype == 0) {
      if (gpa_aligned16(d)) {
        gpa_chunk_vec4(d, begin, end, s);
      } else {
        gpa_chunk<float>(d, begin, end, s);
      }
    } else if (d.dtype == 1) {
      gpa_chunk<__nv_bfloat16>(d, begin, end, s);
    } else {
      gpa_chunk<__half>(d, begin, end, s);
    }
  }
}

template <typename T>
__device__ __forceinline__ void lerp_chunk(const GpaTensorDesc& d, long long begin, long long end, float w) {
  for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
    store_from_float<T>(d.param, i, lerpf(load_as_float<T>(d.param, i), d.z[i], w));
  }
}

__global__ void __launch_bounds__(256) gpa_lerp_kernel(const GpaTensorDesc* __restrict__ table,
                                                       const int2* __restrict__ chunks, int num_chunks, float w) {
  for (int c = blockIdx.x; c < num_chunks; c += gridDim.x) {
    const int2 ref = chunks[c];
    const GpaTensorDesc d = table[ref.x];
    const long long begin = static_cast<long long>(ref.y) * kGpaChunk;
    const long long end = begin + kGpaChunk < d.numel ? begin + kGpaChunk : d.numel;
    if (d.dtype == 0) {
      lerp_chunk<float>(d, begin, end, w);
    } else if (d.dtype == 1) {
      lerp_chunk<__nv_bfloat16>(d, begin, end, w);
    } else {
      lerp_chunk<__half>(d, begin, end, w);
    }
  }
}

int grid_for(long long work_items) {
  const long long cap = sm_count() * 8;
  return static_cast<int>(work_items < cap ? (work_items > 0 ? work_items : 1) : cap);
}

}  // namespace

void launch_affine_identity_split(const MatOp* ops, const int2* chunks, int num_chunks, float a, float b,
                                  cudaStream_t stream) {
  if (num_chunks <= 0) return;
  affine_identity_split_kernel<<<grid_for(num_chunks), 256, 0, stream>>>(ops, chunks, num_chunks, a, b);
}

void launch_identity_error(const MatOp* ops, const int2* chunks, int num_chunks, cudaStream_t stream) {
  if (num_chunks <= 0) return;
  identity_error_kernel<<<grid_for(num_chunks), 256, 0, stream>>>(ops, chunks, num_chunks);
}

void launch_jacobi_eigh(const JacobiDesc* descs, int count, int max_sweeps, float tol, int* sweeps,
                        cudaStream_t stream) {
  if (count <= 0) return;
  constexpr int smem = 2 * kJacobiMaxN * kJacobiPitch * static_cast<int>(sizeof(float));
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(jacobi_eigh_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured = true;
  }
  jacobi_eigh_kernel<<<count, kJacobiThreads, smem, stream>>>(descs, max_sweeps, tol, sweeps);
}

void launch_peer_copy(const CopyDesc* table, const int2* chunks, int num_chunks, cudaStream_t stream) {
  if (num_chunks <= 0) return;
  const int cap = sm_count() * 8;
  peer_copy_kernel<<<num_chunks < cap ? num_chunks : cap, 256, 0, stream>>>(table, chunks, num_chunks);
}

void launch_tf32_split(const float* src, long long src_pitch, float* hi, float* lo, long long dst_pitch, int rows,
                       int cols, cudaStream_t stream) {
  const long long total = static_cast<long long>(rows) * cols;
  if (total == 0) return;
  tf32_split_kernel<<<grid_for((total + 255) / 256), 256, 0, stream>>>(src, src_pitch, hi, lo, dst_pitch, rows, cols);
}

void launch_gpa_adamw(const GpaTensorDesc* table, const int2* chunks, int num_chunks, float lr, float beta1,
                      float beta2, float eps, float bias_correction1, float bias_correction2, float weight_decay,
                      bool wd_on_y, float avg_coeff, float train_interp_coeff, cudaStream_t stream) {
  if (num_chunks <= 0) return;
  GpaScalars s{lr, beta1, beta2, eps, bias_correction1, bias_correction2, weight_decay, avg_coeff, train_interp_coeff,
               wd_on_y ? 1 : 0};
  gpa_adamw_kernel<<<grid_for(num_chunks), 256, 0, stream>>>(table, chunks, num_chunks, s);
}

void launch_gpa_lerp(const GpaTensorDesc* table, const int2* chunks, int num_chunks, float weight,
                     cudaStream_t stream) {
  if (num_chunks <= 0) return;
  gpa_lerp_kernel<<<grid_for(num_chunks), 256, 0, stream>>>(table, chunks, num_chunks, weight);
}

}  // namespace ob200
