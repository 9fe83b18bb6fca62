// Grouped per-block pointwise kernels; see block_kernels.cuh.
#include "block_kernels.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace ob200 {

namespace {

constexpr int kTile = 32;
constexpr int kRowsPerThread = 4;  // 32 x 8 threads cover a 32 x 32 tile

// torch.lerp semantics: the formula switches at weight 0.5.
__device__ __forceinline__ float lerpf(float a, float b, float w) {
  const float d = b - a;
  return w < 0.5f ? a + w * d : b - d * (1.f - w);
}

__device__ __forceinline__ float graft_direction(float f, float v, int kind, float bc2, float eps) {
  if (kind == kGraftAdaGrad) return f / (sqrtf(v / bc2) + eps);
  return f;
}

__global__ void __launch_bounds__(256) grad_prologue_kernel(PrologueArgs a) {
  __shared__ float t_hi[kTile][kTile + 1];
  __shared__ float t_lo[kTile][kTile + 1];
  __shared__ float red[8];

  for (int t = blockIdx.x; t < a.num_tiles; t += gridDim.x) {
    const TileRef ref = a.tiles[t];
    const BlockDesc& b = a.blocks[ref.block];
    const int n_src = a.num_grad_peers > 0 ? a.num_grad_peers : 1;
    const float* const* srcs = a.grad_ptrs + static_cast<long long>(b.grad_slot) * n_src;
    const int i0 = ref.ti * kTile, j0 = ref.tj * kTile;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int j = j0 + tx;
    const bool want_t = b.gt_hi != nullptr;
    float sq = 0.f;
    bool bad = false;

#pragma unroll
    for (int r = 0; r < kRowsPerThread; ++r) {
      const int li = ty + r * 8;
      const int i = i0 + li;
      float hi = 0.f, lo = 0.f;
      if (i < b.m && j < b.n) {
        const long long e = static_cast<long long>(i) * b.n + j;           // contiguous state index
        const long long ge = b.grad_offset + static_cast<long long>(i) * b.param_pitch + j;
        float g;
        if (a.num_grad_peers > 0) {
          // Plain (coherent) loads: the sources are other GPUs' memory written by their last
          // backward pass; fixed rank order keeps the sum identical on every owner.
          g = 0.f;
          for (int r = 0; r < n_src; ++r) g += *reinterpret_cast<const volatile float*>(srcs[r] + ge);
          g *= a.grad_scale;
        } else {
          g = srcs[0][ge];
        }
        if (a.l2_weight_decay != 0.f) g += a.l2_weight_decay * b.param[static_cast<long long>(i) * b.param_pitch + j];
        bad |= !isfinite(g);
        if (a.write_split) {
          hi = tf32_round(g);
          lo = g - hi;
        } else {
          hi = g;
        }
        if (b.g_hi != nullptr) {
          const long long o = static_cast<long long>(i) * b.n_pad + j;
          b.g_hi[o] = hi;
          if (a.write_split) b.g_lo[o] = lo;
        }
        // Filtered gradient: EMA with beta1; the applied estimate uses beta3 on the old EMA.
        float f = g;
        if (b.m1 != nullptr) {
          const float m_old = b.m1[e];
          const float m_new = lerpf(m_old, g, 1.f - a.beta1);
          b.m1[e] = m_new;
          f = (a.beta3 != a.beta1) ? lerpf(m_old, g, 1.f - a.beta3) : m_new;
          f = f / a.bias_correction1;
        }
        {
          const long long o = static_cast<long long>(i) * b.n_pad + j;
          if (a.write_split) {
            const float fh = tf32_round(f);
            b.f_hi[o] = fh;
            b.f_lo[o] = f - fh;
          } else {
            b.f_hi[o] = f;
          }
        }
        if (a.graft_kind != kGraftNone) {
          float v = 0.f;
          if (a.graft_kind == kGraftAdaGrad) {
            v = a.graft_beta2 * b.v[e] + a.graft_weight * g * g;
            b.v[e] = v;
          }
          const float gd = graft_direction(f, v, a.graft_kind, a.graft_bias_correction2, a.graft_epsilon);
          sq += gd * gd;
        }
      }
      if (want_t) {
        t_hi[li][tx] = hi;
        t_lo[li][tx] = lo;
      }
    }
    if (want_t) {
      __syncthreads();
#pragma unroll
      for (int r = 0; r < kRowsPerThread; ++r) {
        const int lj = ty + r * 8;  // column of the source tile = row of the transposed array
        const int jj = j0 + lj;
        const int ii = i0 + tx;
        if (jj < b.n && ii < b.m) {
          const long long o = static_cast<long long>(jj) * b.m_pad + ii;
          b.gt_hi[o] = t_hi[tx][lj];
          if (a.write_split) b.gt_lo[o] = t_lo[tx][lj];
        }
      }
    }
    if (a.graft_kind != kGraftNone) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (tx == 0) red[ty] = sq;
    }
    if (bad) atomicOr(a.status, 2);
    __syncthreads();
    if (a.graft_kind != kGraftNone && threadIdx.x == 0) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += red[w];
      if (s != 0.f) atomicAdd(&b.norms[0], s);
    }
    __syncthreads();
  }
}

template <typename T>
__device__ __forceinline__ void store_send(void* base, long long idx, float x);
template <>
__device__ __forceinline__ void store_send<float>(void* base, long long idx, float x) {
  static_cast<float*>(base)[idx] = x;
}
template <>
__device__ __forceinline__ void store_send<__nv_bfloat16>(void* base, long long idx, float x) {
  static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(x);
}
template <>
__device__ __forceinline__ void store_send<__half>(void* base, long long idx, float x) {
  static_cast<__half*>(base)[idx] = __float2half_rn(x);
}

__global__ void __launch_bounds__(256) direction_epilogue_kernel(EpilogueArgs a) {
  const float lr = *a.lr;
  float mu_x = 0.f, mu_y = 0.f;
  if (a.primal_averaging) {
    mu_x = *a.mu_x;
    mu_y = *a.mu_y;
  }
  for (int t = blockIdx.x; t < a.num_tiles; t += gridDim.x) {
    const TileRef ref = a.tiles[t];
    const BlockDesc& b = a.blocks[ref.block];
    const int i0 = ref.ti * kTile, j0 = ref.tj * kTile;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int j = j0 + tx;
    float scale = 1.f;
    if (!a.graft_only && a.graft_kind != kGraftNone) {
      scale = sqrtf(b.norms[0]) / (sqrtf(b.norms[1]) + 1e-16f);
    }
#pragma unroll
    for (int r = 0; r < kRowsPerThread; ++r) {
      const int i = i0 + ty + r * 8;
      if (i >= b.m || j >= b.n) continue;
      const long long e = static_cast<long long>(i) * b.n + j;
      const long long pe = static_cast<long long>(i) * b.param_pitch + j;
      float p;
      if (a.graft_only) {
        const long long o = static_cast<long long>(i) * b.n_pad + j;
        const float f = a.split_input ? b.f_hi[o] + b.f_lo[o] : b.f_hi[o];
        const float v = (a.graft_kind == kGraftAdaGrad) ? b.v[e] : 0.f;
        p = graft_direction(f, v, a.graft_kind, a.graft_bias_correction2, a.graft_epsilon);
      } else {
        p = b.p[e] * scale;
      }
      const float w = b.param[pe];
      float z = 0.f;
      if (a.primal_averaging) {
        z = b.z[e];
        if (a.wd_alpha != 0.f) z *= 1.f - lr * a.wd_alpha;
      } else if (a.wd_alpha != 0.f) {
        p += a.wd_alpha * w;
      }
      if (a.classic_momentum) {
        const float mo = a.momentum * b.mom[e] + (1.f - a.dampening) * p;
        b.mom[e] = mo;
        p = a.nesterov ? (1.f - a.dampening) * p + a.momentum * mo : mo;
      }
      p *= -lr;
      if (a.primal_averaging) {
        const float gap = z - w;
        b.z[e] = z + p;
        p = (1.f - mu_x * mu_y) * p + (1.f - mu_x) * gap;
      }
      if (a.num_push_peers > 0) {
        for (int r = 0; r < a.num_push_peers; ++r) {
          void* dst = reinterpret_cast<void*>(a.peer_base[r] + b.slot_offset);
          if (a.send_dtype == 1) {
            store_send<__nv_bfloat16>(dst, e, p);
          } else if (a.send_dtype == 2) {
            store_send<__half>(dst, e, p);
          } else {
            store_send<float>(dst, e, p);
          }
        }
      } else if (b.send != nullptr) {
        if (a.send_dtype == 1) {
          store_send<__nv_bfloat16>(b.send, e, p);
        } else if (a.send_dtype == 2) {
          store_send<__half>(b.send, e, p);
        } else {
          store_send<float>(b.send, e, p);
        }
      } else {
        b.param[pe] = w + p;
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ float load_recv(const void* base, long long idx);
template <>
__device__ __forceinline__ float load_recv<float>(const void* base, long long idx) {
  return static_cast<const float*>(base)[idx];
}
template <>
__device__ __forceinline__ float load_recv<__nv_bfloat16>(const void* base, long long idx) {
  return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
}
template <>
__device__ __forceinline__ float load_recv<__half>(const void* base, long long idx) {
  return __half2float(static_cast<const __half*>(base)[idx]);
}

// Every rank applies every block's gathered search direction: param += cast(slot).
__global__ void __launch_bounds__(256) gathered_apply_kernel(const BlockDesc* __restrict__ blocks,
                                                             const TileRef* __restrict__ tiles, int num_tiles,
                                                             int dtype) {
  for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const TileRef ref = tiles[t];
    const BlockDesc& b = blocks[ref.block];
    const int i0 = ref.ti * kTile, j0 = ref.tj * kTile;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int j = j0 + tx;
#pragma unroll
    for (int r = 0; r < kRowsPerThread; ++r) {
      const int i = i0 + ty + r * 8;
      if (i >= b.m || j >= b.n) continue;
      const long long e = static_cast<long long>(i) * b.n + j;
      const long long pe = static_cast<long long>(i) * b.param_pitch + j;
      float d;
      if (dtype == 1) {
        d = load_recv<__nv_bfloat16>(b.send, e);
      } else if (dtype == 2) {
        d = load_recv<__half>(b.send, e);
      } else {
        d = load_recv<float>(b.send, e);
      }
      b.param[pe] += d;
    }
  }
}

__global__ void __launch_bounds__(256) eig_scale_kernel(const BlockDesc* __restrict__ blocks,
                                                        const TileRef* __restrict__ tiles, int num_tiles, float bc2,
                                                        float inv_root, float eps, int write_split) {
  for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const TileRef ref = tiles[t];
    const BlockDesc& b = blocks[ref.block];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int j = ref.tj * kTile + tx;
#pragma unroll
    for (int r = 0; r < kRowsPerThread; ++r) {
      const int i = ref.ti * kTile + ty + r * 8;
      if (i >= b.m || j >= b.n) continue;
      const long long e = static_cast<long long>(i) * b.n + j;
      const float denom = powf(b.ev[e] / bc2, inv_root) + eps;
      const float s = b.p[e] / denom;
      const long long o = static_cast<long long>(i) * b.n_pad + j;
      if (write_split) {
        const float h = tf32_round(s);
        b.f_hi[o] = h;
        b.f_lo[o] = s - h;
      } else {
        b.f_hi[o] = s;
      }
    }
  }
}

__global__ void __launch_bounds__(256) mode_switch_kernel(const BlockDesc* __restrict__ blocks,
                                                          const TileRef* __restrict__ tiles, int num_tiles, float coeff,
                                                          int send_dtype) {
  for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const TileRef ref = tiles[t];
    const BlockDesc& b = blocks[ref.block];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int j = ref.tj * kTile + tx;
#pragma unroll
    for (int r = 0; r < kRowsPerThread; ++r) {
      const int i = ref.ti * kTile + ty + r * 8;
      if (i >= b.m || j >= b.n) continue;
      const long long e = static_cast<long long>(i) * b.n + j;
      const long long pe = static_cast<long long>(i) * b.param_pitch + j;
      const float w = b.param[pe];
      const float delta = (b.z[e] - w) * coeff;
      if (b.send != nullptr) {
        if (send_dtype == 1) {
          store_send<__nv_bfloat16>(b.send, e, delta);
        } else if (send_dtype == 2) {
          store_send<__half>(b.send, e, delta);
        } else {
          store_send<float>(b.send, e, delta);
        }
      } else {
        b.param[pe] = w + delta;
      }
    }
  }
}

__global__ void peer_barrier_kernel(int* local_flags, const unsigned long long* peer_flag_bases, int my_rank,
                                    int world, int seq, int* status) {
  // Everything this rank wrote before the barrier (earlier kernels of the stream) must be
  // visible to the peers that observe the flag.
  __threadfence_system();
  const int r = threadIdx.x;
  if (r < world) {
    int* remote = reinterpret_cast<int*>(peer_flag_bases[r]) + my_rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(seq) : "memory");
    const unsigned long long t0 = globaltimer_ns();
    int seen;
    do {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(local_flags + r) : "memory");
      if (seen >= seq) break;
      if (globaltimer_ns() - t0 > kWaitBudgetNs) {
        atomicOr(status, kErrPeerTimeout);
        break;
      }
      __nanosleep(100);
    } while (true);
  }
  __threadfence_system();
}

int grid_for(int num_tiles) {
  // A few waves of CTAs per SM; the kernels loop over the tile list.
  const int cap = 148 * 8;
  return num_tiles < cap ? num_tiles : cap;
}

}  // namespace

void launch_grad_prologue(const PrologueArgs& args, cudaStream_t stream) {
  if (args.num_tiles <= 0) return;
  grad_prologue_kernel<<<grid_for(args.num_tiles), 256, 0, stream>>>(args);
}

void launch_direction_epilogue(const EpilogueArgs& args, cudaStream_t stream) {
  if (args.num_tiles <= 0) return;
  direction_epilogue_kernel<<<grid_for(args.num_tiles), 256, 0, stream>>>(args);
}

void launch_eig_scale(const BlockDesc* blocks, const TileRef* tiles, int num_tiles, float bias_correction2,
                      float inv_root, float epsilon, int write_split, cudaStream_t stream) {
  if (num_tiles <= 0) return;
  eig_scale_kernel<<<grid_for(num_tiles), 256, 0, stream>>>(blocks, tiles, num_tiles, bias_correction2, inv_root,
                                                            epsilon, write_split);
}

void launch_mode_switch(const BlockDesc* blocks, const TileRef* tiles, int num_tiles, float coeff, int send_dtype,
                        cudaStream_t stream) {
  if (num_tiles <= 0) return;
  mode_switch_kernel<<<grid_for(num_tiles), 256, 0, stream>>>(blocks, tiles, num_tiles, coeff, send_dtype);
}

void launch_peer_barrier(int* local_flags, const unsigned long long* peer_flag_bases, int my_rank, int world,
                         int seq, int* status, cudaStream_t stream) {
  peer_barrier_kernel<<<1, 32, 0, stream>>>(local_flags, peer_flag_bases, my_rank, world, seq, status);
}

void launch_gathered_apply(const BlockDesc* blocks, const TileRef* tiles, int num_tiles, int dtype,
                           cudaStream_t stream) {
  if (num_tiles <= 0) return;
  gathered_apply_kernel<<<grid_for(num_tiles), 256, 0, stream>>>(blocks, tiles, num_tiles, dtype);
}

}  // namespace ob200
