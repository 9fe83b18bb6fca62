// Grouped per-block pointwise kernels; see block_kernels.cuh.
#include "block_kernels.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace ob200 {

namespace {

constexpr int kTile = 32;

// torch.lerp semantics: the formula switches at weight 0.5.
__device__ __forceinline__ float lerpf(float a, float b, float w) {
  const float d = b - a;
  return w < 0.5f ? a + w * d : b - d * (1.f - w);
}

__device__ __forceinline__ float graft_direction(float f, float v, int kind, float bc2, float eps) {
  if (kind == kGraftAdaGrad) return f / (sqrtf(v / bc2) + eps);
  return f;
}

// ---------------------------------------------------------------------------------------------
// The three per-step HBM-bound kernels work on "wide" tiles of 32 rows x 128 columns: a warp owns
// a full 512-byte row segment, a lane four consecutive columns, so that every access is one
// 16-byte transaction and a thread has 4 rows x 16 bytes per array in flight.  Blocks whose
// layout does not allow 16-byte accesses (odd pitches or offsets) take the scalar form of the same
// code, decided once per tile.
// ---------------------------------------------------------------------------------------------
constexpr int kWide = 128;

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Loads 4 consecutive floats (the first `cnt` of them when not `vec`; the rest read as zero).
// kPeer: the source may be another GPU's memory written by its last backward pass, so the load
// must not be served from a stale L1 line (ld.global.cv).
template <bool kPeer>
__device__ __forceinline__ void load4(float (&out)[4], const float* p, bool vec, int cnt) {
  if (vec) {
    const float4 t = kPeer ? __ldcv(reinterpret_cast<const float4*>(p)) : *reinterpret_cast<const float4*>(p);
    out[0] = t.x; out[1] = t.y; out[2] = t.z; out[3] = t.w;
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) out[k] = k < cnt ? (kPeer ? __ldcv(p + k) : p[k]) : 0.f;
  }
}

__device__ __forceinline__ void store4(float* p, const float (&v)[4], bool vec, int cnt) {
  if (vec) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (k < cnt) p[k] = v[k];
  }
}

// Stores 4 consecutive elements of the communication dtype (0 fp32, 1 bf16, 2 fp16) at element e.
__device__ __forceinline__ void store_send4(void* base, long long e, const float (&v)[4], int dtype, bool vec, int cnt) {
  if (dtype == 0) {
    store4(static_cast<float*>(base) + e, v, vec, cnt);
  } else if (dtype == 1) {
    __nv_bfloat16* q = static_cast<__nv_bfloat16*>(base) + e;
    if (vec) {
      uint2 u;
      *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v[0], v[1]);
      *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v[2], v[3]);
      *reinterpret_cast<uint2*>(q) = u;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k < cnt) q[k] = __float2bfloat16_rn(v[k]);
    }
  } else {
    __half* q = static_cast<__half*>(base) + e;
    if (vec) {
      uint2 u;
      *reinterpret_cast<__half2*>(&u.x) = __floats2half2_rn(v[0], v[1]);
      *reinterpret_cast<__half2*>(&u.y) = __floats2half2_rn(v[2], v[3]);
      *reinterpret_cast<uint2*>(q) = u;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k < cnt) q[k] = __float2half_rn(v[k]);
    }
  }
}

__device__ __forceinline__ void load_recv4(float (&out)[4], const void* base, long long e, int dtype, bool vec, int cnt) {
  if (dtype == 0) {
    load4<false>(out, static_cast<const float*>(base) + e, vec, cnt);
  } else if (dtype == 1) {
    const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(base) + e;
    if (vec) {
      const uint2 u = *reinterpret_cast<const uint2*>(q);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
      out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) out[k] = k < cnt ? __bfloat162float(q[k]) : 0.f;
    }
  } else {
    const __half* q = static_cast<const __half*>(base) + e;
    if (vec) {
      const uint2 u = *reinterpret_cast<const uint2*>(q);
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
      out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) out[k] = k < cnt ? __half2float(q[k]) : 0.f;
    }
  }
}

__global__ void __launch_bounds__(256, 3) grad_prologue_kernel(PrologueArgs a) {
  __shared__ float t_hi[kTile][kWide + 1];
  __shared__ float t_lo[kTile][kWide + 1];
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_src = a.num_grad_peers > 0 ? a.num_grad_peers : 1;
  const bool peer = a.num_grad_peers > 0;

  for (int t = blockIdx.x; t < a.num_tiles; t += gridDim.x) {
    const TileRef ref = a.tiles[t];
    const BlockDesc& b = a.blocks[ref.block];
    const float* const* srcs = a.grad_ptrs + static_cast<long long>(b.grad_slot) * n_src;
    const int i0 = ref.ti * kTile, j0 = ref.tj * kWide;
    const int j = j0 + 4 * lane;
    const int cnt = b.n - j < 4 ? b.n - j : 4;  // valid columns of this lane's group (<= 0: none)
    const bool want_t = b.gt_hi != nullptr;
    const bool has_m1 = b.m1 != nullptr, has_v = a.graft_kind == kGraftAdaGrad && b.v != nullptr;
    const bool l2 = a.l2_weight_decay != 0.f, graft = a.graft_kind != kGraftNone && b.norms != nullptr;
    bool vec = ((b.n | b.param_pitch | b.grad_offset) & 3) == 0 && aligned16(b.param) && aligned16(b.m1) && aligned16(b.v);
    for (int r = 0; r < n_src; ++r) vec = vec && aligned16(srcs[r]);

    // ---- all loads of the tile first (4 rows x up to 4 arrays in flight per thread)
    float g[4][4], mo[4][4], vo[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + warp + 8 * r;
      const bool on = i < b.m && cnt > 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) g[r][k] = mo[r][k] = vo[r][k] = 0.f;
      if (!on) continue;
      const long long e = static_cast<long long>(i) * b.n + j;
      const long long pe = static_cast<long long>(i) * b.param_pitch + j;
      if (peer) {
        // Fixed rank order keeps the sum identical on every owner.
        for (int s = 0; s < n_src; ++s) {
          float part[4];
          load4<true>(part, srcs[s] + b.grad_offset + pe, vec, cnt);
#pragma unroll
          for (int k = 0; k < 4; ++k) g[r][k] += part[k];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) g[r][k] *= a.grad_scale;
      } else {
        load4<false>(g[r], srcs[0] + b.grad_offset + pe, vec, cnt);
      }
      if (l2) {
        float w[4];
        load4<false>(w, b.param + pe, vec, cnt);
#pragma unroll
        for (int k = 0; k < 4; ++k) g[r][k] += a.l2_weight_decay * w[k];
      }
      if (has_m1) load4<false>(mo[r], b.m1 + e, vec, cnt);
      if (has_v) load4<false>(vo[r], b.v + e, vec, cnt);
    }

    // ---- compute and store
    float sq = 0.f, psq = 0.f;
    const bool identity_p = b.aux == 2;  // no dim is preconditioned: the direction is the filtered gradient
    bool bad = false;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int li = warp + 8 * r;
      const int i = i0 + li;
      const bool on = i < b.m && cnt > 0;
      float hi[4], lo[4], fh[4], fl[4], mn[4], vn[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gk = g[r][k];
        const bool live = on && k < cnt;
        bad |= live && !isfinite(gk);
        if (a.write_split) {
          hi[k] = tf32_round(gk);
          lo[k] = gk - hi[k];
        } else {
          hi[k] = gk;
          lo[k] = 0.f;
        }
        // Filtered gradient: EMA with beta1; the applied estimate uses beta3 on the old EMA.
        float f = gk;
        mn[k] = 0.f;
        if (has_m1) {
          mn[k] = lerpf(mo[r][k], gk, 1.f - a.beta1);
          f = (a.beta3 != a.beta1) ? lerpf(mo[r][k], gk, 1.f - a.beta3) : mn[k];
          f = f / a.bias_correction1;
        }
        if (a.write_split) {
          fh[k] = tf32_round(f);
          fl[k] = f - fh[k];
        } else {
          fh[k] = f;
          fl[k] = 0.f;
        }
        vn[k] = 0.f;
        if (graft) {
          if (has_v) vn[k] = a.graft_beta2 * vo[r][k] + a.graft_weight * gk * gk;
          const float gd = graft_direction(f, vn[k], a.graft_kind, a.graft_bias_correction2, a.graft_epsilon);
          if (live) sq += gd * gd;
        }
        if (identity_p && live) psq += f * f;
        if (identity_p) mo[r][k] = f;  // the loaded EMA has been consumed: reuse its registers
        if (!live) hi[k] = lo[k] = fh[k] = fl[k] = 0.f;
      }
      if (on) {
        const long long e = static_cast<long long>(i) * b.n + j;
        if (identity_p) store4(b.p + e, mo[r], vec, cnt);
        const long long o = static_cast<long long>(i) * b.n_pad + j;  // n_pad % 4 == 0: always 16-byte stores
        if (b.g_hi != nullptr) {
          store4(b.g_hi + o, hi, true, 4);
          if (a.write_split) store4(b.g_lo + o, lo, true, 4);
        }
        if (b.f_hi != nullptr) {
          store4(b.f_hi + o, fh, true, 4);
          if (a.write_split) store4(b.f_lo + o, fl, true, 4);
        }
        if (has_m1) store4(b.m1 + e, mn, vec, cnt);
        if (has_v) store4(b.v + e, vn, vec, cnt);
      }
      if (want_t) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          t_hi[li][4 * lane + k] = hi[k];
          t_lo[li][4 * lane + k] = lo[k];
        }
      }
    }
    if (want_t) {
      __syncthreads();
      // Transposed store: row jj of G^T holds 32 consecutive source rows = 8 float4.
      const int ii = 4 * (threadIdx.x & 7);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int lj = (threadIdx.x >> 3) + 32 * r;
        const int jj = j0 + lj;
        if (jj < b.n && i0 + ii < b.m) {
          const long long o = static_cast<long long>(jj) * b.m_pad + i0 + ii;  // m_pad % 4 == 0
          const float h[4] = {t_hi[ii][lj], t_hi[ii + 1][lj], t_hi[ii + 2][lj], t_hi[ii + 3][lj]};
          store4(b.gt_hi + o, h, true, 4);
          if (a.write_split) {
            const float l[4] = {t_lo[ii][lj], t_lo[ii + 1][lj], t_lo[ii + 2][lj], t_lo[ii + 3][lj]};
            store4(b.gt_lo + o, l, true, 4);
          }
        }
      }
    }
    if (graft) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (lane == 0) red[warp] = sq;
    }
    if (bad) atomicOr(a.status, 2);
    __syncthreads();
    if (graft && threadIdx.x == 0) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += red[w];
      if (s != 0.f) atomicAdd(&b.norms[0], s);
    }
    __syncthreads();
    if (identity_p && b.norms != nullptr) {  // ||P||^2, which the last preconditioner GEMM reduces otherwise
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) psq += __shfl_xor_sync(0xffffffffu, psq, o);
      if (lane == 0) red[warp] = psq;
      __syncthreads();
      if (threadIdx.x == 0) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += red[w];
        if (s != 0.f) atomicAdd(&b.norms[1], s);
      }
      __syncthreads();
    }
  }
}

// kPlain: no grafting-only step, primal averaging or classic momentum (the common configuration):
// only the direction and the parameter are held per element, which keeps the register count low
// enough for four resident CTAs per SM.
template <bool kPlain>
__global__ void __launch_bounds__(256, kPlain ? 3 : 2) direction_epilogue_kernel(EpilogueArgs a) {
  const float lr = *a.lr;
  float mu_x = 0.f, mu_y = 0.f;
  if (a.primal_averaging) {
    mu_x = *a.mu_x;
    mu_y = *a.mu_y;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t = blockIdx.x; t < a.num_tiles; t += gridDim.x) {
    const TileRef ref = a.tiles[t];
    const BlockDesc& b = a.blocks[ref.block];
    const int i0 = ref.ti * kTile, j = ref.tj * kWide + 4 * lane;
    const int cnt = b.n - j < 4 ? b.n - j : 4;
    if (cnt <= 0 || b.aux == 1) continue;
    float scale = 1.f;
    if (!a.graft_only && a.graft_kind != kGraftNone) scale = sqrtf(b.norms[0]) / (sqrtf(b.norms[1]) + 1e-16f);
    const bool has_v = a.graft_kind == kGraftAdaGrad;
    bool vec = ((b.n | b.param_pitch) & 3) == 0 && aligned16(b.param) && aligned16(b.p) && aligned16(b.v) &&
               aligned16(b.mom) && aligned16(b.z) && aligned16(b.send);
    for (int r = 0; r < a.num_push_peers; ++r) vec = vec && ((a.peer_base[r] + b.slot_offset) & 15) == 0;

    constexpr int kAux = kPlain ? 1 : 4;
    float p[4][4], w[4][4], aux[kAux][4], zz[kAux][4], mm[kAux][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + warp + 8 * r;
      if (i >= b.m) continue;
      const long long e = static_cast<long long>(i) * b.n + j;
      const long long pe = static_cast<long long>(i) * b.param_pitch + j;
      if constexpr (kPlain) {
        load4<false>(p[r], b.p + e, vec, cnt);
        load4<false>(w[r], b.param + pe, vec, cnt);
        continue;
      }
      if (a.graft_only) {
        const long long o = static_cast<long long>(i) * b.n_pad + j;
        load4<false>(p[r], b.f_hi + o, true, 4);
        if (a.split_input) {
          float l[4];
          load4<false>(l, b.f_lo + o, true, 4);
#pragma unroll
          for (int k = 0; k < 4; ++k) p[r][k] += l[k];
        }
        if (has_v) load4<false>(aux[r % kAux], b.v + e, vec, cnt);
      } else {
        load4<false>(p[r], b.p + e, vec, cnt);
      }
      load4<false>(w[r], b.param + pe, vec, cnt);
      if (a.primal_averaging) load4<false>(zz[r % kAux], b.z + e, vec, cnt);
      if (a.classic_momentum) load4<false>(mm[r % kAux], b.mom + e, vec, cnt);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + warp + 8 * r;
      if (i >= b.m) continue;
      const long long e = static_cast<long long>(i) * b.n + j;
      const long long pe = static_cast<long long>(i) * b.param_pitch + j;
      float out[4], znew[4], mnew[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float d;
        if (!kPlain && a.graft_only) {
          d = graft_direction(p[r][k], has_v ? aux[r % kAux][k] : 0.f, a.graft_kind, a.graft_bias_correction2,
                              a.graft_epsilon);
        } else {
          d = p[r][k] * scale;
        }
        const float wk = w[r][k];
        float z = 0.f;
        if (!kPlain && a.primal_averaging) {
          z = zz[r % kAux][k];
          if (a.wd_alpha != 0.f) z *= 1.f - lr * a.wd_alpha;
        } else if (a.wd_alpha != 0.f) {
          d += a.wd_alpha * wk;
        }
        mnew[k] = 0.f;
        if (!kPlain && a.classic_momentum) {
          const float mo = a.momentum * mm[r % kAux][k] + (1.f - a.dampening) * d;
          mnew[k] = mo;
          d = a.nesterov ? (1.f - a.dampening) * d + a.momentum * mo : mo;
        }
        d *= -lr;
        znew[k] = 0.f;
        if (!kPlain && a.primal_averaging) {
          const float gap = z - wk;
          znew[k] = z + d;
          d = (1.f - mu_x * mu_y) * d + (1.f - mu_x) * gap;
        }
        out[k] = d;
      }
      if (!kPlain && a.classic_momentum) store4(b.mom + e, mnew, vec, cnt);
      if (!kPlain && a.primal_averaging) store4(b.z + e, znew, vec, cnt);
      if (a.send_params && (a.num_push_peers > 0 || b.send != nullptr)) {
#pragma unroll
        for (int k = 0; k < 4; ++k) out[k] += w[r][k];
      }
      if (a.num_push_peers > 0) {
        for (int s = 0; s < a.num_push_peers; ++s)
          store_send4(reinterpret_cast<void*>(a.peer_base[s] + b.slot_offset), e, out, a.send_dtype, vec, cnt);
      } else if (b.send != nullptr) {
        store_send4(b.send, e, out, a.send_dtype, vec, cnt);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) out[k] += w[r][k];
        store4(b.param + pe, out, vec, cnt);
      }
    }
  }
}

// Every rank applies every block's gathered search direction: param += cast(slot).
__global__ void __launch_bounds__(256) gathered_apply_kernel(const BlockDesc* __restrict__ blocks,
                                                             const TileRef* __restrict__ tiles, int num_tiles,
                                                             int dtype, const float* __restrict__ lr_ptr,
                                                             float wd_alpha, int copy_params,
                                                             const int* __restrict__ status) {
  // A producer of the gather buffer gave up on a bounded wait (GEMM pipeline, peer barrier): the
  // slots may hold partial or stale directions, so the parameters are left as they are and the
  // host raises when it reads the status word.
  if (status != nullptr && (*status & (kErrGemmTimeout | kErrPeerTimeout)) != 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool scaled = lr_ptr != nullptr;
  const float lr = scaled ? *lr_ptr : 0.f;
  for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const TileRef ref = tiles[t];
    const BlockDesc& b = blocks[ref.block];
    const int i0 = ref.ti * kTile, j = ref.tj * kWide + 4 * lane;
    const int cnt = b.n - j < 4 ? b.n - j : 4;
    if (cnt <= 0) continue;
    const bool vec = ((b.n | b.param_pitch) & 3) == 0 && aligned16(b.param) && aligned16(b.send);
    float d[4][4], w[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + warp + 8 * r;
      if (i >= b.m) continue;
      load_recv4(d[r], b.send, static_cast<long long>(i) * b.n + j, dtype, vec, cnt);
      load4<false>(w[r], b.param + static_cast<long long>(i) * b.param_pitch + j, vec, cnt);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + warp + 8 * r;
      if (i >= b.m) continue;
      if (copy_params) {
#pragma unroll
        for (int k = 0; k < 4; ++k) w[r][k] = d[r][k];
      } else if (scaled) {
        const float sc = b.norms != nullptr ? b.norms[0] : 1.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) w[r][k] -= lr * (sc * d[r][k] + wd_alpha * w[r][k]);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) w[r][k] += d[r][k];
      }
      store4(b.param + static_cast<long long>(i) * b.param_pitch + j, w[r], vec, cnt);
    }
  }
}

__global__ void __launch_bounds__(256) eig_scale_kernel(const BlockDesc* __restrict__ blocks,
                                                        const TileRef* __restrict__ tiles, int num_tiles, float bc2,
                                                        float inv_root, float eps, int write_split) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const TileRef ref = tiles[t];
    const BlockDesc& b = blocks[ref.block];
    const int i0 = ref.ti * kTile, j = ref.tj * kWide + 4 * lane;
    const int cnt = b.n - j < 4 ? b.n - j : 4;
    // The auxiliary descriptor of an order-3 block (its second 2-D view) carries no state: ev and p
    // are null there.
    if (cnt <= 0 || b.aux == 1 || b.ev == nullptr) continue;
    const bool vec = (b.n & 3) == 0 && aligned16(b.ev) && aligned16(b.p);
    float ev[4][4], p[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + warp + 8 * r;
      if (i >= b.m) continue;
      const long long e = static_cast<long long>(i) * b.n + j;
      load4<false>(ev[r], b.ev + e, vec, cnt);
      load4<false>(p[r], b.p + e, vec, cnt);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + warp + 8 * r;
      if (i >= b.m) continue;
      float hi[4], lo[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        // Roots 2 and 4 (the defaults) avoid the general power function, which made the kernel
        // instruction bound.
        const float base = ev[r][k] / bc2;
        const float pw = inv_root == 0.5f ? sqrtf(base) : inv_root == 0.25f ? sqrtf(sqrtf(base)) : powf(base, inv_root);
        const float s = k < cnt ? p[r][k] / (pw + eps) : 0.f;
        hi[k] = write_split ? tf32_round(s) : s;
        lo[k] = s - hi[k];
      }
      const long long o = static_cast<long long>(i) * b.n_pad + j;  // n_pad % 4 == 0
      store4(b.f_hi + o, hi, true, 4);
      if (write_split) store4(b.f_lo + o, lo, true, 4);
    }
  }
}

__global__ void __launch_bounds__(256) mode_switch_kernel(const BlockDesc* __restrict__ blocks,
                                                          const TileRef* __restrict__ tiles, int num_tiles, float coeff,
                                                          int send_dtype) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const TileRef ref = tiles[t];
    const BlockDesc& b = blocks[ref.block];
    const int i0 = ref.ti * kTile, j = ref.tj * kWide + 4 * lane;
    const int cnt = b.n - j < 4 ? b.n - j : 4;
    if (cnt <= 0) continue;
    const bool vec = ((b.n | b.param_pitch) & 3) == 0 && aligned16(b.param) && aligned16(b.z) && aligned16(b.send);
    float w[4][4], z[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + warp + 8 * r;
      if (i >= b.m) continue;
      load4<false>(w[r], b.param + static_cast<long long>(i) * b.param_pitch + j, vec, cnt);
      load4<false>(z[r], b.z + static_cast<long long>(i) * b.n + j, vec, cnt);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + warp + 8 * r;
      if (i >= b.m) continue;
      float delta[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) delta[k] = (z[r][k] - w[r][k]) * coeff;
      if (b.send != nullptr) {
        store_send4(b.send, static_cast<long long>(i) * b.n + j, delta, send_dtype, vec, cnt);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) delta[k] += w[r][k];
        store4(b.param + static_cast<long long>(i) * b.param_pitch + j, delta, vec, cnt);
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
  const int cap = sm_count() * 8;
  return num_tiles < cap ? num_tiles : cap;
}

}  // namespace

void launch_grad_prologue(const PrologueArgs& args, cudaStream_t stream) {
  if (args.num_tiles <= 0) return;
  grad_prologue_kernel<<<grid_for(args.num_tiles), 256, 0, stream>>>(args);
}

void launch_direction_epilogue(const EpilogueArgs& args, cudaStream_t stream) {
  if (args.num_tiles <= 0) return;
  if (!args.graft_only && !args.primal_averaging && !args.classic_momentum) {
    direction_epilogue_kernel<true><<<grid_for(args.num_tiles), 256, 0, stream>>>(args);
  } else {
    direction_epilogue_kernel<false><<<grid_for(args.num_tiles), 256, 0, stream>>>(args);
  }
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

void launch_gathered_apply(const BlockDesc* blocks, const TileRef* tiles, int num_tiles, int dtype, const float* lr,
                           float wd_alpha, bool copy_params, const int* status, cudaStream_t stream) {
  if (num_tiles <= 0) return;
  gathered_apply_kernel<<<grid_for(num_tiles), 256, 0, stream>>>(blocks, tiles, num_tiles, dtype, lr, wd_alpha,
                                                                 copy_params ? 1 : 0, status);
}

}  // namespace ob200
