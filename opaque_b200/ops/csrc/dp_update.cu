// DP-specific bandwidth-bound kernels for sm_100a:
//   * counter-based Philox Gaussian noise added in place,
//   * per-example squared norms and the clip-weighted sum of materialised per-example
//     gradients, scattered to the owning rank's shard (reduce-scatter by peer reductions),
//   * the fused shard step: [Philox Gaussian | DP-FTRL BLT / banded correlated noise] +
//     AdamW with noise bias correction on fp32 master weights + bf16 parameter write-back
//     into EVERY rank's parameter buffer (all-gather by peer stores),
//   * a flag barrier between ranks with a bounded wait.
// Noise is keyed by (seed, global coordinate index): whichever rank owns a coordinate draws
// the same value, so a run is reproducible across 1/2/4/8-GPU layouts and every coordinate
// receives noise exactly once.
#include <string.h>

#include "common.cuh"
#include "api.h"

namespace ob {

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
philox_normal_add_kernel(T* __restrict__ x, long long n, unsigned long long seed, long long offset, float std,
                         unsigned stream_id) {
  // thread handles the aligned 4-block of global coordinates [4b, 4b+4) clipped to [offset, offset+n)
  const long long first_blk = offset >> 2;
  const long long last_blk = (offset + n - 1) >> 2;
  for (long long b = first_blk + blockIdx.x * 256LL + threadIdx.x; b <= last_blk; b += gridDim.x * 256LL) {
    const float4 z = philox_normal4(seed, static_cast<uint64_t>(b), stream_id);
    const float zz[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long g = b * 4 + j - offset;
      if (g >= 0 && g < n) x[g] = static_cast<T>(static_cast<float>(x[g]) + std * zz[j]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Per-example squared L2 norm of materialised gradients G [E, P] (fp32): norm2[e] += sum_p G[e,p]^2.
__global__ void __launch_bounds__(256)
rows_sumsq_kernel(const float* __restrict__ g, long long P, long long ld, float* __restrict__ norm2) {
  __shared__ float red[8];
  const int e = blockIdx.y;
  const float* row = g + static_cast<long long>(e) * ld;
  float acc = 0.f;
  const long long nv = P >> 2;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nv; i += gridDim.x * 256LL) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(row) + i);
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (long long i = (nv << 2) + threadIdx.x; i < P; i += 256) acc += row[i] * row[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffu, t, o);
    if (threadIdx.x == 0) atomicAdd(norm2 + e, t);
  }
}

// out[flat_offset + p] += sum_e c[e] * G[e, p]; with a peer table the destination is the owner's shard.
__global__ void __launch_bounds__(256)
clip_weighted_sum_kernel(const float* __restrict__ g, const float* __restrict__ c, int E, long long P, long long ld,
                         float* out, float* const* peer_out, long long shard_elems, long long flat_offset) {
  const long long nv = P >> 2;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nv; i += gridDim.x * 256LL) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int e = 0; e < E; ++e) {
      const float w = __ldg(c + e);
      if (w == 0.f) continue;            // factor 0 = example dropped (non-finite norm): skip it, 0 * NaN is NaN
      const float4 v = __ldg(reinterpret_cast<const float4*>(g + static_cast<long long>(e) * ld) + i);
      acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
    }
    const long long idx = flat_offset + (i << 2);
    float* dst;
    if (peer_out) {
      const long long owner = idx / shard_elems;
      dst = peer_out[owner] + (idx - owner * shard_elems);
    } else {
      dst = out + idx;
    }
    red_add_v4(dst, acc);
  }
}

// Step-end reduce-scatter of a locally accumulated gradient: every rank adds its full-length fp32 buffer into the
// owners' shards (one 16-byte reduction per four coordinates, 7/8 of them over NVLink at 8 GPUs) and clears it.
// Blocks that are all zero (frozen ranges, padding) send nothing.
__global__ void __launch_bounds__(256)
push_grad_kernel(float* __restrict__ local, long long total, float* const* peer_out, long long shard_elems,
                 const int* status) {
  // a bounded wait that ran out earlier leaves the job in an unknown state: keep the accumulated gradient where it is
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  const long long nv = total >> 2;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nv; i += gridDim.x * 256LL) {
    float4* src = reinterpret_cast<float4*>(local) + i;
    const float4 v = *src;
    if (v.x == 0.f && v.y == 0.f && v.z == 0.f && v.w == 0.f) continue;
    const long long idx = i << 2;
    const long long owner = idx / shard_elems;
    red_add_v4(peer_out[owner] + (idx - owner * shard_elems), v);
    *src = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Clip-weighted embedding gradient: for every token row t, flat[out_offset + ids[t]*D + d] += s[t] * G[t, d].
__global__ void __launch_bounds__(256)
embedding_wgrad_kernel(const __nv_bfloat16* __restrict__ g, const long long* __restrict__ ids,
                       const float* __restrict__ row_scale, long long rows, int D, long long ldg, float* out,
                       float* const* peer_out, long long shard_elems, long long flat_offset) {
  const int vec_per_row = D >> 2;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += gridDim.x * 256LL) {
    const long long t = i / vec_per_row;
    const int d = static_cast<int>(i % vec_per_row) << 2;
    const float s = row_scale ? __ldg(row_scale + t) : 1.f;
    if (s == 0.f) continue;
    const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(g + t * ldg + d);
    const float2 a = __bfloat1622float2(src[0]), b = __bfloat1622float2(src[1]);
    const long long idx = flat_offset + __ldg(ids + t) * D + d;
    float* dst;
    if (peer_out) {
      const long long owner = idx / shard_elems;
      dst = peer_out[owner] + (idx - owner * shard_elems);
    } else {
      dst = out + idx;
    }
    red_add_v4(dst, make_float4(s * a.x, s * a.y, s * b.x, s * b.y));
  }
}

// ---------------------------------------------------------------------------------------------
// Fused shard step.
// Longest correlated-noise recurrence the fused step handles: 63 history buffers for the ring modes (a banded C or a
// banded inverse with up to 64 coefficients), 32 (scale, decay) pairs for BLT.  Up to 8 buffers run fully unrolled.
constexpr int OB_FTRL_MAX_COEF = 64;

struct ShardStepParams {
  float* grad;             // [n] fp32 sum of clipped gradients for this shard; zeroed on exit (unused when peer_grad is set)
  const float* const* peer_grad;   // pull form: [world] full-length fp32 accumulation buffers, one per rank, or nullptr.  The
                           // shard's gradient is then the sum over ranks r = 0..world-1, IN THAT ORDER, of
                           // peer_grad[r][global_offset + i], read here through peer pointers: the reduce-scatter happens
                           // inside this kernel, needs no atomics, and gives the same bits whatever the arrival order.
                           // Nothing is cleared here: every rank clears its own buffer after the closing barrier.
  float* master;           // [n] fp32 parameters
  float* m;                // [n]
  float* v;                // [n]
  float* ftrl_state;       // [nbuf, n] fp32 correlated-noise state, or nullptr
  __nv_bfloat16* const* peer_params;  // [world] bf16 parameter buffers (full length), or nullptr
  __nv_bfloat16* local_params;        // used when peer_params == nullptr
  float* noisy_out;        // optional [n]: the privatised mean gradient (for tests / logging)
  long long n;
  long long global_offset; // flat index of this shard's first coordinate
  int world;
  unsigned long long seed; // Philox key of this step
  float noise_std;         // sigma * C (before normalisation)
  float inv_normalize;     // 1 / normalize_by
  // DP-FTRL: mode 0 = iid Gaussian, 1 = BLT inverse (scale s_j, decay d_j), 2 = banded inverse (IIR),
  // 3 = FIR over past raw draws
  int ftrl_mode, nbuf, ring_head;
  float coef[OB_FTRL_MAX_COEF];   // BLT: s_0..s_{nbuf-1}, d_0..d_{nbuf-1}; banded / FIR: c_0, c_1..c_{nbuf}
  // AdamW-BC
  float lr, b1, b2, eps, wd, bc1, bc2, phi_hat;
  int decoupled_wd, skip_update;
  int opt_mode;            // 0: Adam family (AdamW / AdamW-BC / Adam), 1: SGD with momentum b1 (PyTorch semantics), 2: Lion (b1, b2)
  int nesterov;            // SGD only
  const int* status;       // non-zero: a bounded wait expired earlier in this step; the kernel does nothing
};

__device__ __forceinline__ void ld8(const float* src, float* dst) {
  *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
  *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
}
__device__ __forceinline__ void st8(float* dst, const float* src) {
  *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
  *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
}

// Correlated-noise update for 8 consecutive coordinates with 32-byte vector accesses to the state buffers.
// z: this step's raw N(0,1) draws; x: the correlated noise to add (row t of C^{-1} Z).
__device__ __forceinline__ void ftrl_apply8(const ShardStepParams& p, long long base, const float* z, float* x) {
  float* st = p.ftrl_state + base;
  if (p.ftrl_mode == 1) {
    // buffered-linear-Toeplitz C:  x = z - sum_b s_b S_b ;  S_b <- d_b S_b + x   (first four buffers stay in registers)
    float keep[4][8], corr[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) corr[j] = 0.f;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      if (b < p.nbuf) {
        float t[8];
        ld8(st + b * p.n, t);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          corr[j] += p.coef[b] * t[j];
          if (b < 4) keep[b][j] = t[j];
        }
      }
    }
    for (int b = 8; b < p.nbuf; ++b) {          // beyond the unrolled eight: same recurrence, buffers re-read below
      float t[8];
      ld8(st + b * p.n, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) corr[j] += p.coef[b] * t[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = z[j] - corr[j];
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      if (b < p.nbuf) {
        float t[8];
        if (b < 4) {
#pragma unroll
          for (int j = 0; j < 8; ++j) t[j] = keep[b][j];
        } else {
          ld8(st + b * p.n, t);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = p.coef[p.nbuf + b] * t[j] + x[j];
        st8(st + b * p.n, t);
      }
    }
    for (int b = 8; b < p.nbuf; ++b) {
      float t[8];
      ld8(st + b * p.n, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) t[j] = p.coef[p.nbuf + b] * t[j] + x[j];
      st8(st + b * p.n, t);
    }
  } else {
    // ring of the previous nbuf values: mode 2 keeps outputs (banded C, IIR), mode 3 keeps raw draws (FIR)
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = (p.ftrl_mode == 3) ? p.coef[0] * z[j] : 0.f;
#pragma unroll
    for (int b = 1; b <= 8; ++b) {
      if (b <= p.nbuf) {
        int slot = p.ring_head - b;
        if (slot < 0) slot += p.nbuf;
        float t[8];
        ld8(st + slot * p.n, t);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += p.coef[b] * t[j];
      }
    }
    for (int b = 9; b <= p.nbuf; ++b) {         // longer histories: a plain loop over the ring
      int slot = p.ring_head - b;
      if (slot < 0) slot += p.nbuf;
      float t[8];
      ld8(st + slot * p.n, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += p.coef[b] * t[j];
    }
    if (p.ftrl_mode == 2) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = (z[j] - acc[j]) / p.coef[0];
      st8(st + p.ring_head * p.n, x);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = acc[j];
      st8(st + p.ring_head * p.n, z);
    }
  }
}

// Pull form of the gradient read: this shard's 8 coordinates from every rank's accumulation buffer, summed in rank
// order.  Four ranks' 32-byte loads are in flight per thread before the first add (more would spill registers).
__device__ __forceinline__ void pull_grad8(const ShardStepParams& p, long long base, float* g8) {
#pragma unroll
  for (int j = 0; j < 8; ++j) g8[j] = 0.f;
  for (int r0 = 0; r0 < p.world; r0 += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (r0 + r < p.world) {
        const float4* src = reinterpret_cast<const float4*>(p.peer_grad[r0 + r] + p.global_offset + base);
        a[r] = __ldcg(src);
        b[r] = __ldcg(src + 1);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (r0 + r < p.world) {
        g8[0] += a[r].x; g8[1] += a[r].y; g8[2] += a[r].z; g8[3] += a[r].w;
        g8[4] += b[r].x; g8[5] += b[r].y; g8[6] += b[r].z; g8[7] += b[r].w;
      }
    }
  }
}

// PULL selects the gradient source at compile time, so the ordinary form keeps its register allocation.  FTRL = false is
// the iid-noise step (DP-SGD): without the correlated-noise state it fits three blocks per SM, which this latency-bound
// kernel (Philox rounds, accurate log / sincos / sqrt / divisions in a dependent chain) turns into bandwidth.
template <bool PULL, bool FTRL>
__global__ void __launch_bounds__(256, FTRL ? 2 : 3)
shard_step_kernel(const ShardStepParams p) {
  // The gradient barrier before this kernel may have given up (status != 0): the shard is then not fully reduced, and
  // adding noise to it, stepping and clearing it would release and apply a partial sum.  Leave every buffer untouched;
  // the host reads the status word after the step and raises.
  if (p.status != nullptr && *reinterpret_cast<const volatile int*>(p.status) != 0) return;
  // each thread owns 8 consecutive coordinates (two Philox blocks, one 16-byte bf16 store per peer)
  const long long nv = (p.n + 7) >> 3;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nv; i += gridDim.x * 256LL) {
    const long long base = i << 3;
    const bool full = base + 8 <= p.n;
    float z[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (p.noise_std != 0.f) {
      const uint64_t blk = static_cast<uint64_t>((p.global_offset + base) >> 2);
      const float4 r0 = philox_normal4(p.seed, blk, 0u), r1 = philox_normal4(p.seed, blk + 1, 0u);
      z[0] = r0.x; z[1] = r0.y; z[2] = r0.z; z[3] = r0.w;
      z[4] = r1.x; z[5] = r1.y; z[6] = r1.z; z[7] = r1.w;
    }
    float g8[8], w8[8], m8[8], v8[8];
    if (full) {
      if (PULL) {
        pull_grad8(p, base, g8);
      } else {
        *reinterpret_cast<float4*>(g8) = *reinterpret_cast<const float4*>(p.grad + base);
        *reinterpret_cast<float4*>(g8 + 4) = *reinterpret_cast<const float4*>(p.grad + base + 4);
      }
      if (!p.skip_update) {
        *reinterpret_cast<float4*>(w8) = *reinterpret_cast<const float4*>(p.master + base);
        *reinterpret_cast<float4*>(w8 + 4) = *reinterpret_cast<const float4*>(p.master + base + 4);
        *reinterpret_cast<float4*>(m8) = *reinterpret_cast<const float4*>(p.m + base);
        *reinterpret_cast<float4*>(m8 + 4) = *reinterpret_cast<const float4*>(p.m + base + 4);
        *reinterpret_cast<float4*>(v8) = *reinterpret_cast<const float4*>(p.v + base);
        *reinterpret_cast<float4*>(v8 + 4) = *reinterpret_cast<const float4*>(p.v + base + 4);
      }
    } else {
      for (int j = 0; j < 8; ++j) {
        const long long k = base + j;
        const bool in = k < p.n;
        float gk = 0.f;
        if (in && PULL) {
          for (int r = 0; r < p.world; ++r) gk += __ldcg(p.peer_grad[r] + p.global_offset + k);
        } else if (in) {
          gk = p.grad[k];
        }
        g8[j] = gk;
        w8[j] = (in && !p.skip_update) ? p.master[k] : 0.f;
        m8[j] = (in && !p.skip_update) ? p.m[k] : 0.f;
        v8[j] = (in && !p.skip_update) ? p.v[k] : 0.f;
      }
    }
    float out8[8];
    float x8[8];
    const bool vec_ftrl = FTRL && full && p.ftrl_mode != 0 && ((p.n & 3) == 0);
    if (vec_ftrl) ftrl_apply8(p, base, z, x8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long k = base + j;
      float x = vec_ftrl ? x8[j] : z[j];
      if (FTRL && k < p.n && !vec_ftrl) {
        if (p.ftrl_mode == 1) {
          // row t of C^{-1} Z for a buffered-linear-Toeplitz C:  x = z - sum_b s_b S_b ;  S_b <- d_b S_b + x
          float corr = 0.f;
          for (int b = 0; b < p.nbuf; ++b) corr += p.coef[b] * p.ftrl_state[b * p.n + k];
          x = z[j] - corr;
          for (int b = 0; b < p.nbuf; ++b)
            p.ftrl_state[b * p.n + k] = p.coef[p.nbuf + b] * p.ftrl_state[b * p.n + k] + x;
        } else if (p.ftrl_mode == 2) {
          // banded Toeplitz C with c_0..c_nbuf:  x_t = (z_t - sum_{b>=1} c_b x_{t-b}) / c_0; the history is a
          // ring whose slot (ring_head - b) mod nbuf holds x_{t-b}
          float corr = 0.f;
          for (int b = 1; b <= p.nbuf; ++b) {
            int slot = p.ring_head - b;
            if (slot < 0) slot += p.nbuf;
            corr += p.coef[b] * p.ftrl_state[slot * p.n + k];
          }
          x = (z[j] - corr) / p.coef[0];
          p.ftrl_state[p.ring_head * p.n + k] = x;
        } else if (p.ftrl_mode == 3) {
          // FIR on the raw noise (banded INVERSE factor, lambda-CGD):  x_t = c_0 z_t + sum_{b>=1} c_b z_{t-b};
          // the ring keeps the previous nbuf raw draws
          float acc = p.coef[0] * z[j];
          for (int b = 1; b <= p.nbuf; ++b) {
            int slot = p.ring_head - b;
            if (slot < 0) slot += p.nbuf;
            acc += p.coef[b] * p.ftrl_state[slot * p.n + k];
          }
          p.ftrl_state[p.ring_head * p.n + k] = z[j];
          x = acc;
        }
      }
      const float g = (g8[j] + p.noise_std * x) * p.inv_normalize;
      out8[j] = g;
      float w = w8[j];
      float ge = g;
      if (!p.decoupled_wd) ge += p.wd * w;
      float u;
      if (p.opt_mode == 0) {
        const float m = p.b1 * m8[j] + (1.f - p.b1) * ge;
        const float v = p.b2 * v8[j] + (1.f - p.b2) * ge * ge;
        m8[j] = m;
        v8[j] = v;
        float vh = v / p.bc2;
        const float corrected = vh - p.phi_hat;
        if (corrected > 0.f) vh = corrected;
        u = (m / p.bc1) / (sqrtf(vh) + p.eps);
      } else if (p.opt_mode == 1) {
        // buf <- mu * buf + g (a zero buffer makes the first step buf = g); Nesterov looks ahead by one more mu * buf
        const float m = p.b1 * m8[j] + ge;
        m8[j] = m;
        u = p.nesterov ? ge + p.b1 * m : m;
      } else {
        const float c = p.b1 * m8[j] + (1.f - p.b1) * ge;
        u = c > 0.f ? 1.f : (c < 0.f ? -1.f : 0.f);
        m8[j] = p.b2 * m8[j] + (1.f - p.b2) * ge;
      }
      if (p.decoupled_wd) u += p.wd * w;
      w8[j] = w - p.lr * u;
    }
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (full) {
      if (!PULL) {
        *reinterpret_cast<float4*>(p.grad + base) = zero4;
        *reinterpret_cast<float4*>(p.grad + base + 4) = zero4;
      }
      if (p.noisy_out) {
        *reinterpret_cast<float4*>(p.noisy_out + base) = *reinterpret_cast<const float4*>(out8);
        *reinterpret_cast<float4*>(p.noisy_out + base + 4) = *reinterpret_cast<const float4*>(out8 + 4);
      }
      if (!p.skip_update) {
        *reinterpret_cast<float4*>(p.master + base) = *reinterpret_cast<const float4*>(w8);
        *reinterpret_cast<float4*>(p.master + base + 4) = *reinterpret_cast<const float4*>(w8 + 4);
        *reinterpret_cast<float4*>(p.m + base) = *reinterpret_cast<const float4*>(m8);
        *reinterpret_cast<float4*>(p.m + base + 4) = *reinterpret_cast<const float4*>(m8 + 4);
        *reinterpret_cast<float4*>(p.v + base) = *reinterpret_cast<const float4*>(v8);
        *reinterpret_cast<float4*>(p.v + base + 4) = *reinterpret_cast<const float4*>(v8 + 4);
        uint4 packed;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(w8[2 * j], w8[2 * j + 1]);
        if (p.peer_params) {
          for (int r = 0; r < p.world; ++r)
            *reinterpret_cast<uint4*>(p.peer_params[r] + p.global_offset + base) = packed;
        } else if (p.local_params) {
          *reinterpret_cast<uint4*>(p.local_params + p.global_offset + base) = packed;
        }
      }
    } else {
      for (int j = 0; j < 8; ++j) {
        const long long k = base + j;
        if (k >= p.n) break;
        if (!PULL) p.grad[k] = 0.f;
        if (p.noisy_out) p.noisy_out[k] = out8[j];
        if (p.skip_update) continue;
        p.master[k] = w8[j];
        p.m[k] = m8[j];
        p.v[k] = v8[j];
        const __nv_bfloat16 wb = __float2bfloat16_rn(w8[j]);
        if (p.peer_params) {
          for (int r = 0; r < p.world; ++r) p.peer_params[r][p.global_offset + k] = wb;
        } else if (p.local_params) {
          p.local_params[p.global_offset + k] = wb;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Rank barrier over peer memory: write `epoch` into slot [my_rank] of every rank's flag array,
// then wait until all slots of the local array reached `epoch`.  The wait is bounded.
__global__ void peer_barrier_kernel(int* const* peer_flags, int* local_flags, int rank, int world, int epoch,
                                    int* status, unsigned long long budget_ns) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peer_flags[t] + rank), "r"(epoch) : "memory");
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      int seen;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(local_flags + t) : "memory");
      if (seen >= epoch) break;
      if (globaltimer_ns() - t0 > budget_ns) {
        set_error(status, OB_ERR_WAIT_PEER);
        break;
      }
      __nanosleep(200);
    }
  }
}

}  // namespace ob

using namespace ob;
#define OB_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : -21)

static int grid_for(long long work, int sms) {
  long long g = (work + 255) / 256;
  const long long cap = static_cast<long long>(sms) * 8;
  if (g > cap) g = cap;
  return g < 1 ? 1 : static_cast<int>(g);
}

extern "C" int ob_philox_normal_add(void* x, int dtype_code, long long n, unsigned long long seed, long long offset,
                                    float std, unsigned stream_id, int sms, void* stream) {
  if (n <= 0 || std == 0.f) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for((n + 3) / 4 + 1, sms);
  if (dtype_code == 0)
    philox_normal_add_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(x), n, seed, offset, std, stream_id);
  else if (dtype_code == 1)
    philox_normal_add_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<__nv_bfloat16*>(x), n, seed, offset,
                                                                  std, stream_id);
  else
    return -2;
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_rows_sumsq(const float* g, int E, long long P, long long ld, float* norm2, int sms, void* stream) {
  if (E <= 0 || P <= 0) return 0;
  if ((ld & 3) || (reinterpret_cast<uintptr_t>(g) & 15)) return -2;
  long long gx = (P / 4 + 255) / 256;
  const long long cap = (static_cast<long long>(sms) * 8 + E - 1) / E;
  if (gx > cap) gx = cap;
  if (gx < 1) gx = 1;
  dim3 grid(static_cast<unsigned>(gx), E);
  rows_sumsq_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(g, P, ld, norm2);
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_clip_weighted_sum(const float* g, const float* c, int E, long long P, long long ld, float* out,
                                    float* const* peer_out, long long shard_elems, long long flat_offset, int sms,
                                    void* stream) {
  if (E <= 0 || P <= 0) return 0;
  if ((P & 3) || (ld & 3) || (flat_offset & 3) || (peer_out && (shard_elems & 3))) return -2;
  clip_weighted_sum_kernel<<<grid_for(P / 4, sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g, c, E, P, ld, out, peer_out, shard_elems, flat_offset);
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_push_grad(float* local, long long total, float* const* peer_out, long long shard_elems,
                            const int* status, int sms, void* stream) {
  if (total <= 0) return 0;
  if ((total & 3) || (shard_elems & 3) || peer_out == nullptr) return -2;
  push_grad_kernel<<<grid_for(total / 4, sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(local, total, peer_out, shard_elems, status);
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_embedding_wgrad(const void* g, const long long* ids, const float* row_scale, long long rows, int D,
                                  long long ldg, float* out, float* const* peer_out, long long shard_elems,
                                  long long flat_offset, int sms, void* stream) {
  if (rows <= 0) return 0;
  if ((D & 3) || (ldg & 1) || (flat_offset & 3) || (peer_out && (shard_elems & 3))) return -2;
  embedding_wgrad_kernel<<<grid_for(rows * (D / 4), sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(g), ids, row_scale, rows, D, ldg, out, peer_out, shard_elems, flat_offset);
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_shard_step(float* grad, const float* const* peer_grad, float* master, float* m, float* v, float* ftrl_state,
                             void* const* peer_params, void* local_params, float* noisy_out, long long n,
                             long long global_offset, int world, unsigned long long seed, float noise_std,
                             float inv_normalize, int ftrl_mode, int nbuf, int ring_head, const float* coef,
                             int ncoef, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                             float phi_hat, int decoupled_wd, int skip_update, int opt_mode, int nesterov,
                             const int* status, int sms, void* stream) {
  if (n <= 0) return 0;
  if (global_offset & 7) return -2;
  if (grad == nullptr && peer_grad == nullptr) return -2;
  if (ncoef > OB_FTRL_MAX_COEF || nbuf >= OB_FTRL_MAX_COEF) return -3;
  ShardStepParams p;
  p.grad = grad; p.peer_grad = peer_grad; p.master = master; p.m = m; p.v = v; p.ftrl_state = ftrl_state;
  p.peer_params = reinterpret_cast<__nv_bfloat16* const*>(peer_params);
  p.local_params = static_cast<__nv_bfloat16*>(local_params);
  p.noisy_out = noisy_out;
  p.n = n; p.global_offset = global_offset; p.world = world; p.seed = seed;
  p.noise_std = noise_std; p.inv_normalize = inv_normalize;
  p.ftrl_mode = ftrl_mode; p.nbuf = nbuf; p.ring_head = ring_head;
  for (int i = 0; i < OB_FTRL_MAX_COEF; ++i) p.coef[i] = (coef && i < ncoef) ? coef[i] : 0.f;
  p.lr = lr; p.b1 = b1; p.b2 = b2; p.eps = eps; p.wd = wd; p.bc1 = bc1; p.bc2 = bc2; p.phi_hat = phi_hat;
  p.decoupled_wd = decoupled_wd; p.skip_update = skip_update;
  p.opt_mode = opt_mode; p.nesterov = nesterov;
  if (opt_mode < 0 || opt_mode > 2) return -4;
  p.status = status;
  const dim3 grid = grid_for((n + 7) / 8, sms);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool pull = peer_grad != nullptr, ftrl = ftrl_mode != 0;
  if (pull && ftrl) shard_step_kernel<true, true><<<grid, 256, 0, st>>>(p);
  else if (pull) shard_step_kernel<true, false><<<grid, 256, 0, st>>>(p);
  else if (ftrl) shard_step_kernel<false, true><<<grid, 256, 0, st>>>(p);
  else shard_step_kernel<false, false><<<grid, 256, 0, st>>>(p);
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_peer_barrier(int* const* peer_flags, int* local_flags, int rank, int world, int epoch, int* status,
                               double budget_s, void* stream) {
  if (world > 32) return -2;
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      peer_flags, local_flags, rank, world, epoch, status, static_cast<unsigned long long>(budget_s * 1e9));
  return OB_CHECK_LAUNCH();
}

// ---- CUDA IPC helpers (peer memory plumbing; handles travel through torch.distributed) ---------------
extern "C" int ob_ipc_alloc(void** ptr, long long bytes) {
  if (cudaMalloc(ptr, static_cast<size_t>(bytes)) != cudaSuccess) return -30;
  return cudaMemset(*ptr, 0, static_cast<size_t>(bytes)) == cudaSuccess ? 0 : -31;
}
extern "C" int ob_ipc_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -32; }
extern "C" int ob_ipc_get_handle(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return -33;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int ob_ipc_open_handle(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : -34;
}
extern "C" int ob_ipc_close_handle(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -35; }
extern "C" int ob_last_cuda_error(char* buf, int len) {
  const char* s = cudaGetErrorString(cudaGetLastError());
  int i = 0;
  for (; s[i] && i < len - 1; ++i) buf[i] = s[i];
  buf[i] = 0;
  return 0;
}
