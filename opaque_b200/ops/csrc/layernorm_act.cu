// LayerNorm forward / backward with per-example weight and bias gradients, per-example bias-gradient row sums and
// plain (ungated) activations for sm_100a.  These are the bandwidth-bound pieces of a GPT-2-style block under
// per-example clipping: the weight / bias gradients of LayerNorm and the bias gradients of linear layers are small
// enough to materialise per example ([B, H] each), so they are reduced over an example's T token rows by a kernel and
// added straight into that example's row of the per-example gradient buffer.
// bf16 storage, fp32 math, 16-byte vector accesses, one CTA per row for the normalisation passes.
#include "common.cuh"
#include "api.h"

namespace ob {

struct alignas(16) ln_bf16x8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void ln_unpack8(const ln_bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ ln_bf16x8 ln_pack8(const float* f) {
  ln_bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

constexpr int LN_THREADS = 128;

// two simultaneous block-wide sums
__device__ __forceinline__ float2 ln_block_sum2(float a, float b, float2* red) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = make_float2(a, b);
  __syncthreads();
  float2 t = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < LN_THREADS / 32; ++i) {
    t.x += red[i].x;
    t.y += red[i].y;
  }
  return t;
}

__global__ void __launch_bounds__(LN_THREADS)
layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                     const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
                     float* __restrict__ rstd, int H, float eps) {
  __shared__ float2 red[LN_THREADS / 32];
  const long long row = blockIdx.x;
  const ln_bf16x8* xr = reinterpret_cast<const ln_bf16x8*>(x + row * H);
  const int nv = H >> 3;
  float s = 0.f, ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += LN_THREADS) {
    float f[8];
    ln_unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s += f[j];
      ss += f[j] * f[j];
    }
  }
  const float2 t = ln_block_sum2(s, ss, red);
  const float mu = t.x / H;
  const float var = fmaxf(t.y / H - mu * mu, 0.f);
  const float rs = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    mean[row] = mu;
    rstd[row] = rs;
  }
  const ln_bf16x8* wr = reinterpret_cast<const ln_bf16x8*>(w);
  const ln_bf16x8* br = reinterpret_cast<const ln_bf16x8*>(b);
  ln_bf16x8* yr = reinterpret_cast<ln_bf16x8*>(y + row * H);
  for (int i = threadIdx.x; i < nv; i += LN_THREADS) {
    float f[8], g[8], h[8];
    ln_unpack8(xr[i], f);
    ln_unpack8(wr[i], g);
    if (b != nullptr) ln_unpack8(br[i], h);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = (f[j] - mu) * rs * g[j] + (b != nullptr ? h[j] : 0.f);
    yr[i] = ln_pack8(f);
  }
}

__global__ void __launch_bounds__(LN_THREADS)
layernorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean,
                        const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx, int H) {
  __shared__ float2 red[LN_THREADS / 32];
  const long long row = blockIdx.x;
  const ln_bf16x8* dyr = reinterpret_cast<const ln_bf16x8*>(dy + row * H);
  const ln_bf16x8* xr = reinterpret_cast<const ln_bf16x8*>(x + row * H);
  const ln_bf16x8* wr = reinterpret_cast<const ln_bf16x8*>(w);
  ln_bf16x8* dxr = reinterpret_cast<ln_bf16x8*>(dx + row * H);
  const int nv = H >> 3;
  const float mu = mean[row], rs = rstd[row];
  float s1 = 0.f, s2 = 0.f;
  for (int i = threadIdx.x; i < nv; i += LN_THREADS) {
    float a[8], f[8], g[8];
    ln_unpack8(dyr[i], a);
    ln_unpack8(xr[i], f);
    ln_unpack8(wr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gw = a[j] * g[j];
      s1 += gw;
      s2 += gw * (f[j] - mu) * rs;
    }
  }
  const float2 t = ln_block_sum2(s1, s2, red);
  const float m1 = t.x / H, m2 = t.y / H;
  for (int i = threadIdx.x; i < nv; i += LN_THREADS) {
    float a[8], f[8], g[8];
    ln_unpack8(dyr[i], a);
    ln_unpack8(xr[i], f);
    ln_unpack8(wr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = rs * (a[j] * g[j] - m1 - (f[j] - mu) * rs * m2);
    dxr[i] = ln_pack8(a);
  }
}

// Register-resident variants: 128 threads own one row (up to 128 * VPT 16-byte vectors, masked at the row end) and keep it
// in registers; two rows per CTA; one global read and one write per element.
constexpr int LN_ROW_THREADS = 128;

__device__ __forceinline__ float2 ln_row_group_sum2(float a, float b, float2* red) {     // red: 4 entries of this row group
  a = warp_sum(a);
  b = warp_sum(b);
  const int w = (threadIdx.x & (LN_ROW_THREADS - 1)) >> 5;
  if ((threadIdx.x & 31) == 0) red[w] = make_float2(a, b);
  __syncthreads();
  const float2 t = make_float2(red[0].x + red[1].x + red[2].x + red[3].x, red[0].y + red[1].y + red[2].y + red[3].y);
  __syncthreads();
  return t;
}

template <int VPT>
__global__ void __launch_bounds__(2 * LN_ROW_THREADS)
layernorm_fwd_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                         const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
                         float* __restrict__ rstd, long long rows, int H, float eps) {
  __shared__ float2 red_all[2][4];
  const int grp = threadIdx.x / LN_ROW_THREADS, t = threadIdx.x % LN_ROW_THREADS;
  const long long row = static_cast<long long>(blockIdx.x) * 2 + grp;
  const bool live = row < rows;
  const long long r = live ? row : rows - 1;
  const int nv = H >> 3;
  float f[VPT][8];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = t + v * LN_ROW_THREADS;
    if (i < nv) {
      ln_unpack8(reinterpret_cast<const ln_bf16x8*>(x + r * H)[i], f[v]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s += f[v][j];
        ss += f[v][j] * f[v][j];
      }
    }
  }
  const float2 tot = ln_row_group_sum2(s, ss, red_all[grp]);
  const float mu = tot.x / H;
  const float rs = rsqrtf(fmaxf(tot.y / H - mu * mu, 0.f) + eps);
  if (live && t == 0) {
    mean[row] = mu;
    rstd[row] = rs;
  }
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = t + v * LN_ROW_THREADS;
    if (i < nv) {
      float g[8], h[8];
      ln_unpack8(reinterpret_cast<const ln_bf16x8*>(w)[i], g);
      if (b != nullptr) ln_unpack8(reinterpret_cast<const ln_bf16x8*>(b)[i], h);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[v][j] = (f[v][j] - mu) * rs * g[j] + (b != nullptr ? h[j] : 0.f);
      if (live) reinterpret_cast<ln_bf16x8*>(y + r * H)[i] = ln_pack8(f[v]);
    }
  }
}

template <int VPT>
__global__ void __launch_bounds__(2 * LN_ROW_THREADS)
layernorm_bwd_dx_reg_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                            const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean,
                            const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx, long long rows, int H) {
  __shared__ float2 red_all[2][4];
  const int grp = threadIdx.x / LN_ROW_THREADS, t = threadIdx.x % LN_ROW_THREADS;
  const long long row = static_cast<long long>(blockIdx.x) * 2 + grp;
  const bool live = row < rows;
  const long long r = live ? row : rows - 1;
  const int nv = H >> 3;
  const float mu = mean[r], rs = rstd[r];
  float gw[VPT][8], xh[VPT][8];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = t + v * LN_ROW_THREADS;
    if (i < nv) {
      float c[8];
      ln_unpack8(reinterpret_cast<const ln_bf16x8*>(dy + r * H)[i], gw[v]);
      ln_unpack8(reinterpret_cast<const ln_bf16x8*>(x + r * H)[i], xh[v]);
      ln_unpack8(reinterpret_cast<const ln_bf16x8*>(w)[i], c);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        gw[v][j] *= c[j];
        xh[v][j] = (xh[v][j] - mu) * rs;
        s1 += gw[v][j];
        s2 += gw[v][j] * xh[v][j];
      }
    }
  }
  const float2 tot = ln_row_group_sum2(s1, s2, red_all[grp]);
  const float m1 = tot.x / H, m2 = tot.y / H;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = t + v * LN_ROW_THREADS;
    if (i < nv) {
#pragma unroll
      for (int j = 0; j < 8; ++j) gw[v][j] = rs * (gw[v][j] - m1 - xh[v][j] * m2);
      if (live) reinterpret_cast<ln_bf16x8*>(dx + r * H)[i] = ln_pack8(gw[v]);
    }
  }
}

// Warp-per-row variants for narrow rows (H <= 1024).  A warp walks over rows (stride = warps in the grid) with the
// weight and bias vectors packed in registers for the whole walk, holds one row in registers (VPL 16-byte vectors per
// lane, masked at the row end) and reduces with shuffles only, so a CTA never synchronises.  The kernel is bound by
// the load/store unit's data pipe (a profile of the one-row-per-launch-warp version showed it at 91 % with DRAM at 39 %:
// per row the weight and bias re-reads cost as many wavefronts as the row itself), hence the register-resident
// parameters; two rows per warp in flight measured slower than one (3.0 vs 3.3 TB/s at H = 768).
constexpr int LN_WARPS = 8;

template <int VPL>
__global__ void __launch_bounds__(32 * LN_WARPS, VPL >= 3 ? 2 : 3)
layernorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                          const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
                          float* __restrict__ rstd, long long rows, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const long long stride = static_cast<long long>(gridDim.x) * LN_WARPS;
  long long row = static_cast<long long>(blockIdx.x) * LN_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;                                   // whole warps leave together; nothing below synchronises
  const int nv = H >> 3;
  const float inv_h = 1.f / H;
  ln_bf16x8 wp[VPL], bp[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    const int i = lane + v * 32;
    if (i < nv) {
      wp[v] = reinterpret_cast<const ln_bf16x8*>(w)[i];
      if (b != nullptr) bp[v] = reinterpret_cast<const ln_bf16x8*>(b)[i];
    }
  }
  for (; row < rows; row += stride) {
    const ln_bf16x8* xr = reinterpret_cast<const ln_bf16x8*>(x + row * H);
    float f[VPL][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      if (lane + v * 32 < nv) ln_unpack8(xr[lane + v * 32], f[v]);
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      if (lane + v * 32 < nv) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s += f[v][j];
          ss += f[v][j] * f[v][j];
        }
      }
    s = warp_sum(s);
    ss = warp_sum(ss);
    const float mu = s * inv_h;
    const float rs = rsqrtf(fmaxf(ss * inv_h - mu * mu, 0.f) + eps);
    if (lane == 0) {
      mean[row] = mu;
      rstd[row] = rs;
    }
    ln_bf16x8* yr = reinterpret_cast<ln_bf16x8*>(y + row * H);
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int i = lane + v * 32;
      if (i < nv) {
        float g[8], h[8];
        ln_unpack8(wp[v], g);
        if (b != nullptr) ln_unpack8(bp[v], h);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[v][j] = (f[v][j] - mu) * rs * g[j] + (b != nullptr ? h[j] : 0.f);
        yr[i] = ln_pack8(f[v]);
      }
    }
  }
}

// The backward kernel keeps one row per launched warp and re-reads the weight per row: the weight is a quarter of its
// wavefronts (dy, x in, dx out), and the registers for a resident copy cost more occupancy than the re-reads cost
// (measured inside the GPT-2 step: 17.0 us per launch this way, 19.2 us with the walking form of the forward kernel).
template <int VPL>
__global__ void __launch_bounds__(32 * LN_WARPS)
layernorm_bwd_dx_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                             const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean,
                             const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx, long long rows, int H) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * LN_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nv = H >> 3;
  const float mu = mean[row], rs = rstd[row];
  const ln_bf16x8* gr = reinterpret_cast<const ln_bf16x8*>(dy + row * H);
  const ln_bf16x8* xr = reinterpret_cast<const ln_bf16x8*>(x + row * H);
  float gw[VPL][8], xh[VPL][8];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    const int i = lane + v * 32;
    if (i < nv) {
      float c[8];
      ln_unpack8(gr[i], gw[v]);
      ln_unpack8(xr[i], xh[v]);
      ln_unpack8(reinterpret_cast<const ln_bf16x8*>(w)[i], c);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        gw[v][j] *= c[j];
        xh[v][j] = (xh[v][j] - mu) * rs;
        s1 += gw[v][j];
        s2 += gw[v][j] * xh[v][j];
      }
    }
  }
  const float m1 = warp_sum(s1) / H, m2 = warp_sum(s2) / H;
  ln_bf16x8* or_ = reinterpret_cast<ln_bf16x8*>(dx + row * H);
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    const int i = lane + v * 32;
    if (i < nv) {
#pragma unroll
      for (int j = 0; j < 8; ++j) gw[v][j] = rs * (gw[v][j] - m1 - xh[v][j] * m2);
      or_[i] = ln_pack8(gw[v]);
    }
  }
}

// Per-example reductions over the token rows of each example: out[e, col] += sum_r f(r, col).
//   mode 0: f = g                      (bias gradients: LayerNorm bias, linear bias)
//   mode 1: f = g * (x - mean) * rstd  (LayerNorm weight gradient)
//   mode 2: f = g * x * rstd           (RMSNorm weight gradient)
// grid = (examples, column blocks of 256, row splits).  A 256-thread block reads 8 rows x 256 columns per iteration
// with 16-byte loads (32 column groups x 8 row lanes), folds the row lanes through shared memory and adds the split's
// partial sums into that example's row of the fp32 per-example gradient buffer with atomics.
__global__ void __launch_bounds__(256)
rows_group_sum_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ x,
                      const float* __restrict__ mean, const float* __restrict__ rstd, int rows_per_example, int N,
                      long long ldg, float* __restrict__ out, long long ld_out, int mode, float* __restrict__ out2,
                      long long ld_out2) {
  __shared__ float red[8][256 + 8];
  __shared__ float red2[8][256 + 8];
  const int e = blockIdx.x;
  const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int col = blockIdx.y * 256 + cg * 8;
  const int chunk = (rows_per_example + gridDim.z - 1) / gridDim.z;
  const int r0 = e * rows_per_example + blockIdx.z * chunk;
  const int r1 = min(r0 + chunk, (e + 1) * rows_per_example);
  float acc[8], acc2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = acc2[j] = 0.f;
  if (col < N) {
    for (int r = r0 + rl; r < r1; r += 8) {
      float gv[8];
      ln_unpack8(*reinterpret_cast<const ln_bf16x8*>(g + static_cast<long long>(r) * ldg + col), gv);
      if (mode != 0) {
        float xv[8];
        ln_unpack8(*reinterpret_cast<const ln_bf16x8*>(x + static_cast<long long>(r) * ldg + col), xv);
        const float mu = (mode == 1) ? __ldg(mean + r) : 0.f, rs = __ldg(rstd + r);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[j] += gv[j] * (xv[j] - mu) * rs;
          acc2[j] += gv[j];                      // the bias gradient of the same pass (used when out2 is given)
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += gv[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    red[rl][cg * 8 + j] = acc[j];
    if (out2 != nullptr) red2[rl][cg * 8 + j] = acc2[j];
  }
  __syncthreads();
  const int c = threadIdx.x;
  if (blockIdx.y * 256 + c < N) {
    float t = 0.f, t2 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][c];
    atomicAdd(out + static_cast<long long>(e) * ld_out + blockIdx.y * 256 + c, t);
    if (out2 != nullptr) {
#pragma unroll
      for (int k = 0; k < 8; ++k) t2 += red2[k][c];
      atomicAdd(out2 + static_cast<long long>(e) * ld_out2 + blockIdx.y * 256 + c, t2);
    }
  }
}

// Gradients of the three attention inputs, each [B, heads, T, hd] with arbitrary (16-byte aligned) batch / head / token
// strides and contiguous head vectors, gathered into ONE [B*T, 3*heads*hd] buffer: the layout the fused q/k/v
// projection produced in the forward pass.  One thread moves one 16-byte vector; consecutive threads write
// consecutive destination vectors.
struct MergeHeadsSrc {
  const __nv_bfloat16* p;
  long long sb, sh, st;
};

__global__ void __launch_bounds__(256)
merge_heads3_kernel(MergeHeadsSrc s0, MergeHeadsSrc s1, MergeHeadsSrc s2, __nv_bfloat16* __restrict__ out, int T,
                    int heads, int hd, long long total_vec) {
  const int vec_per_head = hd >> 3;
  const int vec_per_part = heads * vec_per_head;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total_vec; i += gridDim.x * 256LL) {
    const int within = static_cast<int>(i % vec_per_part);
    const long long rest = i / vec_per_part;          // (row, part)
    const int part = static_cast<int>(rest % 3);
    const long long row = rest / 3;
    const int h = within / vec_per_head, v = within % vec_per_head;
    const long long b = row / T, t = row % T;
    const MergeHeadsSrc& s = part == 0 ? s0 : (part == 1 ? s1 : s2);
    reinterpret_cast<ln_bf16x8*>(out)[i] =
        *reinterpret_cast<const ln_bf16x8*>(s.p + b * s.sb + h * s.sh + t * s.st + v * 8);
  }
}

// Plain activations.  act: 0 silu, 1 gelu (erf), 2 gelu (tanh approximation), 3 relu.
__device__ __forceinline__ float pa_fwd(float e, int act) {
  if (act == 0) return e / (1.f + __expf(-e));
  if (act == 1) return 0.5f * e * (1.f + erff(e * 0.70710678118654752f));
  if (act == 3) return fmaxf(e, 0.f);
  const float u = 0.7978845608028654f * (e + 0.044715f * e * e * e);
  return 0.5f * e * (1.f + tanhf(u));
}
__device__ __forceinline__ float pa_bwd(float e, int act) {
  if (act == 0) {
    const float s = 1.f / (1.f + __expf(-e));
    return s * (1.f + e * (1.f - s));
  }
  if (act == 1) {
    const float cdf = 0.5f * (1.f + erff(e * 0.70710678118654752f));
    return cdf + e * 0.3989422804014327f * __expf(-0.5f * e * e);
  }
  if (act == 3) return e > 0.f ? 1.f : 0.f;
  const float u = 0.7978845608028654f * (e + 0.044715f * e * e * e);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * e * (1.f - t * t) * 0.7978845608028654f * (1.f + 0.134145f * e * e);
}

// dy == nullptr: out = act(x);  otherwise out = dy * act'(x)
__global__ void __launch_bounds__(256)
activation_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                  __nv_bfloat16* __restrict__ out, long long nvec, int act) {
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += gridDim.x * 256LL) {
    float e[8], d[8];
    ln_unpack8(reinterpret_cast<const ln_bf16x8*>(x)[i], e);
    if (dy != nullptr) {
      ln_unpack8(reinterpret_cast<const ln_bf16x8*>(dy)[i], d);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = d[j] * pa_bwd(e[j], act);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = pa_fwd(e[j], act);
    }
    reinterpret_cast<ln_bf16x8*>(out)[i] = ln_pack8(e);
  }
}

}  // namespace ob

using namespace ob;

// CTAs of the warp-per-row kernels: one warp per row while that fills fewer CTAs than are resident at once (two per SM
// for rows wider than 512, else three), else that many CTAs, whose warps walk over the rows
static unsigned ln_warp_grid(long long rows, int H) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (rows + ob::LN_WARPS - 1) / ob::LN_WARPS, cap = static_cast<long long>(sms) * (H > 512 ? 2 : 3);
  return static_cast<unsigned>(want < cap ? want : cap);
}

extern "C" int ob_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                                long long rows, int H, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16 *xp = static_cast<const __nv_bfloat16*>(x), *wp = static_cast<const __nv_bfloat16*>(w),
                      *bp = static_cast<const __nv_bfloat16*>(b);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
  const unsigned pairs = static_cast<unsigned>((rows + 1) / 2);
  const unsigned octs = ln_warp_grid(rows, H);
  if (H <= 256) layernorm_fwd_warp_kernel<1><<<octs, 32 * LN_WARPS, 0, st>>>(xp, wp, bp, yp, mean, rstd, rows, H, eps);
  else if (H <= 512) layernorm_fwd_warp_kernel<2><<<octs, 32 * LN_WARPS, 0, st>>>(xp, wp, bp, yp, mean, rstd, rows, H, eps);
  else if (H <= 768) layernorm_fwd_warp_kernel<3><<<octs, 32 * LN_WARPS, 0, st>>>(xp, wp, bp, yp, mean, rstd, rows, H, eps);
  else if (H <= 1024) layernorm_fwd_warp_kernel<4><<<octs, 32 * LN_WARPS, 0, st>>>(xp, wp, bp, yp, mean, rstd, rows, H, eps);
  else if (H <= 2048) layernorm_fwd_reg_kernel<2><<<pairs, 2 * LN_ROW_THREADS, 0, st>>>(xp, wp, bp, yp, mean, rstd, rows, H, eps);
  else if (H <= 4096) layernorm_fwd_reg_kernel<4><<<pairs, 2 * LN_ROW_THREADS, 0, st>>>(xp, wp, bp, yp, mean, rstd, rows, H, eps);
  else layernorm_fwd_kernel<<<static_cast<unsigned>(rows), LN_THREADS, 0, st>>>(xp, wp, bp, yp, mean, rstd, H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ob_layernorm_bwd_dx(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                   void* dx, long long rows, int H, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16 *gp = static_cast<const __nv_bfloat16*>(dy), *xp = static_cast<const __nv_bfloat16*>(x),
                      *wp = static_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(dx);
  const unsigned pairs = static_cast<unsigned>((rows + 1) / 2);
  const unsigned octs = static_cast<unsigned>((rows + LN_WARPS - 1) / LN_WARPS);
  if (H <= 256) layernorm_bwd_dx_warp_kernel<1><<<octs, 32 * LN_WARPS, 0, st>>>(gp, xp, wp, mean, rstd, op, rows, H);
  else if (H <= 512) layernorm_bwd_dx_warp_kernel<2><<<octs, 32 * LN_WARPS, 0, st>>>(gp, xp, wp, mean, rstd, op, rows, H);
  else if (H <= 768) layernorm_bwd_dx_warp_kernel<3><<<octs, 32 * LN_WARPS, 0, st>>>(gp, xp, wp, mean, rstd, op, rows, H);
  else if (H <= 1024) layernorm_bwd_dx_warp_kernel<4><<<octs, 32 * LN_WARPS, 0, st>>>(gp, xp, wp, mean, rstd, op, rows, H);
  else if (H <= 2048) layernorm_bwd_dx_reg_kernel<2><<<pairs, 2 * LN_ROW_THREADS, 0, st>>>(gp, xp, wp, mean, rstd, op, rows, H);
  else if (H <= 4096) layernorm_bwd_dx_reg_kernel<4><<<pairs, 2 * LN_ROW_THREADS, 0, st>>>(gp, xp, wp, mean, rstd, op, rows, H);
  else layernorm_bwd_dx_kernel<<<static_cast<unsigned>(rows), LN_THREADS, 0, st>>>(gp, xp, wp, mean, rstd, op, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ob_rows_group_sum(const void* g, const void* x, const float* mean, const float* rstd, int num_examples,
                                 int rows_per_example, int N, long long ldg, float* out, long long ld_out, int mode,
                                 float* out2, long long ld_out2, void* stream) {
  if (num_examples <= 0 || rows_per_example <= 0 || N <= 0) return 0;
  if ((N & 7) || (ldg & 7) || (reinterpret_cast<uintptr_t>(g) & 15) || (x != nullptr && (reinterpret_cast<uintptr_t>(x) & 15)))
    return -2;
  if ((mode == 1 && (x == nullptr || mean == nullptr || rstd == nullptr)) || (mode == 2 && (x == nullptr || rstd == nullptr)))
    return -3;
  int splits = rows_per_example / 64;
  splits = splits < 1 ? 1 : (splits > 16 ? 16 : splits);
  dim3 grid(num_examples, (N + 255) / 256, splits);
  rows_group_sum_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(x), mean, rstd, rows_per_example, N, ldg,
      out, ld_out, mode, mode == 0 ? nullptr : out2, ld_out2);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ob_merge_heads3(const void* q, const void* k, const void* v, const long long* strides, void* out,
                               long long B, int T, int heads, int hd, int sms, void* stream) {
  if (B <= 0 || T <= 0) return 0;
  if (hd % 8) return -2;
  const void* ptrs[3] = {q, k, v};
  MergeHeadsSrc src[3];
  for (int i = 0; i < 3; ++i) {
    src[i].p = static_cast<const __nv_bfloat16*>(ptrs[i]);
    src[i].sb = strides[3 * i];
    src[i].sh = strides[3 * i + 1];
    src[i].st = strides[3 * i + 2];
    if ((reinterpret_cast<uintptr_t>(ptrs[i]) & 15) || (src[i].sb & 7) || (src[i].sh & 7) || (src[i].st & 7)) return -2;
  }
  if (reinterpret_cast<uintptr_t>(out) & 15) return -2;
  const long long total_vec = B * T * 3 * heads * (hd / 8);
  long long grid = (total_vec + 255) / 256;
  const long long cap = static_cast<long long>(sms) * 16;
  if (grid > cap) grid = cap;
  merge_heads3_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src[0], src[1], src[2], static_cast<__nv_bfloat16*>(out), T, heads, hd, total_vec);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ob_activation(const void* x, const void* dy, void* out, long long numel, int act, int sms, void* stream) {
  if (numel <= 0) return 0;
  if (numel % 8) return -2;
  const long long nvec = numel / 8;
  long long grid = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(sms) * 16;
  if (grid > cap) grid = cap;
  activation_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(out), nvec, act);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
