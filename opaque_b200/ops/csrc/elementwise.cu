// Bandwidth-bound transformer kernels for sm_100a: RMSNorm (+ fused residual add) forward /
// backward with per-example weight gradients, SwiGLU / GeGLU forward / backward, joint Q/K
// rotary embedding, and a fused cross-entropy (online softmax, NLL, in-place dlogits).
// bf16 storage, fp32 math, 16-byte vector accesses; every kernel reads each input once per
// pass and is sized so that one CTA owns one row (norms, cross-entropy) or a flat range.
#include "common.cuh"
#include "api.h"

namespace ob {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : -INFINITY;
  if (warp == 0) {
    t = warp_max(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// ---------------------------------------------------------------------------------------------
// RMSNorm.  mode 0 ("llama"): normalise in fp32, round to bf16, multiply by (offset + w).
//           mode 1 ("gemma"): everything in fp32, one rounding at the end.
constexpr int RN_THREADS = 256;

__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd, int H, float eps, float offset,
                   int mode) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * H);
  const bf16x8* rr = residual ? reinterpret_cast<const bf16x8*>(residual + row * H) : nullptr;
  bf16x8* sr = sum_out ? reinterpret_cast<bf16x8*>(sum_out + row * H) : nullptr;
  const int nv = H >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += RN_THREADS) {
    float f[8];
    unpack8(xr[i], f);
    if (rr) {
      float g[8];
      unpack8(rr[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      const bf16x8 s = pack8(f);
      sr[i] = s;
      unpack8(s, f);   // the normalised tensor is the *stored* (rounded) sum
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  const float total = block_sum<RN_THREADS>(ss, red);
  const float rs = rsqrtf(total / H + eps);
  if (threadIdx.x == 0) rstd[row] = rs;
  const bf16x8* src = sr ? reinterpret_cast<const bf16x8*>(sum_out + row * H) : xr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * H);
  for (int i = threadIdx.x; i < nv; i += RN_THREADS) {
    float f[8], g[8];
    unpack8(src[i], f);
    unpack8(wr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float n = f[j] * rs;
      if (mode == 0) n = __bfloat162float(__float2bfloat16_rn(n));
      f[j] = n * (offset + g[j]);
    }
    yr[i] = pack8(f);
  }
}

// Register-resident variants for the common widths (H = 128 * 8 * VPT, VPT in {1, 2, 4, 8}): 128 threads own one row
// and keep it in registers, two rows per CTA; one global read and one write per element, one shared-memory exchange.
constexpr int RN_ROW_THREADS = 128;

__device__ __forceinline__ float row_group_sum(float v, float* red) {     // red: 4 floats of this row group
  v = warp_sum(v);
  const int w = (threadIdx.x & (RN_ROW_THREADS - 1)) >> 5;
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  const float t = red[0] + red[1] + red[2] + red[3];
  __syncthreads();
  return t;
}

template <int VPT>
__global__ void __launch_bounds__(2 * RN_ROW_THREADS)
rmsnorm_fwd_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                       __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd, long long rows, float eps,
                       float offset, int mode) {
  constexpr int H = RN_ROW_THREADS * 8 * VPT;
  __shared__ float red_all[2][4];
  const int grp = threadIdx.x / RN_ROW_THREADS, t = threadIdx.x % RN_ROW_THREADS;
  const long long row = static_cast<long long>(blockIdx.x) * 2 + grp;
  const bool live = row < rows;
  const long long r = live ? row : rows - 1;               // dead group mirrors the last row (keeps the barriers uniform)
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + r * H);
  float f[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    unpack8(xr[t + v * RN_ROW_THREADS], f[v]);
    if (residual != nullptr) {
      float g[8];
      unpack8(reinterpret_cast<const bf16x8*>(residual + r * H)[t + v * RN_ROW_THREADS], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[v][j] += g[j];
      const bf16x8 sv = pack8(f[v]);
      if (live) reinterpret_cast<bf16x8*>(sum_out + r * H)[t + v * RN_ROW_THREADS] = sv;
      unpack8(sv, f[v]);                                    // the normalised tensor is the stored (rounded) sum
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[v][j] * f[v][j];
  }
  const float rs = rsqrtf(row_group_sum(ss, red_all[grp]) / H + eps);
  if (live && t == 0) rstd[row] = rs;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    float g[8];
    unpack8(reinterpret_cast<const bf16x8*>(w)[t + v * RN_ROW_THREADS], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float n = f[v][j] * rs;
      if (mode == 0) n = __bfloat162float(__float2bfloat16_rn(n));
      f[v][j] = n * (offset + g[j]);
    }
    if (live) reinterpret_cast<bf16x8*>(y + r * H)[t + v * RN_ROW_THREADS] = pack8(f[v]);
  }
}

template <int VPT>
__global__ void __launch_bounds__(2 * RN_ROW_THREADS)
rmsnorm_bwd_dx_reg_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                          const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                          const __nv_bfloat16* __restrict__ dsum_in, __nv_bfloat16* __restrict__ dx, long long rows,
                          float offset) {
  constexpr int H = RN_ROW_THREADS * 8 * VPT;
  __shared__ float red_all[2][4];
  const int grp = threadIdx.x / RN_ROW_THREADS, t = threadIdx.x % RN_ROW_THREADS;
  const long long row = static_cast<long long>(blockIdx.x) * 2 + grp;
  const bool live = row < rows;
  const long long r = live ? row : rows - 1;
  const float rs = rstd[r];
  float gw[VPT][8], xv[VPT][8];
  float dot = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    float c[8];
    unpack8(reinterpret_cast<const bf16x8*>(dy + r * H)[t + v * RN_ROW_THREADS], gw[v]);
    unpack8(reinterpret_cast<const bf16x8*>(x + r * H)[t + v * RN_ROW_THREADS], xv[v]);
    unpack8(reinterpret_cast<const bf16x8*>(w)[t + v * RN_ROW_THREADS], c);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      gw[v][j] *= (offset + c[j]);
      dot += gw[v][j] * xv[v][j];
    }
  }
  const float mean = row_group_sum(dot, red_all[grp]) * rs * rs / H;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    float d[8];
    if (dsum_in != nullptr) unpack8(reinterpret_cast<const bf16x8*>(dsum_in + r * H)[t + v * RN_ROW_THREADS], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float g = rs * (gw[v][j] - xv[v][j] * mean);
      if (dsum_in != nullptr) g += d[j];
      gw[v][j] = g;
    }
    if (live) reinterpret_cast<bf16x8*>(dx + r * H)[t + v * RN_ROW_THREADS] = pack8(gw[v]);
  }
}

// dx (and d residual, which equals dx plus the incoming gradient of the sum stream).
__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                      const __nv_bfloat16* __restrict__ dsum_in, __nv_bfloat16* __restrict__ dx, int H,
                      float offset) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + row * H);
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * H);
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  const bf16x8* dsr = dsum_in ? reinterpret_cast<const bf16x8*>(dsum_in + row * H) : nullptr;
  bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + row * H);
  const int nv = H >> 3;
  const float rs = rstd[row];
  float dot = 0.f;
  for (int i = threadIdx.x; i < nv; i += RN_THREADS) {
    float a[8], b[8], c[8];
    unpack8(dyr[i], a);
    unpack8(xr[i], b);
    unpack8(wr[i], c);
#pragma unroll
    for (int j = 0; j < 8; ++j) dot += a[j] * (offset + c[j]) * b[j];
  }
  const float mean = block_sum<RN_THREADS>(dot, red) * rs * rs / H;
  for (int i = threadIdx.x; i < nv; i += RN_THREADS) {
    float a[8], b[8], c[8], d[8];
    unpack8(dyr[i], a);
    unpack8(xr[i], b);
    unpack8(wr[i], c);
    if (dsr) unpack8(dsr[i], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float g = rs * (a[j] * (offset + c[j]) - b[j] * mean);
      if (dsr) g += d[j];
      a[j] = g;
    }
    dxr[i] = pack8(a);
  }
}

// Per-example weight gradient: dW[e, h] = sum over the rows of example e of dy * x * rstd.
// grid = (examples, H / (2 * threads)); each thread owns two adjacent columns.
__global__ void __launch_bounds__(128)
rmsnorm_bwd_dw_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const float* __restrict__ rstd, const int* __restrict__ seg_offsets, int rows_per_example,
                      float* __restrict__ dw, int H) {
  const int e = blockIdx.x;
  const int col = (blockIdx.y * 128 + threadIdx.x) * 2;
  if (col >= H) return;
  const int r0 = seg_offsets ? seg_offsets[e] : e * rows_per_example;
  const int r1 = seg_offsets ? seg_offsets[e + 1] : r0 + rows_per_example;
  float a0 = 0.f, a1 = 0.f;
  for (int r = r0; r < r1; ++r) {
    const float rs = __ldg(rstd + r);
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dy + static_cast<long long>(r) * H + col));
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + static_cast<long long>(r) * H + col));
    a0 += g.x * v.x * rs;
    a1 += g.y * v.y * rs;
  }
  dw[static_cast<long long>(e) * H + col] = a0;
  dw[static_cast<long long>(e) * H + col + 1] = a1;
}

// ---------------------------------------------------------------------------------------------
// Gated activations.  act: 0 = SwiGLU (silu), 1 = GeGLU exact (erf), 2 = GeGLU tanh approximation.
__device__ __forceinline__ float act_fwd(float e, int act) {
  if (act == 0) return e / (1.f + __expf(-e));
  if (act == 1) return 0.5f * e * (1.f + erff(e * 0.70710678118654752f));
  const float u = 0.7978845608028654f * (e + 0.044715f * e * e * e);
  return 0.5f * e * (1.f + tanhf(u));
}
__device__ __forceinline__ float act_bwd(float e, int act) {
  if (act == 0) {
    const float s = 1.f / (1.f + __expf(-e));
    return s * (1.f + e * (1.f - s));
  }
  if (act == 1) {
    const float cdf = 0.5f * (1.f + erff(e * 0.70710678118654752f));
    return cdf + e * 0.3989422804014327f * __expf(-0.5f * e * e);
  }
  const float u = 0.7978845608028654f * (e + 0.044715f * e * e * e);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * e * (1.f - t * t) * 0.7978845608028654f * (1.f + 0.134145f * e * e);
}

__global__ void __launch_bounds__(256)
glu_fwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
               __nv_bfloat16* __restrict__ out, long long rows, int I, long long ld_in, int act) {
  const long long nvec = rows * (I >> 3);
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += gridDim.x * 256LL) {
    const long long r = i / (I >> 3);
    const int c = static_cast<int>(i % (I >> 3)) << 3;
    float e[8], g[8];
    unpack8(*reinterpret_cast<const bf16x8*>(gate + r * ld_in + c), e);
    unpack8(*reinterpret_cast<const bf16x8*>(up + r * ld_in + c), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = act_fwd(e[j], act) * g[j];
    *reinterpret_cast<bf16x8*>(out + r * I + c) = pack8(e);
  }
}

__global__ void __launch_bounds__(256)
glu_bwd_kernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ gate,
               const __nv_bfloat16* __restrict__ up, __nv_bfloat16* __restrict__ dgate,
               __nv_bfloat16* __restrict__ dup, long long rows, int I, long long ld_in, long long ld_out, int act) {
  const long long nvec = rows * (I >> 3);
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += gridDim.x * 256LL) {
    const long long r = i / (I >> 3);
    const int c = static_cast<int>(i % (I >> 3)) << 3;
    float d[8], e[8], g[8], de[8], dg[8];
    unpack8(*reinterpret_cast<const bf16x8*>(dh + r * I + c), d);
    unpack8(*reinterpret_cast<const bf16x8*>(gate + r * ld_in + c), e);
    unpack8(*reinterpret_cast<const bf16x8*>(up + r * ld_in + c), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[j] = d[j] * act_fwd(e[j], act);
      de[j] = d[j] * g[j] * act_bwd(e[j], act);
    }
    *reinterpret_cast<bf16x8*>(dgate + r * ld_out + c) = pack8(de);
    *reinterpret_cast<bf16x8*>(dup + r * ld_out + c) = pack8(dg);
  }
}

// ---------------------------------------------------------------------------------------------
// Rotary embedding on Q and K in one pass (rotate-half convention, GQA: different head counts).
// q: [rows, Hq, D], k: [rows, Hk, D]; cos/sin: fp32 [positions, D/2]; pos: [rows] or nullptr
// (then position = row % seq_len).  sign = -1 gives the backward pass.
__global__ void __launch_bounds__(256)
rope_qk_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k, const float* __restrict__ cs,
               const float* __restrict__ sn, const int* __restrict__ pos, long long rows, int seq_len, int Hq,
               int Hk, int D, long long ldq, long long ldk, float sign) {
  const int half = D >> 1;
  const int pairs_per_head = half >> 1;                 // two rotation pairs per thread (bf16x2)
  const long long per_row = static_cast<long long>(Hq + Hk) * pairs_per_head;
  const long long total = rows * per_row;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += gridDim.x * 256LL) {
    const long long r = i / per_row;
    int rem = static_cast<int>(i % per_row);
    const int h = rem / pairs_per_head;
    const int d = (rem % pairs_per_head) << 1;
    const int pidx = pos ? pos[r] : static_cast<int>(r % seq_len);
    __nv_bfloat16* base = (h < Hq) ? q + r * ldq + static_cast<long long>(h) * D
                                   : k + r * ldk + static_cast<long long>(h - Hq) * D;
    const float2 c = *reinterpret_cast<const float2*>(cs + static_cast<long long>(pidx) * half + d);
    float2 s = *reinterpret_cast<const float2*>(sn + static_cast<long long>(pidx) * half + d);
    s.x *= sign;
    s.y *= sign;
    const float2 lo = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(base + d));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(base + half + d));
    *reinterpret_cast<__nv_bfloat162*>(base + d) = __floats2bfloat162_rn(lo.x * c.x - hi.x * s.x, lo.y * c.y - hi.y * s.y);
    *reinterpret_cast<__nv_bfloat162*>(base + half + d) = __floats2bfloat162_rn(hi.x * c.x + lo.x * s.x, hi.y * c.y + lo.y * s.y);
  }
}

// Out-of-place rotary embedding with 16-byte accesses: reads Q / K through (batch, token, head) strides (views into a
// fused q|k|v projection buffer, or the [B, H, T, D] gradients an attention kernel returns) and writes contiguous
// [rows, H, D] outputs, so no copy is needed before or after.  One thread rotates 8 + 8 elements (columns d .. d+7 and
// half+d .. half+d+7 of one head).  D % 16 == 0; all pointers and strides 16-byte aligned.
struct RopeSrc {
  const __nv_bfloat16* ptr;
  long long sb, st, sh;      // element strides of batch, token and head; the last dimension is contiguous
};

__global__ void __launch_bounds__(256)
rope_qk_oop_kernel(RopeSrc qs, RopeSrc ks, __nv_bfloat16* __restrict__ qo, __nv_bfloat16* __restrict__ ko,
                   const float* __restrict__ cs, const float* __restrict__ sn, const int* __restrict__ pos,
                   long long rows, int seq_len, int Hq, int Hk, int D, float sign) {
  const int half = D >> 1;
  const int chunks = half >> 3;                          // 8-element chunks per half head
  const long long per_row = static_cast<long long>(Hq + Hk) * chunks;
  const long long total = rows * per_row;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += gridDim.x * 256LL) {
    const long long r = i / per_row;
    const int rem = static_cast<int>(i % per_row);
    const int h = rem / chunks;
    const int d = (rem % chunks) << 3;
    const long long b = r / seq_len, t = r % seq_len;
    const int pidx = pos ? pos[r] : static_cast<int>(t);
    const bool is_q = h < Hq;
    const int hh = is_q ? h : h - Hq;
    const RopeSrc& src = is_q ? qs : ks;
    const __nv_bfloat16* in = src.ptr + b * src.sb + t * src.st + hh * src.sh;
    __nv_bfloat16* out = (is_q ? qo + r * Hq * D : ko + r * Hk * D) + static_cast<long long>(hh) * D;
    const uint4 lo4 = *reinterpret_cast<const uint4*>(in + d);
    const uint4 hi4 = *reinterpret_cast<const uint4*>(in + half + d);
    const float* cp = cs + static_cast<long long>(pidx) * half + d;
    const float* sp = sn + static_cast<long long>(pidx) * half + d;
    const float4 c0 = *reinterpret_cast<const float4*>(cp), c1 = *reinterpret_cast<const float4*>(cp + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const __nv_bfloat162* lo = reinterpret_cast<const __nv_bfloat162*>(&lo4);
    const __nv_bfloat162* hi = reinterpret_cast<const __nv_bfloat162*>(&hi4);
    uint4 olo, ohi;
    __nv_bfloat162* plo = reinterpret_cast<__nv_bfloat162*>(&olo);
    __nv_bfloat162* phi = reinterpret_cast<__nv_bfloat162*>(&ohi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 l = __bfloat1622float2(lo[j]), hv = __bfloat1622float2(hi[j]);
      const float sx = sv[2 * j] * sign, sy = sv[2 * j + 1] * sign;
      plo[j] = __floats2bfloat162_rn(l.x * c[2 * j] - hv.x * sx, l.y * c[2 * j + 1] - hv.y * sy);
      phi[j] = __floats2bfloat162_rn(hv.x * c[2 * j] + l.x * sx, hv.y * c[2 * j + 1] + l.y * sy);
    }
    *reinterpret_cast<uint4*>(out + d) = olo;
    *reinterpret_cast<uint4*>(out + half + d) = ohi;
  }
}

// ---------------------------------------------------------------------------------------------
// Cross-entropy over one row per CTA.  z = softcap * tanh(scale*logit / softcap) (softcap = 0: off).
// Outputs nll[row] = lse - z[label] (label smoothing: minus (eps/V) * (sum z - V*lse) mix), lse[row];
// with write_grad the logits are overwritten by  row_weight * d nll / d logit  (zero for ignored rows).
constexpr int CE_THREADS = 512;

__device__ __forceinline__ float ce_transform(float v, float scale, float softcap) {
  v *= scale;
  if (softcap != 0.f) v = softcap * tanhf(v / softcap);
  return v;
}

template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
cross_entropy_kernel(T* __restrict__ logits, const long long* __restrict__ labels,
                     const float* __restrict__ row_weight, float* __restrict__ nll, float* __restrict__ lse_out,
                     int V, long long ld, float scale, float softcap, float smoothing, long long ignore_index,
                     int write_grad) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  T* z = logits + row * ld;
  const long long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  if (ignored) {
    if (threadIdx.x == 0) {
      nll[row] = 0.f;
      if (lse_out) lse_out[row] = 0.f;
    }
    if (write_grad) {
      int done = 0;
      if constexpr (sizeof(T) == 2) {
        if ((ld & 7) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
          done = V & ~7;
          const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
          for (int i = threadIdx.x; i < (done >> 3); i += CE_THREADS) reinterpret_cast<uint4*>(z)[i] = zero;
        }
      }
      for (int i = done + threadIdx.x; i < V; i += CE_THREADS) z[i] = static_cast<T>(0.f);
    }
    return;
  }
  // pass 1: online max / sum-exp (+ plain sum for label smoothing)
  float m = -INFINITY, s = 0.f, tot = 0.f;
  // bf16 rows with 16-byte aligned starts are read 8 values at a time; the ragged tail (V % 8) and fp32 rows go
  // through the scalar loop
  int v_vec = 0;
  if constexpr (sizeof(T) == 2) {
    if ((ld & 7) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) v_vec = V & ~7;
  }
  if constexpr (sizeof(T) == 2) {
    const bf16x8* zv = reinterpret_cast<const bf16x8*>(z);
    for (int i = threadIdx.x; i < (v_vec >> 3); i += CE_THREADS) {
      float f[8];
      unpack8(zv[i], f);
      float lm = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[j] = ce_transform(f[j], scale, softcap);
        tot += f[j];
        lm = fmaxf(lm, f[j]);
      }
      if (lm > m) {
        s *= __expf(m - lm);
        m = lm;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
    }
  }
  for (int i = v_vec + threadIdx.x; i < V; i += CE_THREADS) {
    const float v = ce_transform(static_cast<float>(z[i]), scale, softcap);
    tot += v;
    if (v > m) {
      s = s * __expf(m - v) + 1.f;
      m = v;
    } else {
      s += __expf(v - m);
    }
  }
  const float gm = block_max<CE_THREADS>(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum<CE_THREADS>(s, red);
  const float lse = gm + __logf(gs);
  float zl = ce_transform(static_cast<float>(z[label]), scale, softcap);
  float loss = lse - zl;
  if (smoothing > 0.f) {
    const float gt = block_sum<CE_THREADS>(tot, red);
    loss = (1.f - smoothing) * loss + smoothing * (lse - gt / V);
  }
  if (threadIdx.x == 0) {
    nll[row] = loss;
    if (lse_out) lse_out[row] = lse;
  }
  if (!write_grad) return;
  const float wgt = row_weight ? row_weight[row] : 1.f;
  if constexpr (sizeof(T) == 2) {
    bf16x8* zv = reinterpret_cast<bf16x8*>(z);
    for (int i = threadIdx.x; i < (v_vec >> 3); i += CE_THREADS) {
      float f[8];
      unpack8(zv[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float raw = f[j] * scale;
        float v = raw, dz = 1.f;
        if (softcap != 0.f) {
          const float t = tanhf(raw / softcap);
          v = softcap * t;
          dz = 1.f - t * t;
        }
        float g = __expf(v - lse) - smoothing / V;
        if (i * 8 + j == label) g -= (1.f - smoothing);
        f[j] = wgt * g * dz * scale;
      }
      zv[i] = pack8(f);
    }
  }
  for (int i = v_vec + threadIdx.x; i < V; i += CE_THREADS) {
    const float raw = static_cast<float>(z[i]) * scale;
    float v = raw, dz = 1.f;
    if (softcap != 0.f) {
      const float t = tanhf(raw / softcap);
      v = softcap * t;
      dz = 1.f - t * t;
    }
    float g = __expf(v - lse) - smoothing / V;
    if (i == label) g -= (1.f - smoothing);
    z[i] = static_cast<T>(wgt * g * dz * scale);
  }
}

}  // namespace ob

// ---------------------------------------------------------------------------------------------
using namespace ob;
#define OB_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : -21)

static int flat_grid(long long work, int per_block, int sms) {
  long long g = (work + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(sms) * 16;
  if (g > cap) g = cap;
  return g < 1 ? 1 : static_cast<int>(g);
}

extern "C" int ob_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* sum_out,
                              float* rstd, long long rows, int H, float eps, float offset, int mode, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16 *xp = static_cast<const __nv_bfloat16*>(x), *rp = static_cast<const __nv_bfloat16*>(residual),
                      *wp = static_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16 *yp = static_cast<__nv_bfloat16*>(y), *sp = static_cast<__nv_bfloat16*>(sum_out);
  const unsigned pairs = static_cast<unsigned>((rows + 1) / 2);
#define OB_RN_FWD(V) rmsnorm_fwd_reg_kernel<V><<<pairs, 2 * RN_ROW_THREADS, 0, st>>>(xp, rp, wp, yp, sp, rstd, rows, eps, offset, mode)
  if (H == 1024) OB_RN_FWD(1);
  else if (H == 2048) OB_RN_FWD(2);
  else if (H == 4096) OB_RN_FWD(4);
  else if (H == 8192) OB_RN_FWD(8);
  else rmsnorm_fwd_kernel<<<static_cast<unsigned>(rows), RN_THREADS, 0, st>>>(xp, rp, wp, yp, sp, rstd, H, eps, offset, mode);
#undef OB_RN_FWD
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dsum_in,
                              void* dx, float* dw_per_example, const int* seg_offsets, int num_examples,
                              int rows_per_example, long long rows, int H, float offset, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dx != nullptr) {
    const __nv_bfloat16 *gp = static_cast<const __nv_bfloat16*>(dy), *xp = static_cast<const __nv_bfloat16*>(x),
                        *wp = static_cast<const __nv_bfloat16*>(w), *dp = static_cast<const __nv_bfloat16*>(dsum_in);
    __nv_bfloat16* op = static_cast<__nv_bfloat16*>(dx);
    const unsigned pairs = static_cast<unsigned>((rows + 1) / 2);
#define OB_RN_BWD(V) rmsnorm_bwd_dx_reg_kernel<V><<<pairs, 2 * RN_ROW_THREADS, 0, st>>>(gp, xp, wp, rstd, dp, op, rows, offset)
    if (H == 1024) OB_RN_BWD(1);
    else if (H == 2048) OB_RN_BWD(2);
    else if (H == 4096) OB_RN_BWD(4);
    else if (H == 8192) OB_RN_BWD(8);
    else rmsnorm_bwd_dx_kernel<<<static_cast<unsigned>(rows), RN_THREADS, 0, st>>>(gp, xp, wp, rstd, dp, op, H, offset);
#undef OB_RN_BWD
  }
  if (dw_per_example != nullptr && num_examples > 0) {
    dim3 grid(num_examples, (H / 2 + 127) / 128);
    rmsnorm_bwd_dw_kernel<<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(dy),
                                                static_cast<const __nv_bfloat16*>(x), rstd, seg_offsets,
                                                rows_per_example, dw_per_example, H);
  }
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_glu_fwd(const void* gate, const void* up, void* out, long long rows, int I, long long ld_in,
                          int act, int sms, void* stream) {
  if (rows <= 0) return 0;
  if (I % 8 || ld_in % 8) return -2;
  glu_fwd_kernel<<<flat_grid(rows * (I / 8), 256, sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
      static_cast<__nv_bfloat16*>(out), rows, I, ld_in, act);
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_glu_bwd(const void* dh, const void* gate, const void* up, void* dgate, void* dup, long long rows,
                          int I, long long ld_in, long long ld_out, int act, int sms, void* stream) {
  if (rows <= 0) return 0;
  if (I % 8 || ld_in % 8 || ld_out % 8) return -2;
  glu_bwd_kernel<<<flat_grid(rows * (I / 8), 256, sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dh), static_cast<const __nv_bfloat16*>(gate),
      static_cast<const __nv_bfloat16*>(up), static_cast<__nv_bfloat16*>(dgate), static_cast<__nv_bfloat16*>(dup),
      rows, I, ld_in, ld_out, act);
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_rope_qk(void* q, void* k, const float* cos_t, const float* sin_t, const int* pos, long long rows,
                          int seq_len, int Hq, int Hk, int D, long long ldq, long long ldk, int backward, int sms,
                          void* stream) {
  if (rows <= 0) return 0;
  if (D % 4) return -2;
  const long long work = rows * (Hq + Hk) * (D / 4);
  rope_qk_kernel<<<flat_grid(work, 256, sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), cos_t, sin_t, pos, rows, seq_len, Hq, Hk, D,
      ldq, ldk, backward ? -1.f : 1.f);
  return OB_CHECK_LAUNCH();
}

// Out-of-place, strided-input form (see rope_qk_oop_kernel): q_in / k_in are read through element strides (batch, token,
// head), q_out / k_out are contiguous [rows, H, D].  Returns -2 when D % 16 != 0, -3 when something is not 16-byte aligned.
extern "C" int ob_rope_qk_oop(const void* q_in, const void* k_in, void* q_out, void* k_out, const float* cos_t,
                              const float* sin_t, const int* pos, long long rows, int seq_len, int Hq, int Hk, int D,
                              long long q_sb, long long q_st, long long q_sh, long long k_sb, long long k_st, long long k_sh,
                              int backward, int sms, void* stream) {
  if (rows <= 0) return 0;
  if (D % 16) return -2;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al(q_in) || !al(k_in) || !al(q_out) || !al(k_out) || !al(cos_t) || !al(sin_t) ||
      ((q_sb | q_st | q_sh | k_sb | k_st | k_sh) & 7) != 0)
    return -3;
  RopeSrc qs{static_cast<const __nv_bfloat16*>(q_in), q_sb, q_st, q_sh};
  RopeSrc ks{static_cast<const __nv_bfloat16*>(k_in), k_sb, k_st, k_sh};
  const long long work = rows * (Hq + Hk) * (D / 16);
  rope_qk_oop_kernel<<<flat_grid(work, 256, sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      qs, ks, static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_out), cos_t, sin_t, pos, rows, seq_len, Hq,
      Hk, D, backward ? -1.f : 1.f);
  return OB_CHECK_LAUNCH();
}

extern "C" int ob_cross_entropy(void* logits, int is_fp32, const long long* labels, const float* row_weight,
                                float* nll, float* lse, long long rows, int V, long long ld, float scale,
                                float softcap, float smoothing, long long ignore_index, int write_grad,
                                void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (scale == 0.f) scale = 1.f;
  if (is_fp32)
    cross_entropy_kernel<float><<<static_cast<unsigned>(rows), CE_THREADS, 0, st>>>(
        static_cast<float*>(logits), labels, row_weight, nll, lse, V, ld, scale, softcap, smoothing, ignore_index,
        write_grad);
  else
    cross_entropy_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), CE_THREADS, 0, st>>>(
        static_cast<__nv_bfloat16*>(logits), labels, row_weight, nll, lse, V, ld, scale, softcap, smoothing,
        ignore_index, write_grad);
  return OB_CHECK_LAUNCH();
}
