// Clip-weighted weight-gradient GEMM for sm_100a.
//
//   D[g][m, n]  (+)=  sum over rows t of segment g of   s[t] * A[t, m] * B[t, n]
//
// A = [T, M] and B = [T, N] are row-major bf16 (output gradients and layer inputs of a
// linear layer, rows = tokens).  The contraction runs over rows, so both operands are
// "MN-major" for the tensor core: TMA brings [64 rows x 64 cols] boxes (128-byte swizzle)
// and tcgen05.mma consumes them through MN-major shared-memory descriptors.  s[t] is the
// per-row clip factor c_example(t) (optional); it is applied to the A tile in shared memory
// by four "scaler" warps between the TMA arrival and the MMA issue, which also zero rows
// outside the segment so that grouped (per-example / per-expert) calls may have ragged ends.
//
// Warp roles (448 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5
// epilogue (TMEM -> registers -> global), warps 6-13 scalers (two groups on alternate k-blocks).  The kernel is persistent: CTAs
// walk a work list of (segment, k-split, m-tile, n-tile); accumulators are double-buffered in
// TMEM so the epilogue of one item overlaps the main loop of the next.
//
// Epilogue: the fp32 tile is either stored or added (red.global.add) at
// flat index  out_offset + g_off + m*ldm + n*ldn.  When a peer table is given the flat index
// space is cut into equal contiguous shards, one per rank, and each element goes straight to
// the owning rank's buffer through its peer pointer: split-K accumulation, accumulation over
// microbatches and the cross-GPU reduce-scatter are the same instruction stream.
// Row-major output (ldn == 1) is transposed through shared memory so every warp-level
// reduction covers four 128-byte row segments (full NVLink packets / L2 lines).
//
// All waits are bounded (see common.cuh); on a timeout the CTA drains its TMA copies, frees
// TMEM and returns with a code in `status`.
#include <cstdio>
#include "common.cuh"
#include "api.h"

namespace ob {

constexpr int WG_BLOCK_M = 128;
constexpr int WG_BLOCK_K = 64;       // rows (tokens) per pipeline stage
constexpr int WG_UMMA_K = 16;
constexpr int WG_THREADS = 448;      // 2 + 4 epilogue + 2 x 4 scaler warps
constexpr int WG_STAGE_LD = 36;      // padded row length (floats) of the epilogue staging tile

struct WgradParams {
  int M, N, T;
  int num_groups;
  const int* seg_offsets;            // [num_groups + 1] or nullptr (one segment [0, T))
  int splits;
  const float* row_scale;            // [T] or nullptr
  float* out;                        // used when peer_out == nullptr
  float* const* peer_out;            // [world] base pointers of every rank's shard
  long long shard_elems;
  const long long* group_out_offset; // [num_groups] or nullptr (g * group_stride)
  long long group_stride;
  long long out_offset;
  long long ldm, ldn;
  int n_valid;                       // only columns n < n_valid are written
  int accumulate;
  int* status;
  unsigned long long wait_budget_ns;
};

template <int BLOCK_N>
struct WgradSmem {
  static constexpr int A_BYTES = WG_BLOCK_K * WG_BLOCK_M * 2;
  static constexpr int B_BYTES = WG_BLOCK_K * BLOCK_N * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BLOCK_N == 256) ? 4 : 6;
  static constexpr int EPI_BYTES = 4 * 32 * WG_STAGE_LD * 4;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024;
};

struct WorkItem {
  int g, m0, n0, row_begin, seg_end, num_kb;
  long long out_base;
};

__device__ __forceinline__ WorkItem decode_work(const WgradParams& p, int w, int tiles_m, int tiles_n,
                                                int block_n) {
  WorkItem it;
  const int mn = tiles_m * tiles_n;
  const int gs = w / mn, r = w % mn;
  it.g = gs / p.splits;
  const int split = gs % p.splits;
  it.m0 = (r / tiles_n) * WG_BLOCK_M;
  it.n0 = (r % tiles_n) * block_n;
  const int b = p.seg_offsets ? p.seg_offsets[it.g] : 0;
  const int e = p.seg_offsets ? p.seg_offsets[it.g + 1] : p.T;
  const int nkb = (e - b + WG_BLOCK_K - 1) / WG_BLOCK_K;
  const int kb0 = static_cast<int>(static_cast<long long>(nkb) * split / p.splits);
  const int kb1 = static_cast<int>(static_cast<long long>(nkb) * (split + 1) / p.splits);
  it.row_begin = b + kb0 * WG_BLOCK_K;
  it.seg_end = min(e, b + kb1 * WG_BLOCK_K);
  it.num_kb = kb1 - kb0;
  it.out_base = p.out_offset + (p.group_out_offset ? p.group_out_offset[it.g]
                                                   : static_cast<long long>(it.g) * p.group_stride);
  return it;
}

__device__ __forceinline__ float* resolve_out(const WgradParams& p, long long idx) {
  if (p.peer_out == nullptr) return p.out + idx;
  const long long owner = idx / p.shard_elems;
  return p.peer_out[owner] + (idx - owner * p.shard_elems);
}

template <int BLOCK_N>
__global__ void __launch_bounds__(WG_THREADS, 1)
wgrad_clip_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const WgradParams p) {
  using S = WgradSmem<BLOCK_N>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  float* epi = reinterpret_cast<float*>(smem + S::STAGES * S::STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE_BYTES + S::EPI_BYTES);
  uint64_t* full = bars;                     // [STAGES]  TMA bytes landed
  uint64_t* empty = bars + S::STAGES;        // [STAGES]  MMAs reading the stage retired
  uint64_t* scaled = bars + 2 * S::STAGES;   // [STAGES]  scaler warps done with the stage
  uint64_t* tmem_full = bars + 3 * S::STAGES;       // [2]
  uint64_t* tmem_empty = bars + 3 * S::STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * S::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + WG_BLOCK_M - 1) / WG_BLOCK_M;
  const int tiles_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int total_work = p.num_groups * p.splits * tiles_m * tiles_n;
  const uint64_t budget = p.wait_budget_ns;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&scaled[s], 4);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BLOCK_N);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, issued_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const WorkItem it = decode_work(p, w, tiles_m, tiles_n, BLOCK_N);
        for (int kb = 0; kb < it.num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_EMPTY, budget)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], S::STAGE_BYTES);
          uint8_t* a_dst = stage_base + stage * S::STAGE_BYTES;
          uint8_t* b_dst = a_dst + S::A_BYTES;
          const int row = it.row_begin + kb * WG_BLOCK_K;
#pragma unroll
          for (int j = 0; j < WG_BLOCK_M / 64; ++j)
            tma_load_2d(a_dst + j * (WG_BLOCK_K * 128), &map_a, &full[stage], it.m0 + 64 * j, row);
#pragma unroll
          for (int j = 0; j < BLOCK_N / 64; ++j)
            tma_load_2d(b_dst + j * (WG_BLOCK_K * 128), &map_b, &full[stage], it.n0 + 64 * j, row);
          issued_mask |= 1u << stage;
          issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
          if (++stage == S::STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // unwind: let every copy this thread started land before the CTA's shared memory goes away
        for (int s = 0; s < S::STAGES; ++s)
          if (issued_mask & (1u << s)) {
            int dummy_abort = 0;
            mbar_wait(&full[s], (issued_phase >> s) & 1u, &dummy_abort, p.status, OB_ERR_DRAIN, budget);
          }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(WG_BLOCK_M, BLOCK_N, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc_iter = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const WorkItem it = decode_work(p, w, tiles_m, tiles_n, BLOCK_N);
        if (it.num_kb == 0) continue;
        const int as = acc_iter & 1;
        if (!mbar_wait(&tmem_empty[as], ((acc_iter >> 1) & 1) ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY,
                       budget)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BLOCK_N;
        for (int kb = 0; kb < it.num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL, budget) ||
              !mbar_wait(&scaled[stage], phase, abort_flag, p.status, OB_ERR_WAIT_SCALED, budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(stage_base + stage * S::STAGE_BYTES);
          const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < WG_BLOCK_K / WG_UMMA_K; ++kk) {
            // MN-major, 128-byte swizzle: 8 rows = 1024 B (stride offset), next 64-column block =
            // BLOCK_K*128 B (leading offset); 16 rows per instruction = 2048 B per k-step.
            const uint64_t ad = make_smem_desc(a_addr + kk * (WG_UMMA_K * 128), WG_BLOCK_K * 128, 1024, 2);
            const uint64_t bd = make_smem_desc(b_addr + kk * (WG_UMMA_K * 128), WG_BLOCK_K * 128, 1024, 2);
            umma_bf16(d_tmem, ad, bd, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == S::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[as]);
        ++acc_iter;
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;                      // TMEM lane quadrant this warp may read
    float* st = epi + (warp - 2) * 32 * WG_STAGE_LD;
    int acc_iter = 0;
    bool ok = true;
    const int n_lim = min(p.N, p.n_valid);
    const bool vec_ok = (p.ldn == 1) && ((n_lim & 3) == 0) && ((p.ldm & 3) == 0) &&
                        (p.peer_out == nullptr || (p.shard_elems & 3) == 0);
    for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      const WorkItem it = decode_work(p, w, tiles_m, tiles_n, BLOCK_N);
      const bool row_major = vec_ok && ((it.out_base & 3) == 0);
      if (it.num_kb == 0 && p.accumulate) continue;
      int as = 0;
      if (it.num_kb > 0) {
        as = acc_iter & 1;
        if (!mbar_wait(&tmem_full[as], (acc_iter >> 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL, budget)) {
          ok = false;
          break;
        }
        tc_fence_after();
      }
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        const int nc = it.n0 + c * 32;
        if (nc >= n_lim) break;
        float v[32];
        if (it.num_kb > 0) {
          tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * BLOCK_N + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        if (row_major) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(st + lane * WG_STAGE_LD + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          __syncwarp();
#pragma unroll
          for (int rr = 0; rr < 8; ++rr) {
            const int r = rr * 4 + (lane >> 3), c4 = (lane & 7) * 4;
            const float4 x = *reinterpret_cast<const float4*>(st + r * WG_STAGE_LD + c4);
            const int m = it.m0 + q * 32 + r, n = nc + c4;
            if (m < p.M && n < n_lim) {
              float* dst = resolve_out(p, it.out_base + static_cast<long long>(m) * p.ldm + n);
              if (p.accumulate) red_add_v4(dst, x);
              else *reinterpret_cast<float4*>(dst) = x;
            }
          }
          __syncwarp();
        } else {
          const int m = it.m0 + q * 32 + lane;
          if (m < p.M) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int n = nc + j;
              if (n < n_lim) {
                float* dst = resolve_out(p, it.out_base + static_cast<long long>(m) * p.ldm + static_cast<long long>(n) * p.ldn);
                if (p.accumulate) red_add_f32(dst, v[j]);
                else *dst = v[j];
              }
            }
          }
        }
      }
      if (it.num_kb > 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[as]);
        ++acc_iter;
      }
    }
  } else {
    // ------------------------------------------------------------------ scalers
    // Two groups of four warps take alternate k-blocks, so the shared-memory round trip of one
    // block overlaps the other group's; the four row factors a thread needs for its NEXT block
    // are fetched before it waits for that block's TMA data.  The factor is rounded toward zero
    // to bf16 and applied with packed bf16x2 multiplies: |stored product| <= |s * g| (1 + 2^-9),
    // which the caller's guard on s absorbs.
    const int group = (warp - 6) >> 2;           // 0 or 1
    const int tid = (threadIdx.x - 6 * 32) & 127;
    const int my_row = tid >> 3;
    long long it_global = 0;                     // k-block counter over the whole work list
    bool ok = true;
    for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      const WorkItem it = decode_work(p, w, tiles_m, tiles_n, BLOCK_N);
      // first k-block of this item that belongs to this group
      int kb = static_cast<int>((group - (it_global & 1) + 2) & 1);
      float sc[4];
      bool have = false;
      auto fetch = [&](int kblock) {
        const int row0 = it.row_begin + kblock * WG_BLOCK_K;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int rg = row0 + my_row + 16 * i;
          sc[i] = (rg < it.seg_end) ? (p.row_scale ? __ldg(p.row_scale + rg) : 1.f) : 0.f;
        }
      };
      if (kb < it.num_kb) { fetch(kb); have = true; }
      for (; kb < it.num_kb; kb += 2) {
        const long long g_it = it_global + kb;
        const int stage = static_cast<int>(g_it % S::STAGES);
        const uint32_t phase = static_cast<uint32_t>((g_it / S::STAGES) & 1);
        const int row0 = it.row_begin + kb * WG_BLOCK_K;
        const bool touch = (p.row_scale != nullptr) || (row0 + WG_BLOCK_K > it.seg_end);
        __nv_bfloat162 s2[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat16 h = __float2bfloat16_rz(sc[i]);
          s2[i] = __halves2bfloat162(h, h);
        }
        if (kb + 2 < it.num_kb) fetch(kb + 2);   // prefetch for the next block of this group
        if (!mbar_wait(&full[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL, budget)) {
          ok = false;
          break;
        }
        if (touch) {
          uint4* a_tile = reinterpret_cast<uint4*>(stage_base + stage * S::STAGE_BYTES);
          uint4 x[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = a_tile[tid + 128 * i];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) h[e] = __hmul2(h[e], s2[i & 3]);
            a_tile[tid + 128 * i] = x[i];
          }
          fence_proxy_async_smem();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&scaled[stage]);
      }
      (void)have;
      it_global += it.num_kb;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BLOCK_N);
  }
}

// ---------------------------------------------------------------------------------------------
// Per-example variant: every example owns a whole number of 64-row k-blocks (uniform rows_per_example), so the clip
// factor is constant over an accumulation run.  The MMA warp accumulates ONE example's A_e^T G_e per TMEM buffer and
// the epilogue warps fold it into fp32 register accumulators as  acc += c_e * P_e  while the tensor core already
// works on the next example in the other buffer.  Operands are never touched in shared memory (no scaling pass, no
// extra barrier in the TMA -> MMA chain) and c_e is applied in full fp32 precision.
constexpr int WP_THREADS = 320;      // TMA warp, MMA warp, 8 epilogue warps (2 per TMEM lane quadrant)
constexpr int WP_BLOCK_N = 256;
constexpr int WP_STAGES = 4;
constexpr int WP_A_BYTES = WG_BLOCK_K * WG_BLOCK_M * 2;
constexpr int WP_B_BYTES = WG_BLOCK_K * WP_BLOCK_N * 2;
constexpr int WP_STAGE_BYTES = WP_A_BYTES + WP_B_BYTES;
constexpr int WP_SMEM = WP_STAGES * WP_STAGE_BYTES + 256 + 1024;

struct WgradPeParams {
  int M, N;
  int num_examples, ex_rows;         // ex_rows is a multiple of WG_BLOCK_K
  int splits;                        // each split owns a contiguous range of examples
  const float* ex_scale;             // [num_examples] or nullptr (all ones)
  float* out;
  float* const* peer_out;
  long long shard_elems;
  long long out_offset;
  long long ldm;
  int accumulate;
  float* norm2_out;                  // NORM kernel: [num_examples] squared Frobenius norms are added here; nothing else is written
  int* status;
  unsigned long long wait_budget_ns;
};

__device__ __forceinline__ float* resolve_out_pe(const WgradPeParams& p, long long idx) {
  if (p.peer_out == nullptr) return p.out + idx;
  const long long owner = idx / p.shard_elems;
  return p.peer_out[owner] + (idx - owner * p.shard_elems);
}

// NORM = true: the direct form of a per-example gradient norm.  The same per-example products P_e = A_e^T G_e pass through
// tensor memory tile by tile, but the epilogue only sums their squares into norm2_out[e]; nothing is scaled, accumulated or
// stored.  Costs 2 T d_in d_out FLOPs per example against T^2 (d_in + d_out) for the Gram-matrix form, so it is the
// cheaper one for long sequences on small layers.
template <bool NORM>
__global__ void __launch_bounds__(WP_THREADS, 1)
wgrad_clip_pe_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const WgradPeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WP_STAGES * WP_STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + WP_STAGES;
  uint64_t* tmem_full = bars + 2 * WP_STAGES;
  uint64_t* tmem_empty = bars + 2 * WP_STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * WP_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + WG_BLOCK_M - 1) / WG_BLOCK_M;
  const int tiles_n = (p.N + WP_BLOCK_N - 1) / WP_BLOCK_N;
  const int total_work = p.splits * tiles_m * tiles_n;
  const int kpe = p.ex_rows / WG_BLOCK_K;
  const uint64_t budget = p.wait_budget_ns;

  if (threadIdx.x == 0) {
    for (int s = 0; s < WP_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * WP_BLOCK_N);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // work item w -> (split, m tile, n tile); split s owns examples [e0, e1)
  auto decode = [&](int w, int& m0, int& n0, int& e0, int& e1) {
    const int mn = tiles_m * tiles_n;
    const int split = w / mn, r = w % mn;
    m0 = (r / tiles_n) * WG_BLOCK_M;
    n0 = (r % tiles_n) * WP_BLOCK_N;
    e0 = static_cast<int>(static_cast<long long>(p.num_examples) * split / p.splits);
    e1 = static_cast<int>(static_cast<long long>(p.num_examples) * (split + 1) / p.splits);
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, issued_mask = 0, issued_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        int m0, n0, e0, e1;
        decode(w, m0, n0, e0, e1);
        const int nkb = (e1 - e0) * kpe;
        const int row_begin = e0 * p.ex_rows;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_EMPTY, budget)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], WP_STAGE_BYTES);
          uint8_t* a_dst = smem + stage * WP_STAGE_BYTES;
          uint8_t* b_dst = a_dst + WP_A_BYTES;
          const int row = row_begin + kb * WG_BLOCK_K;
#pragma unroll
          for (int j = 0; j < WG_BLOCK_M / 64; ++j)
            tma_load_2d(a_dst + j * (WG_BLOCK_K * 128), &map_a, &full[stage], m0 + 64 * j, row);
#pragma unroll
          for (int j = 0; j < WP_BLOCK_N / 64; ++j)
            tma_load_2d(b_dst + j * (WG_BLOCK_K * 128), &map_b, &full[stage], n0 + 64 * j, row);
          issued_mask |= 1u << stage;
          issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
          if (++stage == WP_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        for (int s = 0; s < WP_STAGES; ++s)
          if (issued_mask & (1u << s)) {
            int dummy_abort = 0;
            mbar_wait(&full[s], (issued_phase >> s) & 1u, &dummy_abort, p.status, OB_ERR_DRAIN, budget);
          }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(WG_BLOCK_M, WP_BLOCK_N, 1, 1);
      int stage = 0, acc_iter = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        int m0, n0, e0, e1;
        decode(w, m0, n0, e0, e1);
        for (int e = e0; ok && e < e1; ++e) {
          const int as = acc_iter & 1;
          if (!mbar_wait(&tmem_empty[as], ((acc_iter >> 1) & 1) ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY,
                         budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + as * WP_BLOCK_N;
          for (int kb = 0; kb < kpe; ++kb) {
            if (!mbar_wait(&full[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL, budget)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(smem + stage * WP_STAGE_BYTES);
            const uint32_t b_addr = a_addr + WP_A_BYTES;
#pragma unroll
            for (int kk = 0; kk < WG_BLOCK_K / WG_UMMA_K; ++kk) {
              const uint64_t ad = make_smem_desc(a_addr + kk * (WG_UMMA_K * 128), WG_BLOCK_K * 128, 1024, 2);
              const uint64_t bd = make_smem_desc(b_addr + kk * (WG_UMMA_K * 128), WG_BLOCK_K * 128, 1024, 2);
              umma_bf16(d_tmem, ad, bd, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(&empty[stage]);
            if (++stage == WP_STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          umma_commit(&tmem_full[as]);
          ++acc_iter;
        }
      }
    }
  } else {
    const int q = warp & 3;                      // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;            // which 128 of the tile's 256 columns
    int acc_iter = 0;
    bool ok = true;
    const bool vec_ok = ((p.ldm & 3) == 0) && ((p.N & 3) == 0) && ((p.out_offset & 3) == 0) &&
                        (p.peer_out == nullptr || (p.shard_elems & 3) == 0);
    for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      int m0, n0, e0, e1;
      decode(w, m0, n0, e0, e1);
      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;
      for (int e = e0; e < e1; ++e) {
        const int as = acc_iter & 1;
        const float c = p.ex_scale ? __ldg(p.ex_scale + e) : 1.f;
        if (!mbar_wait(&tmem_full[as], (acc_iter >> 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL, budget)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if constexpr (NORM) {
          // rows / columns outside the matrices were zero-filled by the tensor maps, so no masking is needed
          float ss = 0.f;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            float v[32];
            tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * WP_BLOCK_N + half * 128 + ch * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) ss = fmaf(v[j], v[j], ss);
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          if (lane == 0) atomicAdd(p.norm2_out + e, ss);
        } else if (c != 0.f) {
        // an example with factor 0 (non-finite norm, padding) is skipped, not multiplied: 0 * NaN would poison the sum
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            float v[32];
            tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * WP_BLOCK_N + half * 128 + ch * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[ch * 32 + j] = fmaf(c, v[j], acc[ch * 32 + j]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[as]);
        ++acc_iter;
      }
      if (!ok) break;
      if constexpr (NORM) continue;
      if (e1 <= e0 && p.accumulate) continue;
      const int m = m0 + q * 32 + lane;
      if (m < p.M) {
        const long long row_base = p.out_offset + static_cast<long long>(m) * p.ldm;
#pragma unroll
        for (int j4 = 0; j4 < 32; ++j4) {
          const int n = n0 + half * 128 + 4 * j4;
          if (n >= p.N) break;
          if (vec_ok) {
            float* dst = resolve_out_pe(p, row_base + n);
            const float4 x = make_float4(acc[4 * j4], acc[4 * j4 + 1], acc[4 * j4 + 2], acc[4 * j4 + 3]);
            if (p.accumulate) red_add_v4(dst, x);
            else *reinterpret_cast<float4*>(dst) = x;
          } else {
#pragma unroll
            for (int t = 0; t < 4; ++t)
              if (n + t < p.N) {
                float* dst = resolve_out_pe(p, row_base + n + t);
                if (p.accumulate) red_add_f32(dst, acc[4 * j4 + t]);
                else *dst = acc[4 * j4 + t];
              }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * WP_BLOCK_N);
  }
}

// ---------------------------------------------------------------------------------------------
// host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

static thread_local char g_map_detail[192] = {0};

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with row pitch `ld` elements.
int make_bf16_map_2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                     int box_cols, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -10;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((ld * 2) & 15) != 0) {
    snprintf(g_map_detail, sizeof(g_map_detail), "operand not 16-byte aligned: base=%p ld=%lld", base, ld);
    return -11;
  }
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  // Driver entry points need a context bound to the calling thread; framework worker threads (autograd) may never
  // have made a runtime call of their own on the default device, so bind the primary context once per thread.
  static thread_local bool bound = false;
  if (!bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) bound = true;
  }
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    snprintf(g_map_detail, sizeof(g_map_detail), "tensor map rejected (CUresult %d): base=%p rows=%lld cols=%lld ld=%lld box=%dx%d",
             static_cast<int>(r), base, rows, cols, ld, box_cols, box_rows);
  return r == CUDA_SUCCESS ? 0 : -12;
}

template <int BLOCK_N>
static int launch_wgrad(const CUtensorMap& ma, const CUtensorMap& mb, const WgradParams& p, int sms,
                        cudaStream_t stream) {
  using S = WgradSmem<BLOCK_N>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(wgrad_clip_kernel<BLOCK_N>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL) !=
        cudaSuccess)
      return -20;
    configured = true;
  }
  const int tiles_m = (p.M + WG_BLOCK_M - 1) / WG_BLOCK_M, tiles_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const long long total = static_cast<long long>(p.num_groups) * p.splits * tiles_m * tiles_n;
  if (total <= 0) return 0;
  const int grid = static_cast<int>(total < sms ? total : sms);
  wgrad_clip_kernel<BLOCK_N><<<grid, WG_THREADS, S::TOTAL, stream>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace ob

extern "C" int ob_wgrad_clip(const void* a, const void* b, int T, int M, int N, long long lda, long long ldb,
                             const float* row_scale, const int* seg_offsets, int num_groups, int splits,
                             float* out, float* const* peer_out, long long shard_elems,
                             const long long* group_out_offset, long long group_stride, long long out_offset,
                             long long ldm, long long ldn, int n_valid, int accumulate, int block_n, int* status,
                             double wait_budget_s, int num_sms, void* stream) {
  using namespace ob;
  if (T <= 0 || M <= 0 || N <= 0 || num_groups <= 0) return 0;
  if (splits < 1) splits = 1;
  CUtensorMap ma, mb;
  int rc = make_bf16_map_2d(&ma, a, T, M, lda, 64, WG_BLOCK_K);
  if (rc) return rc;
  rc = make_bf16_map_2d(&mb, b, T, N, ldb, 64, WG_BLOCK_K);
  if (rc) return rc;
  WgradParams p;
  p.M = M; p.N = N; p.T = T;
  p.num_groups = num_groups;
  p.seg_offsets = seg_offsets;
  p.splits = splits;
  p.row_scale = row_scale;
  p.out = out;
  p.peer_out = peer_out;
  p.shard_elems = shard_elems;
  p.group_out_offset = group_out_offset;
  p.group_stride = group_stride;
  p.out_offset = out_offset;
  p.ldm = ldm; p.ldn = ldn;
  p.n_valid = n_valid > 0 ? n_valid : N;
  p.accumulate = accumulate;
  p.status = status;
  p.wait_budget_ns = static_cast<unsigned long long>(wait_budget_s * 1e9);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (block_n == 256) return launch_wgrad<256>(ma, mb, p, num_sms, st);
  if (block_n == 128) return launch_wgrad<128>(ma, mb, p, num_sms, st);
  if (block_n == 64) return launch_wgrad<64>(ma, mb, p, num_sms, st);
  return -1;
}

static int launch_wgrad_pe(const void* a, const void* b, int num_examples, int ex_rows, int M, int N, long long lda,
                           long long ldb, const float* ex_scale, int splits, float* out, float* const* peer_out,
                           long long shard_elems, long long out_offset, long long ldm, int accumulate, float* norm2_out,
                           int* status, double wait_budget_s, int num_sms, void* stream) {
  using namespace ob;
  if (num_examples <= 0 || ex_rows <= 0 || M <= 0 || N <= 0) return 0;
  if (ex_rows % WG_BLOCK_K) return -3;
  if (splits < 1) splits = 1;
  if (splits > num_examples) splits = num_examples;
  if (splits > 1 && !accumulate && norm2_out == nullptr) return -4;   // split partial sums must be reduced into the destination
  const long long T = static_cast<long long>(num_examples) * ex_rows;
  if (T > 0x7fffffffLL) return -5;
  CUtensorMap ma, mb;
  int rc = make_bf16_map_2d(&ma, a, T, M, lda, 64, WG_BLOCK_K);
  if (rc) return rc;
  rc = make_bf16_map_2d(&mb, b, T, N, ldb, 64, WG_BLOCK_K);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(wgrad_clip_pe_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, WP_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(wgrad_clip_pe_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, WP_SMEM) != cudaSuccess)
      return -20;
    configured = true;
  }
  WgradPeParams p;
  p.M = M; p.N = N;
  p.num_examples = num_examples; p.ex_rows = ex_rows;
  p.splits = splits;
  p.ex_scale = ex_scale;
  p.out = out;
  p.peer_out = peer_out;
  p.shard_elems = shard_elems;
  p.out_offset = out_offset;
  p.ldm = ldm;
  p.accumulate = accumulate;
  p.norm2_out = norm2_out;
  p.status = status;
  p.wait_budget_ns = static_cast<unsigned long long>(wait_budget_s * 1e9);
  const long long tiles = static_cast<long long>((M + WG_BLOCK_M - 1) / WG_BLOCK_M) * ((N + WP_BLOCK_N - 1) / WP_BLOCK_N);
  const long long total = tiles * splits;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  if (norm2_out != nullptr)
    wgrad_clip_pe_kernel<true><<<grid, WP_THREADS, WP_SMEM, static_cast<cudaStream_t>(stream)>>>(ma, mb, p);
  else
    wgrad_clip_pe_kernel<false><<<grid, WP_THREADS, WP_SMEM, static_cast<cudaStream_t>(stream)>>>(ma, mb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

extern "C" int ob_wgrad_clip_pe(const void* a, const void* b, int num_examples, int ex_rows, int M, int N, long long lda,
                                long long ldb, const float* ex_scale, int splits, float* out, float* const* peer_out,
                                long long shard_elems, long long out_offset, long long ldm, int accumulate, int* status,
                                double wait_budget_s, int num_sms, void* stream) {
  return launch_wgrad_pe(a, b, num_examples, ex_rows, M, N, lda, ldb, ex_scale, splits, out, peer_out, shard_elems, out_offset,
                         ldm, accumulate, nullptr, status, wait_budget_s, num_sms, stream);
}

// Direct per-example gradient norms: norm2[e] += || a_e^T b_e ||_F^2 for example e = rows [e * ex_rows, (e + 1) * ex_rows)
// of a [T, M] and b [T, N] (ex_rows % 64 == 0).  `splits` spreads the examples of one tile over several CTAs.
extern "C" int ob_direct_norm2(const void* a, const void* b, int num_examples, int ex_rows, int M, int N, long long lda,
                               long long ldb, int splits, float* norm2, int* status, double wait_budget_s, int num_sms,
                               void* stream) {
  if (norm2 == nullptr) return -6;
  return launch_wgrad_pe(a, b, num_examples, ex_rows, M, N, lda, ldb, nullptr, splits, nullptr, nullptr, 0, 0, N, 0, norm2, status,
                         wait_budget_s, num_sms, stream);
}

extern "C" int ob_last_detail(char* buf, int len) {
  int i = 0;
  for (; ob::g_map_detail[i] && i < len - 1; ++i) buf[i] = ob::g_map_detail[i];
  buf[i] = 0;
  return 0;
}
