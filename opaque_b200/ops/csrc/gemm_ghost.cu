// Ghost per-example gradient norms of a linear layer on sm_100a.
//
// For example i with token rows A_i [T, Da] (layer inputs) and G_i [T, Dg] (output
// gradients) the weight gradient is A_i^T G_i and its squared Frobenius norm equals
//     sum over (t, t') of (A_i A_i^T)[t, t'] * (G_i G_i^T)[t, t'],
// so it can be computed without ever forming the [Da, Dg] per-example gradient.  One work
// item is (example, 128 x 128 tile of the T x T Gram matrices, upper triangle only): the two
// Gram tiles are accumulated side by side in TMEM by tcgen05.mma (K-major operands, 128-byte
// swizzle, TMA-fed), and the epilogue multiplies them element-wise, masks rows / columns that
// fall outside the example, doubles off-diagonal tiles and adds the tile's sum to norm2[i].
// A diagonal tile multiplies a row block with itself, so its producer loads that block once and both operand
// descriptors point at it (the kernel is bound by the L2 -> shared-memory feed, not by the tensor pipe).
//
// With `ids` given (embedding layers) the first Gram matrix is replaced by the indicator
// [ids_t == ids_t'], which is the Gram matrix of one-hot rows.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer / TMEM owner, warps 2-5 epilogue; persistent
// CTAs, double-buffered accumulators, bounded waits (see common.cuh).
#include "common.cuh"
#include "api.h"

namespace ob {

int make_bf16_map_2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                     int box_cols, int box_rows);

constexpr int GH_TILE = 128;
constexpr int GH_BLOCK_K = 64;
constexpr int GH_STAGES = 6;
constexpr int GH_TILE_BYTES = GH_TILE * GH_BLOCK_K * 2;    // 16 KB
constexpr int GH_STAGE_BYTES = 2 * GH_TILE_BYTES;
constexpr int GH_THREADS = 192;
constexpr int GH_SMEM = GH_STAGES * GH_STAGE_BYTES + 256 + 1024;

struct GhostParams {
  int B, T, Da, Dg;      // B segments of (at most) T rows
  const int* ids;        // [rows] or nullptr
  const int* seg;        // [B + 1] row offsets of ragged segments, or nullptr (segment b = rows [b*T, (b+1)*T))
  const int* seg_out;    // [B] accumulator index of every segment, or nullptr (identity)
  float* norm2;          // accumulated with atomics
  int* status;
  unsigned long long wait_budget_ns;
};

struct GhostItem {
  int ex, tb, tb2;
};

__device__ __forceinline__ GhostItem ghost_decode(int w, int pairs, int nt) {
  GhostItem it;
  it.ex = w / pairs;
  int r = w % pairs;
  int tb = 0;
  while (r >= nt - tb) {
    r -= nt - tb;
    ++tb;
  }
  it.tb = tb;
  it.tb2 = tb + r;
  return it;
}

__global__ void __launch_bounds__(GH_THREADS, 1)
ghost_norm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_g,
                  const GhostParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GH_STAGES * GH_STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + GH_STAGES;
  uint64_t* tmem_full = bars + 2 * GH_STAGES;
  uint64_t* tmem_empty = bars + 2 * GH_STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GH_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = (p.T + GH_TILE - 1) / GH_TILE;
  const int pairs = nt * (nt + 1) / 2;
  const int total_work = p.B * pairs;
  const int ka = p.ids ? 0 : (p.Da + GH_BLOCK_K - 1) / GH_BLOCK_K;
  const int kg = (p.Dg + GH_BLOCK_K - 1) / GH_BLOCK_K;
  const int num_kb = ka + kg;
  const uint64_t budget = p.wait_budget_ns;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GH_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_g);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, issued_mask = 0, issued_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const GhostItem it = ghost_decode(w, pairs, nt);
        const int s0 = p.seg ? p.seg[it.ex] : it.ex * p.T;
        const int len = p.seg ? p.seg[it.ex + 1] - s0 : p.T;
        if (it.tb2 * GH_TILE >= len) continue;                 // tile pair lies outside this (ragged) segment
        const int r1 = s0 + it.tb * GH_TILE, r2 = s0 + it.tb2 * GH_TILE;
        const bool diag = it.tb == it.tb2;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_EMPTY, budget)) {
            ok = false;
            break;
          }
          // a diagonal tile multiplies a row block with itself: one load serves both operands
          mbar_expect_tx(&full[stage], diag ? GH_TILE_BYTES : GH_STAGE_BYTES);
          uint8_t* dst = smem + stage * GH_STAGE_BYTES;
          const CUtensorMap* map = kb < ka ? &map_a : &map_g;
          const int col = (kb < ka ? kb : kb - ka) * GH_BLOCK_K;
          tma_load_2d(dst, map, &full[stage], col, r1);
          if (!diag) tma_load_2d(dst + GH_TILE_BYTES, map, &full[stage], col, r2);
          issued_mask |= 1u << stage;
          issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
          if (++stage == GH_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        for (int s = 0; s < GH_STAGES; ++s)
          if (issued_mask & (1u << s)) {
            int dummy_abort = 0;
            mbar_wait(&full[s], (issued_phase >> s) & 1u, &dummy_abort, p.status, OB_ERR_DRAIN, budget);
          }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(GH_TILE, GH_TILE, 0, 0);
      int stage = 0, acc_iter = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const GhostItem it = ghost_decode(w, pairs, nt);
        if (p.seg && it.tb2 * GH_TILE >= p.seg[it.ex + 1] - p.seg[it.ex]) continue;
        const uint32_t b_off = it.tb == it.tb2 ? 0u : static_cast<uint32_t>(GH_TILE_BYTES);
        const int as = acc_iter & 1;
        if (!mbar_wait(&tmem_empty[as], ((acc_iter >> 1) & 1) ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY,
                       budget)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL, budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t t1 = smem_u32(smem + stage * GH_STAGE_BYTES), t2 = t1 + b_off;
          const uint32_t d_tmem = tmem_base + as * 256 + (kb < ka ? 0 : 128);
          const bool first = (kb == 0) || (kb == ka);
#pragma unroll
          for (int kk = 0; kk < GH_BLOCK_K / 16; ++kk) {
            // K-major, 128-byte swizzle: rows are 128 B apart, 8-row groups 1024 B apart; a k-step
            // of 16 elements moves the start address by 32 B inside the swizzled row.
            const uint64_t ad = make_smem_desc(t1 + kk * 32, 16, 1024, 2);
            const uint64_t bd = make_smem_desc(t2 + kk * 32, 16, 1024, 2);
            umma_bf16(d_tmem, ad, bd, idesc, (first && kk == 0) ? 0u : 1u);
          }
          umma_commit(&empty[stage]);
          if (++stage == GH_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[as]);
        ++acc_iter;
      }
    }
  } else {
    const int q = warp & 3;
    int acc_iter = 0;
    bool ok = true;
    for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      const GhostItem it = ghost_decode(w, pairs, nt);
      const int s0 = p.seg ? p.seg[it.ex] : it.ex * p.T;
      const int len = p.seg ? p.seg[it.ex + 1] - s0 : p.T;
      if (it.tb2 * GH_TILE >= len) continue;
      const int as = acc_iter & 1;
      if (!mbar_wait(&tmem_full[as], (acc_iter >> 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL, budget)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int t = it.tb * GH_TILE + q * 32 + lane;
      const int my_id = (p.ids && t < len) ? p.ids[s0 + t] : -1;
      float acc = 0.f;
      for (int c = 0; c < GH_TILE / 32; ++c) {
        float sg[32], sa[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * 256 + c * 32;
        tmem_ld32(taddr + 128, sg);
        if (!p.ids) tmem_ld32(taddr, sa);
        tmem_ld_wait();
        const int tc0 = it.tb2 * GH_TILE + c * 32;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int t2 = tc0 + j;
          float a;
          if (p.ids) {
            const int other = (t2 < len) ? __ldg(p.ids + s0 + t2) : -2;
            a = (other == my_id) ? 1.f : 0.f;
          } else {
            a = sa[j];
          }
          if (t < len && t2 < len) acc += a * sg[j];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[as]);
      ++acc_iter;
      acc = warp_sum(acc);
      if (lane == 0) atomicAdd(p.norm2 + (p.seg_out ? p.seg_out[it.ex] : it.ex), (it.tb == it.tb2 ? 1.f : 2.f) * acc);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// Wide variant: one work item is a 128 x 256 block of the T x T Gram matrices (row block tb, column blocks 2cb and
// 2cb+1).  Per k-block the tensor core reads 48 KB of shared memory for 4.2 MFLOP instead of 32 KB for 2.1 MFLOP, which
// lifts the shared-memory bound of the 128 x 128 tiles.  The two Gram tiles fill TMEM (2 x 256 columns), so
// accumulators are single-buffered: the next item's MMAs start when the 8 epilogue warps have drained both tiles.
// Column blocks below the diagonal inside a super-block get weight 0, the diagonal block 1, blocks above it 2.
constexpr int GW_TILE_N = 256;
constexpr int GW_STAGES = 4;
constexpr int GW_A_BYTES = GH_TILE * GH_BLOCK_K * 2;       // 16 KB: rows of the row block
constexpr int GW_B_BYTES = GW_TILE_N * GH_BLOCK_K * 2;     // 32 KB: rows of the two column blocks
constexpr int GW_STAGE_BYTES = GW_A_BYTES + GW_B_BYTES;
constexpr int GW_THREADS = 320;                            // TMA, MMA, 8 epilogue warps
constexpr int GW_SMEM = GW_STAGES * GW_STAGE_BYTES + 256 + 1024;

struct GhostWideItem {
  int ex, tb, cb;
};

// items of one example, ordered by row block: row block tb owns super-blocks cb = tb/2 .. ncb-1
__device__ __forceinline__ GhostWideItem ghost_wide_decode(int w, int per_example, int nt, int ncb) {
  GhostWideItem it;
  it.ex = w / per_example;
  int r = w % per_example;
  int tb = 0;
  while (r >= ncb - (tb >> 1)) {
    r -= ncb - (tb >> 1);
    ++tb;
  }
  it.tb = tb;
  it.cb = (tb >> 1) + r;
  (void)nt;
  return it;
}

__global__ void __launch_bounds__(GW_THREADS, 1)
ghost_norm_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_g,
                       const GhostParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GW_STAGES * GW_STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + GW_STAGES;
  uint64_t* tmem_full = bars + 2 * GW_STAGES;
  uint64_t* tmem_empty = bars + 2 * GW_STAGES + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GW_STAGES + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nt = (p.T + GH_TILE - 1) / GH_TILE;
  const int ncb = (nt + 1) / 2;
  int per_example = 0;
  for (int tb = 0; tb < nt; ++tb) per_example += ncb - (tb >> 1);
  const int total_work = p.B * per_example;
  const int ka = p.ids ? 0 : (p.Da + GH_BLOCK_K - 1) / GH_BLOCK_K;
  const int kg = (p.Dg + GH_BLOCK_K - 1) / GH_BLOCK_K;
  const int num_kb = ka + kg;
  const uint64_t budget = p.wait_budget_ns;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GW_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, 8);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_g);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // segment of example `ex`: first row and length; an item is skipped when its column blocks start past the end
  auto segment = [&](int ex, int& s0, int& len) {
    s0 = p.seg ? p.seg[ex] : ex * p.T;
    len = p.seg ? p.seg[ex + 1] - s0 : p.T;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, issued_mask = 0, issued_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const GhostWideItem it = ghost_wide_decode(w, per_example, nt, ncb);
        int s0, len;
        segment(it.ex, s0, len);
        if (it.tb * GH_TILE >= len || it.cb * GW_TILE_N >= len) continue;
        const int r1 = s0 + it.tb * GH_TILE, r2 = s0 + it.cb * GW_TILE_N;
        const bool diag = (it.tb >> 1) == it.cb;              // the row block is one of the two column blocks
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_EMPTY, budget)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], diag ? GW_B_BYTES : GW_STAGE_BYTES);
          uint8_t* dst = smem + stage * GW_STAGE_BYTES;
          const CUtensorMap* map = kb < ka ? &map_a : &map_g;
          const int col = (kb < ka ? kb : kb - ka) * GH_BLOCK_K;
          if (!diag) tma_load_2d(dst, map, &full[stage], col, r1);
          tma_load_2d(dst + GW_A_BYTES, map, &full[stage], col, r2);
          tma_load_2d(dst + GW_A_BYTES + GW_A_BYTES, map, &full[stage], col, r2 + GH_TILE);
          issued_mask |= 1u << stage;
          issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
          if (++stage == GW_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        for (int s = 0; s < GW_STAGES; ++s)
          if (issued_mask & (1u << s)) {
            int dummy_abort = 0;
            mbar_wait(&full[s], (issued_phase >> s) & 1u, &dummy_abort, p.status, OB_ERR_DRAIN, budget);
          }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(GH_TILE, GW_TILE_N, 0, 0);
      int stage = 0, acc_iter = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const GhostWideItem it = ghost_wide_decode(w, per_example, nt, ncb);
        int s0, len;
        segment(it.ex, s0, len);
        if (it.tb * GH_TILE >= len || it.cb * GW_TILE_N >= len) continue;
        // on a diagonal super-block the A operand is read from the copy of that row block inside the B operand
        const uint32_t a_off = (it.tb >> 1) == it.cb ? static_cast<uint32_t>(GW_A_BYTES + (it.tb & 1) * GW_A_BYTES) : 0u;
        if (!mbar_wait(tmem_empty, (acc_iter & 1) ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY, budget)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL, budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t st0 = smem_u32(smem + stage * GW_STAGE_BYTES);
          const uint32_t t1 = st0 + a_off, t2 = st0 + GW_A_BYTES;
          const uint32_t d_tmem = tmem_base + (kb < ka ? 0 : GW_TILE_N);
          const bool first = (kb == 0) || (kb == ka);
#pragma unroll
          for (int kk = 0; kk < GH_BLOCK_K / 16; ++kk) {
            const uint64_t ad = make_smem_desc(t1 + kk * 32, 16, 1024, 2);
            const uint64_t bd = make_smem_desc(t2 + kk * 32, 16, 1024, 2);
            umma_bf16(d_tmem, ad, bd, idesc, (first && kk == 0) ? 0u : 1u);
          }
          umma_commit(&empty[stage]);
          if (++stage == GW_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(tmem_full);
        ++acc_iter;
      }
    }
  } else {
    const int q = warp & 3;                  // TMEM lane quadrant
    const int half = (warp - 2) >> 2;        // which of the two 128-column blocks
    int acc_iter = 0;
    bool ok = true;
    for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      const GhostWideItem it = ghost_wide_decode(w, per_example, nt, ncb);
      int s0, len;
      segment(it.ex, s0, len);
      if (it.tb * GH_TILE >= len || it.cb * GW_TILE_N >= len) continue;
      if (!mbar_wait(tmem_full, acc_iter & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL, budget)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int cblk = 2 * it.cb + half;
      const float weight = cblk < it.tb ? 0.f : (cblk == it.tb ? 1.f : 2.f);
      const int t = it.tb * GH_TILE + q * 32 + lane;
      float acc = 0.f;
      if (weight != 0.f && cblk * GH_TILE < len) {
        const int my_id = (p.ids && t < len) ? p.ids[s0 + t] : -1;
        for (int c = 0; c < GH_TILE / 32; ++c) {
          float sg[32], sa[32];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * GH_TILE + c * 32;
          tmem_ld32(taddr + GW_TILE_N, sg);
          if (!p.ids) tmem_ld32(taddr, sa);
          tmem_ld_wait();
          const int tc0 = cblk * GH_TILE + c * 32;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int t2 = tc0 + j;
            float a;
            if (p.ids) {
              const int other = (t2 < len) ? __ldg(p.ids + s0 + t2) : -2;
              a = (other == my_id) ? 1.f : 0.f;
            } else {
              a = sa[j];
            }
            if (t < len && t2 < len) acc += a * sg[j];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty);
      ++acc_iter;
      acc = warp_sum(acc);
      if (lane == 0 && acc != 0.f) atomicAdd(p.norm2 + (p.seg_out ? p.seg_out[it.ex] : it.ex), weight * acc);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace ob

// 1 (default): 128 x 256 Gram blocks for examples of >= 1024 rows; 2: whenever an example spans two row blocks;
// 0: always 128 x 128 blocks
static int wide_enabled = 1;
extern "C" int ob_ghost_set_wide(int enabled) {
  const int old = wide_enabled;
  wide_enabled = enabled;
  return old;
}

extern "C" int ob_ghost_norm(const void* a, const void* g, const int* ids, int B, int T, int Da, int Dg,
                             long long lda, long long ldg, float* norm2, const int* seg, const int* seg_out,
                             long long total_rows, int* status, double wait_budget_s, int num_sms, void* stream) {
  using namespace ob;
  if (B <= 0 || T <= 0 || Dg <= 0) return 0;
  const long long rows = seg ? total_rows : static_cast<long long>(B) * T;
  if (rows <= 0) return 0;
  CUtensorMap ma, mg;
  int rc = make_bf16_map_2d(&mg, g, rows, Dg, ldg, GH_BLOCK_K, GH_TILE);
  if (rc) return rc;
  if (ids == nullptr) {
    rc = make_bf16_map_2d(&ma, a, rows, Da, lda, GH_BLOCK_K, GH_TILE);
    if (rc) return rc;
  } else {
    ma = mg;
  }
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(ghost_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GH_SMEM) != cudaSuccess)
      return -20;
    configured = true;
  }
  GhostParams p;
  p.B = B; p.T = T; p.Da = Da; p.Dg = Dg;
  p.ids = ids;
  p.seg = seg;
  p.seg_out = seg_out;
  p.norm2 = norm2;
  p.status = status;
  p.wait_budget_ns = static_cast<unsigned long long>(wait_budget_s * 1e9);
  const int nt = (T + GH_TILE - 1) / GH_TILE;
  // measured: the wide blocks win from about 1024 rows per example (less wasted work below the diagonal); below that
  // the 128 x 128 blocks with double-buffered accumulators are as fast or faster
  if (wide_enabled == 2 ? nt >= 2 : (wide_enabled == 1 && nt >= 8)) {
    static bool configured_wide = false;
    if (!configured_wide) {
      if (cudaFuncSetAttribute(ghost_norm_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GW_SMEM) != cudaSuccess)
        return -22;
      configured_wide = true;
    }
    const int ncb = (nt + 1) / 2;
    long long per_example = 0;
    for (int tb = 0; tb < nt; ++tb) per_example += ncb - (tb >> 1);
    const long long total = static_cast<long long>(B) * per_example;
    const int grid = static_cast<int>(total < num_sms ? total : num_sms);
    ghost_norm_wide_kernel<<<grid, GW_THREADS, GW_SMEM, static_cast<cudaStream_t>(stream)>>>(ma, mg, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -21;
  }
  const long long total = static_cast<long long>(B) * (nt * (nt + 1) / 2);
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  ghost_norm_kernel<<<grid, GH_THREADS, GH_SMEM, static_cast<cudaStream_t>(stream)>>>(ma, mg, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
