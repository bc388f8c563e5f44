// Dense forward / data-gradient GEMM on CTA pairs (sm_100a, tcgen05 cta_group::2):
//
//     D[M, N] = A[M, K1] * op1(B) + A2[M, K2] * op2(B2) + bias          (bf16 in / bf16 out, fp32 accumulation)
//
// Two CTAs of a 2x1 cluster share one 512 x 256 output tile.  Each CTA loads ITS OWN 256 rows of A and ITS OWN half
// (128 columns of N) of the B tile with ordinary TMA copies of this GPU's memory; one thread of the leader CTA
// (cluster rank 0) issues `tcgen05.mma.cta_group::2` (M = 256 across the pair) over both CTAs' shared memory, twice per
// k-step: once for each 128-row half of a CTA's A tile, each half with its own 256-column accumulator in that CTA's tensor
// memory.  Per k-block an SM stages 48 KB for 2 x (128 x 256 x 64) of tensor work: half the bytes per FLOP of a single-CTA
// 128 x 256 tile.  Measured need for it: with 32 KB per (128 x 256 x 64) the tensor pipe was 81 % busy at 11.4 TB/s of
// L2-to-SM traffic, whatever the number of stages.
//
// Protocol (every wait bounded; a timeout records a code in the status word and the kernel unwinds):
//   * full[s]  (leader only, 1 arrival + 96 KB of transactions): the leader's producer arms it for both CTAs' bytes;
//     the peer's producer points its copies' completion at the leader's barrier (shared::cluster address from `mapa`).
//   * empty[s] (each CTA, 1 arrival): the leader's `tcgen05.commit` arrives at both CTAs' barriers at once.
//   * tmem_full[h] (each CTA, 1 arrival, h = accumulator half): same two-CTA commit after the last k-block of a tile.
//   * tmem_empty[h] (leader only, 16 arrivals): the eight epilogue warps of both CTAs; the peer's arrive remotely.
//     All warps drain half 0 first, then half 1, and the next tile begins with half-0 work (see the MMA issuer).
// No copy in this file uses cluster multicast.
//
// Epilogues: plain store (+ bias), or GLU: the B halves come from TWO weight matrices (gate rows to rank 0, up rows to
// rank 1), so every accumulator row holds 128 gate and 128 up pre-activations and the epilogue writes
// act(gate) * up, optionally together with gate and up themselves for the backward pass.
// Second K segment: LoRA (x A^T)(s B)^T in the forward pass, or the second operand pair of dX = dG Wg + dU Wu.
//
// Reference counterpart: the library GEMMs inside packages/opaque-patches/src/opaque/api/patches/kernels/lora.py:217-293
// and the gate/up/SwiGLU sequence of kernels/swiglu.py:29-58.
#include "common.cuh"
#include "api.h"
#include "die_map.cuh"

#include <atomic>
#include <cstdlib>

namespace ob {

int make_bf16_map_2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                     int box_cols, int box_rows);

constexpr int GP_BM = 256;           // rows of M per CTA (512 per pair tile): two 128-row halves, one accumulator each
constexpr int GP_MMA_M = 128;        // rows of one accumulator per CTA (the pair instruction has M = 256)
constexpr int GP_BN = 256;           // accumulator columns per pair tile
constexpr int GP_BNH = 128;          // columns of N whose B rows one CTA stages
constexpr int GP_BK = 64;
#ifndef OB_PAIR_STAGES
#define OB_PAIR_STAGES 4
#endif
#ifndef OB_PAIR_INTERLEAVE
#define OB_PAIR_INTERLEAVE 1
#endif
#ifndef OB_PAIR_RELAXED
#define OB_PAIR_RELAXED 0
#endif
constexpr int GP_STAGES = OB_PAIR_STAGES;
constexpr int GP_A_BYTES = GP_BM * GP_BK * 2;
constexpr int GP_B_BYTES = GP_BNH * GP_BK * 2;
constexpr int GP_STAGE_BYTES = GP_A_BYTES + GP_B_BYTES;
constexpr int GP_THREADS = 320;       // TMA warp, MMA warp, 2 x 4 epilogue warps
constexpr int GP_GROUP_M = 8;        // pair tiles (512 rows each) per raster band (measured: 8 >= 4 > 16 on the MLP shapes)
constexpr int GP_SLAB_BYTES = 4096;   // per epilogue warp: a 32-row x 64-column (or 2 x 32-column) bf16 staging tile
constexpr int GP_SMEM = GP_STAGES * GP_STAGE_BYTES + 8 * GP_SLAB_BYTES + 256 + 1024;

enum : int { GP_EPI_STORE = 0, GP_EPI_GLU = 1, GP_EPI_CE = 2, GP_EPI_GLUBWD = 3 };

struct PairParams {
  int M, N, K1, K2;
  int kn1, kn2;                      // 1: the segment's B operand is stored [K, N] (N-major), 0: [N, K]
  __nv_bfloat16* out;                // STORE: [M, N];  GLU: [M, N / 2] activations
  long long ldo;
  __nv_bfloat16* out_gate;           // GLU only, optional: pre-activations, pitch ldo
  __nv_bfloat16* out_up;
  const __nv_bfloat16* bias;         // STORE only
  int act;                           // GLU: 0 silu, 1 gelu (erf), 2 gelu (tanh)
  int group_m;                       // pair tiles (512 rows each) per raster band
  // CE epilogue (output head + cross-entropy statistics; `out` optional: the bf16, soft-capped logits)
  const long long* labels;           // [M]
  float4* ce_partials;               // [M, tiles_n]: (max, sum exp(z - max), z[label] or 0, sum z) over the tile's columns
  float softcap;                     // > 0: z = softcap * tanh(z / softcap)
  int* status;
  unsigned long long wait_budget_ns;
  int tma_store;                     // STORE: the output leaves through bulk tensor stores (map_out is valid)
  // GLU-backward epilogue (data gradient of a gated MLP's down projection): the accumulator is dH; with the stored
  // pre-activations it becomes dGate (-> out) and dUp (-> out_up) without dH ever reaching memory
  const __nv_bfloat16* glu_g;        // [M, N] gate pre-activations, pitch ld_gu
  const __nv_bfloat16* glu_u;        // [M, N] up pre-activations
  long long ld_gu;
  // Die-aware tile assignment (see gp_schedule); claim == nullptr: cluster c simply takes tiles c, c + clusters, ...
  unsigned long long* claim;         // this launch's claim word (zero on entry, zero again after the last claim)
  int n_front;                       // clusters expected on die 0: slots [0, n_front) walk tiles [0, split)
  int split;                         //   and slots [n_front, clusters) walk tiles [split, total)
};

// ---------------------------------------------------------------------------------------------- cluster helpers
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load issued by one CTA of a pair; the completion bytes go to `bar_cluster_addr`, which may be the peer's.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival at the barrier at this shared-memory offset in EVERY CTA of `cta_mask`, once all MMAs issued so far
// by this thread have finished (an mbarrier signal, not a data copy).
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(cta_mask)
               : "memory");
}

// Tile assignment of one cluster: tiles first, first + stride, ... < end (in raster order).
//
// A B200 is two dies, each with its own half of the L2; a tile operand that an SM finds only in the other die's half
// costs a trip over the die-to-die link (2.4x the latency, measured).  Tiles that are adjacent in raster order share
// their A rows or B columns, so the clusters of one die should work on one contiguous range of the raster and the
// clusters of the other die on the rest: each die then pulls the remote-homed half of ITS operands once, instead of
// both dies pulling everything.  Which die a cluster sits on is only known once it runs (%smid and the probed map of
// die_map.cuh), so the assignment is claimed at start-up: clusters on die 0 take slots from the front of [0, clusters),
// clusters on die 1 from the back, with ONE 64-bit atomic each (low word: front claims so far, high word: back claims).
// Exactly `clusters` claims are made per launch, so every slot is taken exactly once whatever the placement; a cluster
// that finds the slots of its own die exhausted simply gets one of the other range.  The last claimer zeroes the word.
struct GpSchedule {
  int first, end, stride;
};

__device__ __forceinline__ GpSchedule gp_claim_schedule(const PairParams& p, int total_work, int cluster_id,
                                                        int num_clusters) {
  GpSchedule s;
  s.first = cluster_id;
  s.end = total_work;
  s.stride = num_clusters;
  if (p.claim == nullptr) return s;
  unsigned smid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  const int die = g_sm_die[smid & (DM_MAX_SMS - 1)];
  const unsigned long long old = atomicAdd(p.claim, die ? (1ull << 32) : 1ull);
  const int lo = static_cast<int>(old & 0xffffffffull), hi = static_cast<int>(old >> 32);
  if (lo + hi == num_clusters - 1) atomicExch(p.claim, 0ull);
  const int slot = die ? num_clusters - 1 - hi : lo;
  if (lo + hi >= num_clusters || slot < 0 || slot >= num_clusters) {
    // more claims than clusters: the word was shared with another launch in flight; refuse to compute anything
    set_error(p.status, OB_ERR_CLAIM);
    s.first = s.end = 0;
    return s;
  }
  if (slot < p.n_front) {
    s.first = slot;
    s.stride = p.n_front;
    s.end = p.split;
  } else {
    s.first = p.split + (slot - p.n_front);
    s.stride = num_clusters - p.n_front;
    s.end = total_work;
  }
  return s;
}

// Every role of both CTAs reads the schedule from the LEADER's shared memory (written before the start-up cluster barrier).
__device__ __forceinline__ GpSchedule gp_read_schedule(const int* sched_local) {
  const uint32_t a = map_to_cta(smem_u32(sched_local), 0);
  GpSchedule s;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(s.first) : "r"(a) : "memory");
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(s.end) : "r"(a + 4) : "memory");
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(s.stride) : "r"(a + 8) : "memory");
  return s;
}

// Wait used by roles that are far from the critical path (epilogue warps waiting a whole main loop for their tile): the
// polling thread sleeps between tries, which leaves issue slots and power to the tensor pipe.
__device__ __forceinline__ bool mbar_wait_idle(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                               int code, uint64_t budget_ns) {
#if OB_PAIR_RELAXED
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    __nanosleep(OB_PAIR_RELAXED);
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > budget_ns) {
        *abort_flag = 1;
        set_error(status, code);
        return false;
      }
    }
  }
#else
  return mbar_wait(bar, parity, abort_flag, status, code, budget_ns);
#endif
}

struct GpItem {
  int row0;      // first row of this CTA's half of the pair tile
  int nt;        // tile index along N
};

__device__ __forceinline__ GpItem gp_decode(int w, int tiles_m, int tiles_n, int rank, int group_m) {
  const int band = group_m * tiles_n;
  const int b = w / band, r = w % band;
  const int m_in_band = min(group_m, tiles_m - b * group_m);
  const int mt = b * group_m + r % m_in_band;
  GpItem it;
  it.row0 = mt * (2 * GP_BM) + rank * GP_BM;
  it.nt = r / m_in_band;
  return it;
}

// The activation is a compile-time choice inside the loops that use it: with a run-time selector per element the
// compiler evaluated all three (erf and tanh expansions included) for every value and selected afterwards, which made
// the GLU drain six times longer than its stores.
template <int ACT>
__device__ __forceinline__ float gp_act(float g) {
  if constexpr (ACT == 0) return g / (1.0f + __expf(-g));
  if constexpr (ACT == 1) return 0.5f * g * (1.0f + erff(g * 0.70710678118654752f));
  const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
  return 0.5f * g * (1.0f + t);
}

// Value and derivative of the gate activation (compile-time choice, see gp_act).
template <int ACT>
__device__ __forceinline__ void gp_act_grad(float g, float& a, float& da) {
  if constexpr (ACT == 0) {
    const float sg = 1.0f / (1.0f + __expf(-g));
    a = g * sg;
    da = sg * (1.0f + g * (1.0f - sg));
  } else if constexpr (ACT == 1) {
    const float cdf = 0.5f * (1.0f + erff(g * 0.70710678118654752f));
    a = g * cdf;
    da = cdf + g * 0.3989422804014327f * __expf(-0.5f * g * g);
  } else {
    const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
    a = 0.5f * g * (1.0f + t);
    da = 0.5f * (1.0f + t) + 0.5f * g * (1.0f - t * t) * 0.7978845608028654f * (1.0f + 0.134145f * g * g);
  }
}

// 64 columns of one row: packed bf16 dH (pd) and the row's gate / up pre-activations (16-byte loads) -> packed
// dGate = dH * up * act'(gate) and dUp = dH * act(gate).  dH enters bf16-rounded, as it would from memory.
template <int ACT>
__device__ __forceinline__ void gp_glu_bwd64(const uint32_t* pd, const __nv_bfloat16* grow, const __nv_bfloat16* urow,
                                             bool in_row, uint32_t* og, uint32_t* ou) {
#pragma unroll
  for (int s8 = 0; s8 < 8; ++s8) {
    uint4 g4 = make_uint4(0u, 0u, 0u, 0u), u4 = g4;
    if (in_row) {
      g4 = __ldg(reinterpret_cast<const uint4*>(grow) + s8);
      u4 = __ldg(reinterpret_cast<const uint4*>(urow) + s8);
    }
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t d2 = pd[4 * s8 + j];
      const float dx = __uint_as_float(d2 << 16), dy = __uint_as_float(d2 & 0xffff0000u);
      const float gx = __uint_as_float(gw[j] << 16), gy = __uint_as_float(gw[j] & 0xffff0000u);
      const float ux = __uint_as_float(uw[j] << 16), uy = __uint_as_float(uw[j] & 0xffff0000u);
      float ax, dax, ay, day;
      gp_act_grad<ACT>(gx, ax, dax);
      gp_act_grad<ACT>(gy, ay, day);
      og[4 * s8 + j] = pack_bf16x2(dx * ux * dax, dy * uy * day);
      ou[4 * s8 + j] = pack_bf16x2(dx * ax, dy * ay);
    }
  }
}

// pkg[j] <- bf16x2(act(g) * u) from packed bf16 pairs of g and u (32 registers = 64 values per lane)
template <int ACT>
__device__ __forceinline__ void gp_glu_inplace(uint32_t* pkg, const uint32_t* pku) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float gx = __uint_as_float(pkg[j] << 16), gy = __uint_as_float(pkg[j] & 0xffff0000u);
    const float ux = __uint_as_float(pku[j] << 16), uy = __uint_as_float(pku[j] & 0xffff0000u);
    pkg[j] = pack_bf16x2(gp_act<ACT>(gx) * ux, gp_act<ACT>(gy) * uy);
  }
}

// Cross-entropy statistics of 64 logits per lane, given as 32 packed bf16 pairs: running maximum m, sum of exp(z - m),
// the label's logit and the plain sum.  FULL: all 64 columns lie inside the vocabulary (no per-column checks).
// Two accumulators per quantity keep the dependent chains short; exp is one FFMA + ex2.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <bool FULL>
__device__ __forceinline__ void ce_fold64(const uint32_t* pk, int nc, int N, int lab, float& m, float& ssum, float& zlab,
                                          float& ztot) {
  constexpr float LOG2E = 1.4426950408889634f;
  float lm0 = -INFINITY, lm1 = -INFINITY, t0 = 0.f, t1 = 0.f;
  const int d = lab - nc;                                  // position of the label inside this round, if 0 <= d < 64
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float x = __uint_as_float(pk[j] << 16), y = __uint_as_float(pk[j] & 0xffff0000u);
    if (FULL || nc + 2 * j < N) {
      t0 += x;
      lm0 = fmaxf(lm0, x);
    }
    if (FULL || nc + 2 * j + 1 < N) {
      t1 += y;
      lm1 = fmaxf(lm1, y);
    }
    if (d == 2 * j) zlab = x;
    if (d == 2 * j + 1) zlab = y;
  }
  ztot += t0 + t1;
  const float lm = fmaxf(lm0, lm1);
  if (lm > m) {
    ssum *= ex2_approx((m - lm) * LOG2E);                 // m = -inf on the first round: ex2(-inf) = 0
    m = lm;
  }
  const float ml = m * LOG2E;
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float x = __uint_as_float(pk[j] << 16), y = __uint_as_float(pk[j] & 0xffff0000u);
    if (FULL || nc + 2 * j < N) s0 += ex2_approx(fmaf(x, LOG2E, -ml));
    if (FULL || nc + 2 * j + 1 < N) s1 += ex2_approx(fmaf(y, LOG2E, -ml));
  }
  ssum += s0 + s1;
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GP_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_b_up, const __grid_constant__ CUtensorMap map_a2,
                 const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_b2_up,
                 const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_out_gate,
                 const __grid_constant__ CUtensorMap map_out_up, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared-memory window starts at the same offset in both CTAs, so the rounded offsets agree too
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* slabs = smem + GP_STAGES * GP_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(slabs + 8 * GP_SLAB_BYTES);
  uint64_t* full = bars;                               // used in the leader CTA only
  uint64_t* empty = bars + GP_STAGES;
  uint64_t* tmem_full = bars + 2 * GP_STAGES;          // [2]: one per accumulator half
  uint64_t* tmem_empty = bars + 2 * GP_STAGES + 2;     // [2], used in the leader CTA only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GP_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* sched = reinterpret_cast<int*>(tmem_slot + 2);  // [3]: first, end, stride (valid in the leader CTA)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int tiles_n = EPI == GP_EPI_GLU ? (p.N / 2 + GP_BNH - 1) / GP_BNH : (p.N + GP_BN - 1) / GP_BN;
  const int tiles_m = (p.M + 2 * GP_BM - 1) / (2 * GP_BM);
  const int total_work = tiles_m * tiles_n;
  const int nk1 = (p.K1 + GP_BK - 1) / GP_BK;
  const int nk2 = (p.K2 + GP_BK - 1) / GP_BK;
  const int num_kb = nk1 + nk2;
  const uint64_t budget = p.wait_budget_ns;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GP_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 16);                   // eight epilogue warps in each CTA
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(rank == 1 && EPI == GP_EPI_GLU ? &map_b_up : &map_b);
    if (nk2) {
      tma_prefetch_desc(&map_a2);
      tma_prefetch_desc(rank == 1 && EPI == GP_EPI_GLU ? &map_b2_up : &map_b2);
    }
  }
  if (warp == 1) {                   // one warp of EACH CTA takes part in a pair allocation
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  if (leader && threadIdx.x == 64) {  // a thread with nothing else to do during start-up claims the cluster's tiles
    const GpSchedule sc = gp_claim_schedule(p, total_work, cluster_id, num_clusters);
    sched[0] = sc.first;
    sched[1] = sc.end;
    sched[2] = sc.stride;
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                // both CTAs' barriers are initialised before any remote arrival or copy
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const GpSchedule sc = gp_read_schedule(sched);

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer (one per CTA)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const CUtensorMap* mb1 = (EPI == GP_EPI_GLU && rank == 1) ? &map_b_up : &map_b;
      const CUtensorMap* mb2 = (EPI == GP_EPI_GLU && rank == 1) ? &map_b2_up : &map_b2;
      for (int w = sc.first; ok && w < sc.end; w += sc.stride) {
        const GpItem it = gp_decode(w, tiles_m, tiles_n, rank, p.group_m);
        // first column of N (= row of a [N, K] operand) of this CTA's half of the B tile
        const int bn0 = EPI == GP_EPI_GLU ? it.nt * GP_BNH : it.nt * GP_BN + static_cast<int>(rank) * GP_BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_EMPTY, budget)) {
            ok = false;
            break;
          }
          if (leader) mbar_expect_tx(&full[stage], 2 * GP_STAGE_BYTES);
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          uint8_t* a_dst = smem + stage * GP_STAGE_BYTES;
          uint8_t* b_dst = a_dst + GP_A_BYTES;
          const bool first = kb < nk1;
          const int k0 = (first ? kb : kb - nk1) * GP_BK;
          tma_load_2d_pair(a_dst, first ? &map_a : &map_a2, bar, k0, it.row0);          // 256 rows x 64 k in one box
          const CUtensorMap* mb = first ? mb1 : mb2;
          if (first ? p.kn1 : p.kn2) {
#pragma unroll
            for (int j = 0; j < GP_BNH / 64; ++j)
              tma_load_2d_pair(b_dst + j * (GP_BK * 128), mb, bar, bn0 + 64 * j, k0);
          } else {
            tma_load_2d_pair(b_dst, mb, bar, k0, bn0);
          }
          if (++stage == GP_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer (leader CTA only)
      // Each CTA holds 256 rows of A per stage: two 128-row halves, one accumulator (256 TMEM columns) each, both
      // multiplied with the SAME B tile, so a stage's 48 KB feed 2 x (128 x 256 x 64) of work per SM.
      // The two accumulators fill all of tensor memory, so a tile's epilogue cannot hide behind the next tile's whole
      // main loop.  It hides behind its first k-blocks instead: the epilogue warps drain half 0 first, and the next
      // tile starts with the half-0 products of its first GP_STAGES k-blocks while half 1 is still being drained.
      constexpr uint32_t idesc_k = make_idesc_bf16(2 * GP_MMA_M, GP_BN, 0, 0);
      constexpr uint32_t idesc_n = make_idesc_bf16(2 * GP_MMA_M, GP_BN, 0, 1);
      int stage = 0, acc_iter = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto issue_one = [&](int h, int kb, int st, int kk) {
        const uint32_t a_addr = smem_u32(smem + st * GP_STAGE_BYTES);
        const uint32_t b_addr = a_addr + GP_A_BYTES;
        const bool kn = kb < nk1 ? p.kn1 != 0 : p.kn2 != 0;
        // K-major operand: rows 128 B apart, 8-row groups 1024 B apart, 32 B per 16-element k-step.
        // N-major operand: 64-column blocks GP_BK*128 B apart, 8-row (k) groups 1024 B apart, 2048 B per k-step.
        const uint64_t ad = make_smem_desc(a_addr + h * (GP_MMA_M * 128) + kk * 32, 16, 1024, 2);
        const uint64_t bd = kn ? make_smem_desc(b_addr + kk * (16 * 128), GP_BK * 128, 1024, 2)
                               : make_smem_desc(b_addr + kk * 32, 16, 1024, 2);
        umma_bf16_pair(tmem_base + h * GP_BN, ad, bd, kn ? idesc_n : idesc_k, (kb > 0 || kk > 0) ? 1u : 0u);
      };
      auto issue_half = [&](int h, int kb, int st) {
#pragma unroll
        for (int kk = 0; kk < GP_BK / 16; ++kk) issue_one(h, kb, st, kk);
        if (kb == num_kb - 1) umma_commit_pair(&tmem_full[h], 3);   // this half's accumulators (both CTAs) are complete
      };
      // steady state: the two accumulators alternate k-step by k-step, so no instruction waits on the one before it
      auto issue_both = [&](int kb, int st) {
#if OB_PAIR_INTERLEAVE
#pragma unroll
        for (int kk = 0; kk < GP_BK / 16; ++kk) {
          issue_one(0, kb, st, kk);
          issue_one(1, kb, st, kk);
        }
        if (kb == num_kb - 1) {
          umma_commit_pair(&tmem_full[0], 3);
          umma_commit_pair(&tmem_full[1], 3);
        }
#else
        issue_half(0, kb, st);
        issue_half(1, kb, st);
#endif
      };
      for (int w = sc.first; ok && w < sc.end; w += sc.stride) {
        const uint32_t acc_parity = static_cast<uint32_t>(acc_iter & 1);
        const int lead = num_kb < GP_STAGES ? num_kb : GP_STAGES;
        // head of the tile: half 0 of the first `lead` k-blocks, then half 1 of the same stages
        for (int i = 0; ok && i < lead; ++i) {
          int st = stage + i;
          uint32_t ph = phase;
          if (st >= GP_STAGES) { st -= GP_STAGES; ph ^= 1; }
          if (!mbar_wait(&full[st], ph, abort_flag, p.status, OB_ERR_WAIT_FULL, budget)) { ok = false; break; }
          if (i == 0 && !mbar_wait(&tmem_empty[0], acc_parity ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY, budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_half(0, i, st);
        }
        for (int i = 0; ok && i < lead; ++i) {
          if (i == 0) {
            if (!mbar_wait(&tmem_empty[1], acc_parity ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY, budget)) {
              ok = false;
              break;
            }
            tc_fence_after();
          }
          issue_half(1, i, stage);
          umma_commit_pair(&empty[stage], 3);          // frees the stage in both CTAs
          if (++stage == GP_STAGES) { stage = 0; phase ^= 1; }
        }
        // tail of the tile, the mirror image: half 0 finishes its last `tail` k-blocks first and is handed to the epilogue
        // while half 1 still has `tail` k-blocks of work on the same (still resident) stages, so the tensor pipe is busy
        // during the drain of half 0, and the drain of half 1 overlaps the head of the next tile.
        const int tail = num_kb - lead < GP_STAGES ? num_kb - lead : GP_STAGES;
        for (int kb = lead; ok && kb < num_kb - tail; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL, budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_both(kb, stage);
          umma_commit_pair(&empty[stage], 3);
          if (++stage == GP_STAGES) { stage = 0; phase ^= 1; }
        }
        for (int i = 0; ok && i < tail; ++i) {
          int st = stage + i;
          uint32_t ph = phase;
          if (st >= GP_STAGES) { st -= GP_STAGES; ph ^= 1; }
          if (!mbar_wait(&full[st], ph, abort_flag, p.status, OB_ERR_WAIT_FULL, budget)) { ok = false; break; }
          tc_fence_after();
          issue_half(0, num_kb - tail + i, st);
        }
        for (int i = 0; ok && i < tail; ++i) {
          issue_half(1, num_kb - tail + i, stage);
          umma_commit_pair(&empty[stage], 3);
          if (++stage == GP_STAGES) { stage = 0; phase ^= 1; }
        }
        ++acc_iter;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (8 per CTA)
    // Warp (q, g): TMEM lane quarter q = warp % 4 (the only lanes a warp may read), column group g = 0 for warps 2-5 and
    // 1 for warps 6-9.  All eight warps drain accumulator half 0 first (each its own rows and columns), release it, then
    // half 1: the tensor pipe gets half 0 back after half the drain time.
    const int q = warp & 3;
    const int g = (warp - 2) >> 2;
    uint8_t* slab = slabs + (warp - 2) * GP_SLAB_BYTES;
    int acc_iter = 0;
    bool ok = true;
    const bool vec_ok = ((p.ldo & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        (EPI != GP_EPI_GLU || p.out_gate == nullptr ||
                         (((reinterpret_cast<uintptr_t>(p.out_gate) | reinterpret_cast<uintptr_t>(p.out_up)) & 15) == 0)) &&
                        (EPI != GP_EPI_GLUBWD || (reinterpret_cast<uintptr_t>(p.out_up) & 15) == 0);
    for (int w = sc.first; ok && w < sc.end; w += sc.stride) {
      const GpItem it = gp_decode(w, tiles_m, tiles_n, rank, p.group_m);
      auto release_half = [&](int hh) {          // this warp is done READING accumulator half hh
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive(&tmem_empty[hh]);
          else mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[hh]), 0));
        }
      };
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        if (!mbar_wait_idle(&tmem_full[h], acc_iter & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL, budget)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int row = it.row0 + h * GP_MMA_M + q * 32 + lane;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + h * GP_BN;
        if constexpr (EPI == GP_EPI_STORE) {
          // Both 64-column rounds of this warp's share go to registers (packed bf16) first, so the accumulator half is
          // back with the tensor pipe before a single store is issued; the stores then overlap the next MMAs.
          const int n0 = it.nt * GP_BN + g * (GP_BN / 2);
          const int row0w = row - lane;
          uint32_t pk[2][32];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int nc = n0 + c * 64;
            if (nc < p.N) {
              float v[64];
              tmem_ld32(t_row + g * (GP_BN / 2) + c * 64, v);
              tmem_ld32(t_row + g * (GP_BN / 2) + c * 64 + 32, v + 32);
              tmem_ld_wait();
              if (p.bias != nullptr) add_bias64(v, p.bias, nc, p.N);
#pragma unroll
              for (int j = 0; j < 32; ++j) pk[c][j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
            }
          }
          release_half(h);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int nc = n0 + c * 64;
            if (nc < p.N)
              store_tile64_packed(slab, pk[c], &map_out, p.tma_store != 0, nc, row0w, p.out, p.ldo, p.M - row0w, p.N - nc,
                                  vec_ok, lane);
          }
        } else if constexpr (EPI == GP_EPI_CE) {
          // Output head: the logits tile never leaves the SM unless `out` asks for it.  Each thread owns one row and folds
          // its 128 columns of the tile into (max, sum exp, label logit, plain sum); the partials (two per tile and row)
          // are combined per row in a fixed order by lce_combine_kernel, so the result does not depend on which CTA ran
          // which tile.
          const int n0 = it.nt * GP_BN + g * (GP_BN / 2);
          const long long label = row < p.M ? p.labels[row] : -1;
          const int lab = (label >= 0 && label < p.N) ? static_cast<int>(label) : -(1 << 30);     // never matches a column
          float m = -INFINITY, ssum = 0.f, zlab = 0.f, ztot = 0.f;
          if (p.out != nullptr) {
            // Training: the logits are stored (bf16) for the backward pass, and the statistics are taken from the stored,
            // rounded values.  So the accumulator is read, soft-capped and packed to bf16 first and handed back; the
            // exponentials and the stores then run beside the next tile's MMAs (with K = 768 the drain of a tile is
            // otherwise longer than its main loop).
            const int row0w = row - lane;
            uint32_t pk[2][32];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const int nc = n0 + c * 64;
              if (nc < p.N) {
                float v[64];
                tmem_ld32(t_row + g * (GP_BN / 2) + c * 64, v);
                tmem_ld32(t_row + g * (GP_BN / 2) + c * 64 + 32, v + 32);
                tmem_ld_wait();
                if (p.softcap > 0.f) {
#pragma unroll
                  for (int j = 0; j < 64; ++j) v[j] = p.softcap * tanhf(v[j] / p.softcap);
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) pk[c][j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
              }
            }
            release_half(h);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const int nc = n0 + c * 64;
              if (nc < p.N) {
                if (nc + 64 <= p.N) ce_fold64<true>(pk[c], nc, p.N, lab, m, ssum, zlab, ztot);
                else ce_fold64<false>(pk[c], nc, p.N, lab, m, ssum, zlab, ztot);
                store_tile64_packed(slab, pk[c], &map_out, p.tma_store != 0, nc, row0w, p.out, p.ldo, p.M - row0w, p.N - nc,
                                    vec_ok, lane);
              }
            }
          } else {
            // Forward only (evaluation, reference log-probabilities): fp32 statistics, nothing stored.
#pragma unroll 1
            for (int c = 0; c < GP_BN / 2 / 32; ++c) {
              const int nc = n0 + c * 32;
              if (nc >= p.N) break;
              float v[32];
              tmem_ld32(t_row + g * (GP_BN / 2) + c * 32, v);
              tmem_ld_wait();
              if (p.softcap > 0.f) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = p.softcap * tanhf(v[j] / p.softcap);
              }
              float lm = -INFINITY;
              const int d = lab - nc;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const bool in = nc + j < p.N;
                const float z = v[j];
                v[j] = in ? z : -INFINITY;
                if (in) {
                  ztot += z;
                  lm = fmaxf(lm, z);
                }
                if (d == j) zlab = z;
              }
              if (lm > m) {
                ssum *= __expf(m - lm);
                m = lm;
              }
#pragma unroll
              for (int j = 0; j < 32; ++j) ssum += __expf(v[j] - m);      // exp(-inf) = 0 for masked columns
            }
            release_half(h);
          }
          if (row < p.M)
            p.ce_partials[static_cast<long long>(row) * (2 * tiles_n) + 2 * it.nt + g] = make_float4(m, ssum, zlab, ztot);
        } else if constexpr (EPI == GP_EPI_GLUBWD) {
          // Data gradient of the down projection with the gated activation's backward in the epilogue: the tile is dH;
          // it is read, rounded to bf16 and packed, the accumulator half goes back, and the row's gate / up
          // pre-activations turn it into dGate and dUp tiles, which leave through the slab.  N % 64 == 0 (host-checked).
          const int n0 = it.nt * GP_BN + g * (GP_BN / 2);
          const int row0w = row - lane;
          uint32_t pd[2][32];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int nc = n0 + c * 64;
            if (nc < p.N) {
              float v[64];
              tmem_ld32(t_row + g * (GP_BN / 2) + c * 64, v);
              tmem_ld32(t_row + g * (GP_BN / 2) + c * 64 + 32, v + 32);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) pd[c][j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
            }
          }
          release_half(h);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int nc = n0 + c * 64;
            if (nc < p.N) {
              const bool in_row = row < p.M;
              const __nv_bfloat16* grow = p.glu_g + static_cast<long long>(row) * p.ld_gu + nc;
              const __nv_bfloat16* urow = p.glu_u + static_cast<long long>(row) * p.ld_gu + nc;
              uint32_t og[32], ou[32];
              if (p.act == 0) gp_glu_bwd64<0>(pd[c], grow, urow, in_row, og, ou);
              else if (p.act == 1) gp_glu_bwd64<1>(pd[c], grow, urow, in_row, og, ou);
              else gp_glu_bwd64<2>(pd[c], grow, urow, in_row, og, ou);
              const bool tma = p.tma_store != 0;
              store_tile64_packed(slab, og, &map_out, tma, nc, row0w, p.out, p.ldo, p.M - row0w, p.N - nc, vec_ok, lane);
              store_tile64_packed(slab, ou, &map_out_up, tma, nc, row0w, p.out_up, p.ldo, p.M - row0w, p.N - nc, vec_ok, lane);
            }
          }
        } else {
          // GLU: this warp's 64 columns of h come from 64 gate and 64 up columns of the same rows.  Everything is read
          // and packed first (four rounds of 16 + 16 columns), the accumulator half is released, then up to three
          // [32 x 64] tiles (gate, up, h) leave through the slab.
          const int nh = p.N / 2;
          const int n0 = it.nt * GP_BNH + g * (GP_BNH / 2);
          const int row0w = row - lane;
          uint32_t pkg[32], pku[32];
#pragma unroll
          for (int c = 0; c < 4; ++c) {            // 16 + 16 columns per round: few fp32 registers in flight
            if (n0 + c * 16 < nh) {
              float gt[16], up[16];
              tmem_ld16(t_row + g * (GP_BNH / 2) + c * 16, gt);
              tmem_ld16(t_row + GP_BNH + g * (GP_BNH / 2) + c * 16, up);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                pkg[8 * c + j] = pack_bf16x2(gt[2 * j], gt[2 * j + 1]);
                pku[8 * c + j] = pack_bf16x2(up[2 * j], up[2 * j + 1]);
              }
            }
          }
          release_half(h);
          // h is formed from the ROUNDED pre-activations (what the backward pass reads when they are stored), after the
          // accumulator has gone back (the activation needs no tensor memory) and in place, to keep registers free
          if (n0 < nh) {
            const bool tma = p.tma_store != 0;
            if (p.out_gate != nullptr) {
              store_tile64_packed(slab, pkg, &map_out_gate, tma, n0, row0w, p.out_gate, p.ldo, p.M - row0w, nh - n0, vec_ok, lane);
              store_tile64_packed(slab, pku, &map_out_up, tma, n0, row0w, p.out_up, p.ldo, p.M - row0w, nh - n0, vec_ok, lane);
            }
            if (p.act == 0) gp_glu_inplace<0>(pkg, pku);
            else if (p.act == 1) gp_glu_inplace<1>(pkg, pku);
            else gp_glu_inplace<2>(pkg, pku);
            store_tile64_packed(slab, pkg, &map_out, tma, n0, row0w, p.out, p.ldo, p.M - row0w, nh - n0, vec_ok, lane);
          }
        }
      }
      ++acc_iter;
    }
    if (lane == 0) tma_store_wait_all();         // this lane's bulk stores are done before shared memory is given back
  }

  // Nobody leaves (or frees tensor memory) while the other CTA may still signal this CTA's barriers, complete copies
  // on them or accumulate into its tensor memory.
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up (after its whole budget), so some copies of this CTA may never be consumed.  They were issued at
    // least one budget ago and a tile copy lasts microseconds; one more millisecond lets any straggler land before the
    // shared memory is given back.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) {}
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Short-K variant: 256 x 256 pair tiles with DOUBLE-BUFFERED accumulators.
//
// The 512 x 256 kernel above fills tensor memory with one tile, so its drain hides only behind the first k-blocks of the
// next tile; with K = 768 (GPT-2's projections: 12 k-blocks) the drain is as long as the main loop and every SM pair
// stores at the same moment.  Here each CTA owns 128 rows and one 128 x 256 accumulator per tile (256 TMEM columns),
// two of them alternate, and the eight epilogue warps drain tile i during the whole main loop of tile i + 1.  A stage
// is 32 KB per CTA (128 rows of A, 128 columns' worth of B) for 128 x 256 x 64 of work: 64 bytes per tensor clock,
// against 96 for the single-CTA 128 x 256 tile and 48 for the 512 x 256 pair tile.  Plain store epilogue (+ bias,
// + second K segment) only.  Same barrier protocol and unwind rules as gemm_pair_kernel.
constexpr int GD_BM = 128;                              // rows of M per CTA (256 per pair)
constexpr int GD_STAGES = 6;
constexpr int GD_A_BYTES = GD_BM * GP_BK * 2;
constexpr int GD_B_BYTES = GP_BNH * GP_BK * 2;
constexpr int GD_STAGE_BYTES = GD_A_BYTES + GD_B_BYTES;
constexpr int GD_GROUP_M = 16;                          // pair tiles (256 rows each) per raster band
constexpr int GD_SMEM = GD_STAGES * GD_STAGE_BYTES + 8 * GP_SLAB_BYTES + 256 + 1024;
static_assert((2 * GD_STAGES + 4) * 8 + 8 <= 256, "barrier block");

__device__ __forceinline__ GpItem gd_decode(int w, int tiles_m, int tiles_n, int rank) {
  const int band = GD_GROUP_M * tiles_n;
  const int b = w / band, r = w % band;
  const int m_in_band = min(GD_GROUP_M, tiles_m - b * GD_GROUP_M);
  const int mt = b * GD_GROUP_M + r % m_in_band;
  GpItem it;
  it.row0 = mt * (2 * GD_BM) + rank * GD_BM;
  it.nt = r / m_in_band;
  return it;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GP_THREADS, 1)
gemm_pair_db_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
                    const __grid_constant__ CUtensorMap map_out, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* slabs = smem + GD_STAGES * GD_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(slabs + 8 * GP_SLAB_BYTES);
  uint64_t* full = bars;                               // used in the leader CTA only
  uint64_t* empty = bars + GD_STAGES;
  uint64_t* tmem_full = bars + 2 * GD_STAGES;          // [2]: one per accumulator buffer
  uint64_t* tmem_empty = bars + 2 * GD_STAGES + 2;     // [2], used in the leader CTA only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GD_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* sched = reinterpret_cast<int*>(tmem_slot + 2);  // [3]: first, end, stride (valid in the leader CTA)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int tiles_n = (p.N + GP_BN - 1) / GP_BN;
  const int tiles_m = (p.M + 2 * GD_BM - 1) / (2 * GD_BM);
  const int total_work = tiles_m * tiles_n;
  const int nk1 = (p.K1 + GP_BK - 1) / GP_BK;
  const int nk2 = (p.K2 + GP_BK - 1) / GP_BK;
  const int num_kb = nk1 + nk2;
  const uint64_t budget = p.wait_budget_ns;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GD_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 16);                   // eight epilogue warps in each CTA
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (nk2) {
      tma_prefetch_desc(&map_a2);
      tma_prefetch_desc(&map_b2);
    }
  }
  if (warp == 1) {                   // one warp of EACH CTA takes part in a pair allocation
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  if (leader && threadIdx.x == 64) {  // a thread with nothing else to do during start-up claims the cluster's tiles
    const GpSchedule sc = gp_claim_schedule(p, total_work, cluster_id, num_clusters);
    sched[0] = sc.first;
    sched[1] = sc.end;
    sched[2] = sc.stride;
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                // both CTAs' barriers are initialised before any remote arrival or copy
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const GpSchedule sc = gp_read_schedule(sched);

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer (one per CTA)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = sc.first; ok && w < sc.end; w += sc.stride) {
        const GpItem it = gd_decode(w, tiles_m, tiles_n, rank);
        const int bn0 = it.nt * GP_BN + static_cast<int>(rank) * GP_BNH;     // this CTA's half of the B tile
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_EMPTY, budget)) {
            ok = false;
            break;
          }
          if (leader) mbar_expect_tx(&full[stage], 2 * GD_STAGE_BYTES);
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          uint8_t* a_dst = smem + stage * GD_STAGE_BYTES;
          uint8_t* b_dst = a_dst + GD_A_BYTES;
          const bool first = kb < nk1;
          const int k0 = (first ? kb : kb - nk1) * GP_BK;
          tma_load_2d_pair(a_dst, first ? &map_a : &map_a2, bar, k0, it.row0);
          const CUtensorMap* mb = first ? &map_b : &map_b2;
          if (first ? p.kn1 : p.kn2) {
#pragma unroll
            for (int j = 0; j < GP_BNH / 64; ++j)
              tma_load_2d_pair(b_dst + j * (GP_BK * 128), mb, bar, bn0 + 64 * j, k0);
          } else {
            tma_load_2d_pair(b_dst, mb, bar, k0, bn0);
          }
          if (++stage == GD_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer (leader CTA only)
      constexpr uint32_t idesc_k = make_idesc_bf16(2 * GD_BM, GP_BN, 0, 0);
      constexpr uint32_t idesc_n = make_idesc_bf16(2 * GD_BM, GP_BN, 0, 1);
      int stage = 0, acc_iter = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = sc.first; ok && w < sc.end; w += sc.stride) {
        const int as = acc_iter & 1;
        if (!mbar_wait(&tmem_empty[as], ((acc_iter >> 1) & 1) ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY,
                       budget)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * GP_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL, budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * GD_STAGE_BYTES);
          const uint32_t b_addr = a_addr + GD_A_BYTES;
          const bool kn = kb < nk1 ? p.kn1 != 0 : p.kn2 != 0;
#pragma unroll
          for (int kk = 0; kk < GP_BK / 16; ++kk) {
            // K-major operand: rows 128 B apart, 8-row groups 1024 B apart, 32 B per 16-element k-step.
            // N-major operand: 64-column blocks GP_BK*128 B apart, 8-row (k) groups 1024 B apart, 2048 B per k-step.
            const uint64_t ad = make_smem_desc(a_addr + kk * 32, 16, 1024, 2);
            const uint64_t bd = kn ? make_smem_desc(b_addr + kk * (16 * 128), GP_BK * 128, 1024, 2)
                                   : make_smem_desc(b_addr + kk * 32, 16, 1024, 2);
            umma_bf16_pair(d_tmem, ad, bd, kn ? idesc_n : idesc_k, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage], 3);          // frees the stage in both CTAs
          if (++stage == GD_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tmem_full[as], 3);           // this tile's accumulators (both CTAs) are complete
        ++acc_iter;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (8 per CTA)
    const int q = warp & 3;                  // TMEM lane quarter this warp may read
    const int g = (warp - 2) >> 2;           // 128-column half of the tile
    uint8_t* slab = slabs + (warp - 2) * GP_SLAB_BYTES;
    int acc_iter = 0;
    bool ok = true;
    const bool vec_ok = ((p.ldo & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    for (int w = sc.first; ok && w < sc.end; w += sc.stride) {
      const GpItem it = gd_decode(w, tiles_m, tiles_n, rank);
      const int as = acc_iter & 1;
      if (!mbar_wait_idle(&tmem_full[as], (acc_iter >> 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL, budget)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row0 = it.row0 + q * 32;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * GP_BN + g * (GP_BN / 2);
      uint32_t pk[2][32];                    // both rounds in registers, then the accumulator goes back (see above)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int nc = it.nt * GP_BN + g * (GP_BN / 2) + c * 64;
        if (nc < p.N) {
          float v[64];
          tmem_ld32(t_row + c * 64, v);
          tmem_ld32(t_row + c * 64 + 32, v + 32);
          tmem_ld_wait();
          if (p.bias != nullptr) add_bias64(v, p.bias, nc, p.N);
#pragma unroll
          for (int j = 0; j < 32; ++j) pk[c][j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(&tmem_empty[as]);
        else mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[as]), 0));
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int nc = it.nt * GP_BN + g * (GP_BN / 2) + c * 64;
        if (nc < p.N)
          store_tile64_packed(slab, pk[c], &map_out, p.tma_store != 0, nc, row0, p.out, p.ldo, p.M - row0, p.N - nc, vec_ok,
                              lane);
      }
      ++acc_iter;
    }
    if (lane == 0) tma_store_wait_all();
  }

  // Nobody leaves (or frees tensor memory) while the other CTA may still signal this CTA's barriers, complete copies
  // on them or accumulate into its tensor memory.
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();              // lets copies issued before a timed-out wait land (see above)
    while (globaltimer_ns() - t0 < 1000000ull) {}
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// One warp per row: combines the per-tile partials of the CE epilogue in a fixed order.
__global__ void __launch_bounds__(256)
lce_combine_kernel(const float4* __restrict__ partials, const long long* __restrict__ labels, float* __restrict__ nll,
                   float* __restrict__ lse_out, long long rows, int tiles_n, int V, float smoothing,
                   long long ignore_index) {
  const long long row = (blockIdx.x * 256LL + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const long long label = labels[row];
  const bool ignored = label == ignore_index || label < 0 || label >= V;
  float m = -INFINITY, s = 0.f, zl = 0.f, zt = 0.f;
  for (int t = lane; t < tiles_n; t += 32) {
    const float4 q = partials[row * tiles_n + t];
    if (q.x > m) {
      s = s * __expf(m - q.x) + q.y;
      m = q.x;
    } else if (q.x > -INFINITY) {
      s += q.y * __expf(q.x - m);
    }
    zl += q.z;
    zt += q.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mm = fmaxf(m, m2);
    s = (m > -INFINITY ? s * __expf(m - mm) : 0.f) + (m2 > -INFINITY ? s2 * __expf(m2 - mm) : 0.f);
    m = mm;
    zl += __shfl_xor_sync(0xffffffffu, zl, o);
    zt += __shfl_xor_sync(0xffffffffu, zt, o);
  }
  if (lane == 0) {
    const float lse = m + __logf(s);
    float loss = lse - zl;
    if (smoothing > 0.f) loss = (1.f - smoothing) * loss + smoothing * (lse - zt / V);
    nll[row] = ignored ? 0.f : loss;
    if (lse_out) lse_out[row] = ignored ? 0.f : lse;
  }
}

// In place: stored (soft-capped, bf16) logits -> w_row * d nll / d raw logits, one read and one write per element.
__global__ void __launch_bounds__(256)
lce_dlogits_kernel(__nv_bfloat16* __restrict__ z, const long long* __restrict__ labels, const float* __restrict__ lse,
                   const float* __restrict__ row_weight, int V, long long ld, float softcap, float smoothing,
                   long long ignore_index) {
  const long long row = blockIdx.x;
  __nv_bfloat16* zr = z + row * ld;
  const long long label = labels[row];
  const bool ignored = label == ignore_index || label < 0 || label >= V;
  const float w = ignored ? 0.f : (row_weight ? row_weight[row] : 1.f);
  const float l = lse[row];
  const float sm = smoothing / V;
  const bool vec = (ld & 7) == 0 && (reinterpret_cast<uintptr_t>(z) & 15) == 0;
  const int v_vec = vec ? (V & ~7) : 0;
  for (int i = threadIdx.x; i < (v_vec >> 3); i += 256) {
    uint4 pk = reinterpret_cast<uint4*>(zr)[i];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
    if (w == 0.f) {
      pk = make_uint4(0u, 0u, 0u, 0u);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        float g0 = __expf(f.x - l) - sm, g1 = __expf(f.y - l) - sm;
        if (i * 8 + 2 * j == label) g0 -= 1.f - smoothing;
        if (i * 8 + 2 * j + 1 == label) g1 -= 1.f - smoothing;
        if (softcap > 0.f) {
          const float t0 = f.x / softcap, t1 = f.y / softcap;
          g0 *= 1.f - t0 * t0;
          g1 *= 1.f - t1 * t1;
        }
        h[j] = __floats2bfloat162_rn(w * g0, w * g1);
      }
    }
    reinterpret_cast<uint4*>(zr)[i] = pk;
  }
  for (int i = v_vec + threadIdx.x; i < V; i += 256) {
    const float f = __bfloat162float(zr[i]);
    float g = __expf(f - l) - sm;
    if (i == label) g -= 1.f - smoothing;
    if (softcap > 0.f) {
      const float t = f / softcap;
      g *= 1.f - t * t;
    }
    zr[i] = __float2bfloat16_rn(w * g);
  }
}

// Raster band height in pair tiles (L2 reuse of the B tiles inside a band); OB_PAIR_GROUP_M overrides it for experiments.
static int pair_group_m() {
  static int v = 0;
  if (v == 0) {
    const char* e = getenv("OB_PAIR_GROUP_M");
    v = e ? atoi(e) : GP_GROUP_M;
    if (v < 1) v = GP_GROUP_M;
  }
  return v;
}

static int pair_grid(const void* kernel, int sms, int smem_bytes = GP_SMEM) {
  // clusters that can be co-resident (two CTAs of a pair must sit on paired SMs); one cluster per SM pair
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sms), 1, 1);
  cfg.blockDim = dim3(GP_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters <= 0) {
    cudaGetLastError();
    clusters = sms / 2;
  }
  if (clusters > sms / 2) clusters = sms / 2;
  return clusters;
}

}  // namespace ob

namespace ob {
// ---- die-aware tile assignment: host side ------------------------------------------------------------------------
// Claim words: a ring in device memory, one word per launch, each back to zero after its launch's last claim.  Two
// launches share a word only if 4096 pair-GEMM launches lie between them and both are in flight at once; a kernel that
// sees that reports OB_ERR_CLAIM instead of computing.
constexpr int GP_CLAIM_RING = 4096;
static __device__ unsigned long long g_pair_claim[GP_CLAIM_RING];

// Off by default: on the shapes measured it cut the sectors crossing the die-to-die link by 15 - 22 % and changed
// neither the kernel time nor the tensor-pipe utilisation (the loads are not what the MMA thread waits for most).
// OB_PAIR_DIE_AWARE=1 or ob_pair_set_die_aware(1) switches it on.
static std::atomic<int> g_die_aware{-1};
static int pair_die_aware() {
  int v = g_die_aware.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* e = getenv("OB_PAIR_DIE_AWARE");
    v = (e && atoi(e) != 0) ? 1 : 0;
    g_die_aware.store(v, std::memory_order_relaxed);
  }
  return v;
}

// Tensor map for bulk stores of a [rows, cols] bf16 output (32-row x 64-column boxes); returns false when the output
// is not aligned for it (the kernels then store with ordinary vector / scalar stores).
static bool pair_out_map(CUtensorMap* m, void* out, long long rows, long long cols, long long ldo) {
  if (out == nullptr || (reinterpret_cast<uintptr_t>(out) & 15) != 0 || ((ldo * 2) & 15) != 0) return false;
  return make_bf16_map_2d(m, out, rows, cols, ldo, 64, 32) == 0;
}

static void pair_set_schedule(PairParams* p, long long total, int clusters, cudaStream_t st) {
  p->claim = nullptr;
  p->n_front = clusters;
  p->split = static_cast<int>(total);
  if (!pair_die_aware() || p->status == nullptr || clusters < 4 || total < 4) return;
  static std::atomic<bool> ready[64];
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!ready[dev].load(std::memory_order_acquire)) {
    // the probe synchronises the device: never during a stream capture (ob_pair_init() runs it at load time instead)
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
      cudaGetLastError();
      return;
    }
    die_map_for_current_device();
    ready[dev].store(true, std::memory_order_release);
  }
  const DieMap& dm = die_map_for_current_device();
  if (!dm.valid) return;
  static unsigned long long* ring[64] = {};
  if (ring[dev] == nullptr) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_pair_claim) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    ring[dev] = static_cast<unsigned long long*>(sym);
  }
  static std::atomic<unsigned> next{0};
  const int tp = dm.tpcs[0] + dm.tpcs[1];
  int n_front = static_cast<int>((static_cast<long long>(clusters) * dm.tpcs[0] + tp / 2) / tp);
  if (n_front < 1) n_front = 1;
  if (n_front > clusters - 1) n_front = clusters - 1;
  const long long waves = (total + clusters - 1) / clusters;
  long long split = (total * n_front + clusters / 2) / clusters;
  const long long lo = total - static_cast<long long>(clusters - n_front) * waves, hi = static_cast<long long>(n_front) * waves;
  if (split < lo) split = lo;
  if (split > hi) split = hi;
  if (split < 1) split = 1;
  if (split > total - 1) split = total - 1;
  p->claim = ring[dev] + (next.fetch_add(1, std::memory_order_relaxed) % GP_CLAIM_RING);
  p->n_front = n_front;
  p->split = static_cast<int>(split);
}

}  // namespace ob

// Die-aware tile assignment on (1) / off (0) for later launches of this process; returns the previous setting.
extern "C" int ob_pair_set_die_aware(int on) {
  const int prev = ob::pair_die_aware();
  ob::g_die_aware.store(on ? 1 : 0, std::memory_order_relaxed);
  return prev;
}

// Probes the die map of the current device (no-op after the first call); call once outside any stream capture.
extern "C" int ob_pair_init() {
  using namespace ob;
  const DieMap& dm = die_map_for_current_device();
  return dm.valid ? dm.tpcs[0] * 1000 + dm.tpcs[1] : 0;
}

// smid -> die (0 / 1) of the current device as probed; returns the number of SMs, 0 when no two-die split was found.
extern "C" int ob_die_map(unsigned char* out, int n) {
  using namespace ob;
  const DieMap& dm = die_map_for_current_device();
  if (!dm.valid) return 0;
  for (int i = 0; i < n && i < DM_MAX_SMS; ++i) out[i] = dm.die[i];
  return dm.sms;
}

// D = A op1(B) + A2 op2(B2) + bias on CTA pairs.  b_kn / b2_kn = 1: that operand is stored [K, N].
// glu != 0: `b` holds the gate rows and `b_up` the up rows ([N/2, K] each, or [K, N/2] with b_kn); N counts gate and up
// columns together; out [M, N/2] = act(gate) * up, and out_gate / out_up (optional, both or none) receive the
// pre-activations.  glu_act: 0 silu, 1 gelu erf, 2 gelu tanh.  With a second segment in GLU mode b2 / b2_up likewise.
extern "C" int ob_gemm_pair(const void* a, const void* b, const void* b_up, const void* a2, const void* b2,
                            const void* b2_up, const void* bias, void* out, void* out_gate, void* out_up,
                            long long rows_a, int N, int K1, int K2, long long lda, long long ldb, long long lda2,
                            long long ldb2, long long ldo, int b_kn, int b2_kn, int glu, int glu_act, int* status,
                            double wait_budget_s, int num_sms, void* stream) {
  using namespace ob;
  if (rows_a <= 0 || N <= 0 || K1 <= 0) return 0;
  if (rows_a > 0x7fffffffLL - 2 * GP_BM) return -50;
  if (K2 > 0 && (a2 == nullptr || b2 == nullptr)) return -51;
  if (glu && (b_up == nullptr || (N & 1) || (K2 > 0 && b2_up == nullptr) || bias != nullptr)) return -52;
  if (glu && ((out_gate == nullptr) != (out_up == nullptr))) return -53;
  const int nb = glu ? N / 2 : N;               // columns of N covered by ONE B operand
  CUtensorMap ma, mb, mbu, ma2, mb2, mb2u;
  int rc = make_bf16_map_2d(&ma, a, rows_a, K1, lda, GP_BK, GP_BM);
  if (rc) return rc;
  auto b_map = [&](CUtensorMap* m, const void* base, int K, long long ld, int kn) {
    return kn ? make_bf16_map_2d(m, base, K, nb, ld, 64, GP_BK) : make_bf16_map_2d(m, base, nb, K, ld, GP_BK, GP_BNH);
  };
  rc = b_map(&mb, b, K1, ldb, b_kn);
  if (rc) return rc;
  if (glu) {
    rc = b_map(&mbu, b_up, K1, ldb, b_kn);
    if (rc) return rc;
  } else {
    mbu = mb;
  }
  if (K2 > 0) {
    rc = make_bf16_map_2d(&ma2, a2, rows_a, K2, lda2, GP_BK, GP_BM);
    if (rc) return rc;
    rc = b_map(&mb2, b2, K2, ldb2, b2_kn);
    if (rc) return rc;
    if (glu) {
      rc = b_map(&mb2u, b2_up, K2, ldb2, b2_kn);
      if (rc) return rc;
    } else {
      mb2u = mb2;
    }
  } else {
    ma2 = ma;
    mb2 = mb;
    mb2u = mbu;
  }
  static bool configured = false;
  static int clusters_store = 0, clusters_glu = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<GP_EPI_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, GP_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_pair_kernel<GP_EPI_GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, GP_SMEM) != cudaSuccess)
      return -54;
    clusters_store = pair_grid(reinterpret_cast<const void*>(gemm_pair_kernel<GP_EPI_STORE>), num_sms);
    clusters_glu = pair_grid(reinterpret_cast<const void*>(gemm_pair_kernel<GP_EPI_GLU>), num_sms);
    configured = true;
  }
  PairParams p = {};
  p.group_m = pair_group_m();
  p.M = static_cast<int>(rows_a);
  p.N = N; p.K1 = K1; p.K2 = K2;
  p.kn1 = b_kn; p.kn2 = b2_kn;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.out_gate = static_cast<__nv_bfloat16*>(out_gate);
  p.out_up = static_cast<__nv_bfloat16*>(out_up);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.act = glu_act;
  p.status = status;
  p.wait_budget_ns = static_cast<unsigned long long>(wait_budget_s * 1e9);
  const long long tiles_m = (rows_a + 2 * GP_BM - 1) / (2 * GP_BM);
  const long long tiles_n = glu ? (nb + GP_BNH - 1) / GP_BNH : (N + GP_BN - 1) / GP_BN;
  const long long total = tiles_m * tiles_n;
  const int avail = glu ? clusters_glu : clusters_store;
  const int clusters = static_cast<int>(total < avail ? total : avail);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  pair_set_schedule(&p, total, clusters, st);
  CUtensorMap mo = ma, mog = ma, mou = ma;
  p.tma_store = pair_out_map(&mo, out, rows_a, nb, ldo) ? 1 : 0;          // nb: the width of the output (N / 2 for GLU)
  if (glu && out_gate != nullptr && p.tma_store)
    p.tma_store = (pair_out_map(&mog, out_gate, rows_a, nb, ldo) && pair_out_map(&mou, out_up, rows_a, nb, ldo)) ? 1 : 0;
  if (glu)
    gemm_pair_kernel<GP_EPI_GLU><<<2 * clusters, GP_THREADS, GP_SMEM, st>>>(ma, mb, mbu, ma2, mb2, mb2u, mo, mog, mou, p);
  else
    gemm_pair_kernel<GP_EPI_STORE><<<2 * clusters, GP_THREADS, GP_SMEM, st>>>(ma, mb, mbu, ma2, mb2, mb2u, mo, mog, mou, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -55;
}

// Data gradient of a gated MLP's down projection fused with the activation's backward:
//   dH = dY[M, K] * op(W)  (W stored [K, N] with b_kn = 1: the down-projection weight as stored),  N = intermediate size,
//   dGate = dH * up * act'(gate),  dUp = dH * act(gate)   (bf16 [M, N], pitch ld_out);  dH never reaches memory.
// gate / up: the stored pre-activations [M, N] (pitch ld_gu).  N % 64 == 0; all rows 16-byte aligned.
extern "C" int ob_gemm_pair_glu_bwd(const void* dy, const void* w, const void* gate, const void* up, void* dgate, void* dup,
                                    long long rows_a, int N, int K, long long lddy, long long ldw, long long ld_gu,
                                    long long ld_out, int b_kn, int glu_act, int* status, double wait_budget_s,
                                    int num_sms, void* stream) {
  using namespace ob;
  if (rows_a <= 0 || N <= 0 || K <= 0) return 0;
  if (rows_a > 0x7fffffffLL - 2 * GP_BM) return -50;
  if (gate == nullptr || up == nullptr || dgate == nullptr || dup == nullptr) return -57;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if ((N & 63) != 0 || (ld_gu & 7) != 0 || (ld_out & 7) != 0 || !al(gate) || !al(up) || !al(dgate) || !al(dup)) return -58;
  CUtensorMap ma, mb;
  int rc = make_bf16_map_2d(&ma, dy, rows_a, K, lddy, GP_BK, GP_BM);
  if (rc) return rc;
  rc = b_kn ? make_bf16_map_2d(&mb, w, K, N, ldw, 64, GP_BK) : make_bf16_map_2d(&mb, w, N, K, ldw, GP_BK, GP_BNH);
  if (rc) return rc;
  static bool configured = false;
  static int clusters_gb = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<GP_EPI_GLUBWD>, cudaFuncAttributeMaxDynamicSharedMemorySize, GP_SMEM) != cudaSuccess)
      return -54;
    clusters_gb = pair_grid(reinterpret_cast<const void*>(gemm_pair_kernel<GP_EPI_GLUBWD>), num_sms);
    configured = true;
  }
  PairParams p = {};
  p.group_m = pair_group_m();
  p.M = static_cast<int>(rows_a);
  p.N = N; p.K1 = K; p.K2 = 0;
  p.kn1 = b_kn; p.kn2 = 0;
  p.out = static_cast<__nv_bfloat16*>(dgate);
  p.out_up = static_cast<__nv_bfloat16*>(dup);
  p.ldo = ld_out;
  p.glu_g = static_cast<const __nv_bfloat16*>(gate);
  p.glu_u = static_cast<const __nv_bfloat16*>(up);
  p.ld_gu = ld_gu;
  p.act = glu_act;
  p.status = status;
  p.wait_budget_ns = static_cast<unsigned long long>(wait_budget_s * 1e9);
  const long long total = ((rows_a + 2 * GP_BM - 1) / (2 * GP_BM)) * ((N + GP_BN - 1) / GP_BN);
  const int clusters = static_cast<int>(total < clusters_gb ? total : clusters_gb);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  pair_set_schedule(&p, total, clusters, st);
  CUtensorMap mog = ma, mou = ma;
  p.tma_store = (pair_out_map(&mog, dgate, rows_a, N, ld_out) && pair_out_map(&mou, dup, rows_a, N, ld_out)) ? 1 : 0;
  gemm_pair_kernel<GP_EPI_GLUBWD><<<2 * clusters, GP_THREADS, GP_SMEM, st>>>(ma, mb, mb, ma, mb, mb, mog, ma, mou, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -55;
}

// The double-buffered 256 x 256 pair-tile kernel (plain store epilogue); arguments as in ob_gemm_pair.
extern "C" int ob_gemm_pair_db(const void* a, const void* b, const void* a2, const void* b2, const void* bias, void* out,
                               long long rows_a, int N, int K1, int K2, long long lda, long long ldb, long long lda2,
                               long long ldb2, long long ldo, int b_kn, int b2_kn, int* status, double wait_budget_s,
                               int num_sms, void* stream) {
  using namespace ob;
  if (rows_a <= 0 || N <= 0 || K1 <= 0) return 0;
  if (rows_a > 0x7fffffffLL - 2 * GD_BM) return -50;
  if (K2 > 0 && (a2 == nullptr || b2 == nullptr)) return -51;
  CUtensorMap ma, mb, ma2, mb2;
  int rc = make_bf16_map_2d(&ma, a, rows_a, K1, lda, GP_BK, GD_BM);
  if (rc) return rc;
  auto b_map = [&](CUtensorMap* m, const void* base, int K, long long ld, int kn) {
    return kn ? make_bf16_map_2d(m, base, K, N, ld, 64, GP_BK) : make_bf16_map_2d(m, base, N, K, ld, GP_BK, GP_BNH);
  };
  rc = b_map(&mb, b, K1, ldb, b_kn);
  if (rc) return rc;
  if (K2 > 0) {
    rc = make_bf16_map_2d(&ma2, a2, rows_a, K2, lda2, GP_BK, GD_BM);
    if (rc) return rc;
    rc = b_map(&mb2, b2, K2, ldb2, b2_kn);
    if (rc) return rc;
  } else {
    ma2 = ma;
    mb2 = mb;
  }
  static bool configured = false;
  static int clusters_db = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_pair_db_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GD_SMEM) != cudaSuccess)
      return -54;
    clusters_db = pair_grid(reinterpret_cast<const void*>(gemm_pair_db_kernel), num_sms, GD_SMEM);
    configured = true;
  }
  PairParams p = {};
  p.M = static_cast<int>(rows_a);
  p.N = N; p.K1 = K1; p.K2 = K2;
  p.kn1 = b_kn; p.kn2 = b2_kn;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = status;
  p.wait_budget_ns = static_cast<unsigned long long>(wait_budget_s * 1e9);
  const long long total = ((rows_a + 2 * GD_BM - 1) / (2 * GD_BM)) * ((N + GP_BN - 1) / GP_BN);
  const int clusters = static_cast<int>(total < clusters_db ? total : clusters_db);
  pair_set_schedule(&p, total, clusters, static_cast<cudaStream_t>(stream));
  CUtensorMap mo = ma;
  p.tma_store = pair_out_map(&mo, out, rows_a, N, ldo) ? 1 : 0;
  gemm_pair_db_kernel<<<2 * clusters, GP_THREADS, GD_SMEM, static_cast<cudaStream_t>(stream)>>>(ma, mb, ma2, mb2, mo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -55;
}

// Bit patterns of the descriptors the tensor-core kernels build, for host-side checks.
extern "C" unsigned int ob_debug_idesc_bf16(int m, int n, int a_mn_major, int b_mn_major) {
  return ob::make_idesc_bf16(m, n, a_mn_major, b_mn_major);
}

// Output head fused with the cross-entropy statistics:  logits = hidden[M, K] * weight[N, K]^T on CTA pairs; the epilogue
// folds every 128-column half of a logits tile into per-row partials (scratch `partials`: M * 2 * ceil(N / 256) float4) and a second
// small kernel combines them in a fixed order into nll[M] and lse[M].  The logits themselves are written (bf16, after the
// soft cap) only when `logits_out` is given.  softcap > 0: z = softcap * tanh(z / softcap).  Rows whose label is
// `ignore_index` or outside [0, N) get nll = lse = 0.
extern "C" int ob_linear_ce_fwd(const void* hidden, const void* weight, const long long* labels, void* logits_out,
                                float* partials, float* nll, float* lse, long long rows, int N, int K, long long ldh,
                                long long ldw, long long ldo, float softcap, float smoothing, long long ignore_index,
                                int* status, double wait_budget_s, int num_sms, void* stream) {
  using namespace ob;
  if (rows <= 0 || N <= 0 || K <= 0) return 0;
  if (rows > 0x7fffffffLL - 2 * GP_BM) return -50;
  if (labels == nullptr || partials == nullptr || nll == nullptr) return -56;
  CUtensorMap ma, mb;
  int rc = make_bf16_map_2d(&ma, hidden, rows, K, ldh, GP_BK, GP_BM);
  if (rc) return rc;
  rc = make_bf16_map_2d(&mb, weight, N, K, ldw, GP_BK, GP_BNH);
  if (rc) return rc;
  static bool configured = false;
  static int clusters_ce = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<GP_EPI_CE>, cudaFuncAttributeMaxDynamicSharedMemorySize, GP_SMEM) != cudaSuccess)
      return -54;
    clusters_ce = pair_grid(reinterpret_cast<const void*>(gemm_pair_kernel<GP_EPI_CE>), num_sms);
    configured = true;
  }
  PairParams p = {};
  p.group_m = pair_group_m();
  p.M = static_cast<int>(rows);
  p.N = N; p.K1 = K; p.K2 = 0;
  p.out = static_cast<__nv_bfloat16*>(logits_out);
  p.ldo = ldo;
  p.labels = labels;
  p.ce_partials = reinterpret_cast<float4*>(partials);
  p.softcap = softcap;
  p.status = status;
  p.wait_budget_ns = static_cast<unsigned long long>(wait_budget_s * 1e9);
  const long long tiles_m = (rows + 2 * GP_BM - 1) / (2 * GP_BM);
  const int tiles_n = (N + GP_BN - 1) / GP_BN;
  const long long total = tiles_m * tiles_n;
  const int clusters = static_cast<int>(total < clusters_ce ? total : clusters_ce);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  pair_set_schedule(&p, total, clusters, st);
  CUtensorMap mo = ma;
  p.tma_store = (logits_out != nullptr && pair_out_map(&mo, logits_out, rows, N, ldo)) ? 1 : 0;
  gemm_pair_kernel<GP_EPI_CE><<<2 * clusters, GP_THREADS, GP_SMEM, st>>>(ma, mb, mb, ma, mb, mb, mo, ma, ma, p);
  if (cudaGetLastError() != cudaSuccess) return -55;
  const long long warps = rows;
  lce_combine_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, st>>>(
      reinterpret_cast<const float4*>(partials), labels, nll, lse, rows, 2 * tiles_n, N, smoothing, ignore_index);
  return cudaGetLastError() == cudaSuccess ? 0 : -57;
}

// In place on the logits stored by ob_linear_ce_fwd: z <- row_weight * d nll / d (raw logits).
extern "C" int ob_linear_ce_dlogits(void* logits, const long long* labels, const float* lse, const float* row_weight,
                                    long long rows, int N, long long ld, float softcap, float smoothing,
                                    long long ignore_index, void* stream) {
  using namespace ob;
  if (rows <= 0 || N <= 0) return 0;
  lce_dlogits_kernel<<<static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), labels, lse, row_weight, N, ld, softcap, smoothing, ignore_index);
  return cudaGetLastError() == cudaSuccess ? 0 : -58;
}

// ------------------------------------------------------------------------------------------------------------------
// The same forward (losses and log-sum-exps, logits never stored) for callers that must not allocate: the per-tile
// statistics go to a fixed array inside the library image instead of caller-provided scratch.  See no_alloc.h for who
// needs this, the size limit and the sharing rules.
#include "no_alloc.h"
#include <cstdio>
#include <mutex>

// In HOST code this name is only a handle for the symbol, not a device address; device code may use it directly.
static __device__ __align__(256) float4 g_lce_static_partials[OB_NO_ALLOC_MAX_PARTIALS];

namespace {
constexpr int kMaxDevices = 64;
float4* g_lce_static_ptr[kMaxDevices] = {nullptr};
std::mutex g_lce_static_mutex;
thread_local char g_no_alloc_error[256] = {0};

// Device address of the static scratch array on the CURRENT device (looked up once per device, then cached).
int lce_static_scratch(float4** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_no_alloc_error, sizeof(g_no_alloc_error), "cudaGetDevice failed or device index %d is outside [0, %d)", dev, kMaxDevices);
    return -61;
  }
  std::lock_guard<std::mutex> lock(g_lce_static_mutex);
  if (g_lce_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_lce_static_partials);
    if (err != cudaSuccess || ptr == nullptr) {
      snprintf(g_no_alloc_error, sizeof(g_no_alloc_error), "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(err));
      return -62;
    }
    g_lce_static_ptr[dev] = static_cast<float4*>(ptr);
  }
  *out = g_lce_static_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int ob_no_alloc_last_error(char* buf, int len) {
  int i = 0;
  for (; g_no_alloc_error[i] && i < len - 1; ++i) buf[i] = g_no_alloc_error[i];
  if (len > 0) buf[i] = 0;
  return 0;
}

extern "C" int ob_linear_ce_fwd_noalloc(const void* hidden, const void* weight, const long long* labels, float* nll,
                                        float* lse, long long rows, int N, int K, long long ldh, long long ldw,
                                        float softcap, float smoothing, long long ignore_index, int* status,
                                        double wait_budget_s, int num_sms, void* stream) {
  using namespace ob;
  g_no_alloc_error[0] = 0;
  if (rows <= 0 || N <= 0 || K <= 0) return 0;
  if (hidden == nullptr || weight == nullptr || labels == nullptr || nll == nullptr) {
    snprintf(g_no_alloc_error, sizeof(g_no_alloc_error), "hidden, weight, labels and nll must be device pointers");
    return -56;
  }
  const int tiles_n = (N + GP_BN - 1) / GP_BN;
  const long long need = rows * 2LL * tiles_n;
  if (need > OB_NO_ALLOC_MAX_PARTIALS) {
    snprintf(g_no_alloc_error, sizeof(g_no_alloc_error),
             "problem too large for the static scratch: rows * 2 * ceil(N / 256) = %lld records, the array holds %d "
             "(rows = %lld, N = %d): split the rows over several calls",
             need, OB_NO_ALLOC_MAX_PARTIALS, rows, N);
    return OB_NO_ALLOC_TOO_LARGE;
  }
  float4* partials = nullptr;
  int rc = lce_static_scratch(&partials);
  if (rc) return rc;
  CUtensorMap ma, mb;
  rc = make_bf16_map_2d(&ma, hidden, rows, K, ldh, GP_BK, GP_BM);
  if (rc == 0) rc = make_bf16_map_2d(&mb, weight, N, K, ldw, GP_BK, GP_BNH);
  if (rc) {
    snprintf(g_no_alloc_error, sizeof(g_no_alloc_error), "operands must have 16-byte aligned rows (tensor map code %d)", rc);
    return rc;
  }
  static bool configured = false;
  static int clusters_ce = 0;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<GP_EPI_CE>, cudaFuncAttributeMaxDynamicSharedMemorySize, GP_SMEM) != cudaSuccess) {
      snprintf(g_no_alloc_error, sizeof(g_no_alloc_error), "cudaFuncSetAttribute(shared memory) failed");
      return -54;
    }
    clusters_ce = pair_grid(reinterpret_cast<const void*>(gemm_pair_kernel<GP_EPI_CE>), num_sms);
    configured = true;
  }
  PairParams p = {};
  p.group_m = pair_group_m();
  p.M = static_cast<int>(rows);
  p.N = N; p.K1 = K; p.K2 = 0;
  p.out = nullptr;                    // forward only: the logits never reach memory
  p.ldo = 0;
  p.labels = labels;
  p.ce_partials = partials;
  p.softcap = softcap;
  p.status = status;
  p.wait_budget_ns = static_cast<unsigned long long>(wait_budget_s * 1e9);
  const long long tiles_m = (rows + 2 * GP_BM - 1) / (2 * GP_BM);
  const long long total = tiles_m * tiles_n;
  const int clusters = static_cast<int>(total < clusters_ce ? total : clusters_ce);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  gemm_pair_kernel<GP_EPI_CE><<<2 * clusters, GP_THREADS, GP_SMEM, st>>>(ma, mb, mb, ma, mb, mb, ma, ma, ma, p);
  cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess) {
    lce_combine_kernel<<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, st>>>(
        partials, labels, nll, lse, rows, 2 * tiles_n, N, smoothing, ignore_index);
    err = cudaGetLastError();
  }
  if (err != cudaSuccess) {
    snprintf(g_no_alloc_error, sizeof(g_no_alloc_error), "kernel launch failed: %s", cudaGetErrorString(err));
    return -55;
  }
  return 0;
}
