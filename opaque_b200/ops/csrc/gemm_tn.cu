// Forward / data-gradient GEMM family on sm_100a:   D[M, N] = A[M, K1] * op(B) + A2[M, K2] * B2[N, K2]^T + bias
//
// One persistent tcgen05 kernel covers the three library-shaped products of the model path that need something a
// plain library GEMM cannot do in one pass:
//
//   * LoRA-fused linear:   y = x W^T + (x A^T) (s B)^T        -- second K segment (A2, B2) accumulated into the same
//                                                                TMEM tile, so y is written once and never re-read;
//   * grouped (MoE) GEMMs: rows are sorted by expert; group e owns rows [offs[e], offs[e+1]) of A and D and the
//                          e-th slab of B.  Tiles never mix experts; rows past a group's end are masked at the store;
//   * data gradients:      op(B) = B for B stored [K, N] row-major (an N-major operand), so dX = dY W needs no
//                          transposed copy of W;  op(B) = B^T for B stored [N, K] (K-major, the usual weight layout).
//
// Tile 128 x 256, K block 64, 4-stage TMA ring (128-byte swizzle), accumulators double-buffered in TMEM (2 x 256
// columns) so the epilogue of tile i overlaps the MMAs of tile i+1.  Warp 0 issues TMA, warp 1 issues tcgen05.mma and
// owns TMEM, warps 2-9 convert fp32 accumulators to bf16 and store them as whole 128-byte row segments (staged through
// a swizzled shared-memory slab per warp): with a short K (768) the drain of one tile takes about as long as its MMAs,
// so four warps storing one 16-byte piece per lane and row left the tensor pipe waiting.  Every wait is bounded.
#include "common.cuh"
#include "api.h"

namespace ob {

int make_bf16_map_2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                     int box_cols, int box_rows);

constexpr int GT_BM = 128;
constexpr int GT_BN = 256;
constexpr int GT_BK = 64;
constexpr int GT_STAGES = 4;
constexpr int GT_A_BYTES = GT_BM * GT_BK * 2;
constexpr int GT_B_BYTES = GT_BN * GT_BK * 2;
constexpr int GT_STAGE_BYTES = GT_A_BYTES + GT_B_BYTES;
constexpr int GT_THREADS = 320;      // TMA producer warp, MMA warp, 8 epilogue warps
constexpr int GT_SLAB_BYTES = 4096;   // per epilogue warp: 32 rows x 64 columns of bf16 on their way to memory
constexpr int GT_MAX_GROUPS = 256;
constexpr int GT_GROUP_M = 16;       // m-tiles per raster band (L2 reuse of the B tiles inside a band)
constexpr int GT_SMEM = GT_STAGES * GT_STAGE_BYTES + 8 * GT_SLAB_BYTES + 256 + (GT_MAX_GROUPS + 2) * 4 + 1024;

struct GemmParams {
  int M, N, K1, K2;
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* bias;
  const int* group_offs;   // [num_groups + 1] or nullptr
  int num_groups;
  int b_group_rows;        // distance, in rows of B, between consecutive groups' slabs
  int tma_store;           // the output leaves through bulk tensor stores (map_out is valid)
  int* status;
  unsigned long long wait_budget_ns;
};

struct GtItem {
  int row0, row_end, n0, b_row;
};

// Tile w of the persistent schedule.  `cursor` is the caller's monotone group cursor (grouped mode only).
__device__ __forceinline__ GtItem gt_decode(const GemmParams& p, int w, int tiles_m, int tiles_n, const int* tile_start,
                                            int& cursor) {
  GtItem it;
  if (p.group_offs == nullptr) {
    const int band = GT_GROUP_M * tiles_n;
    const int b = w / band, r = w % band;
    const int m_in_band = min(GT_GROUP_M, tiles_m - b * GT_GROUP_M);
    const int mt = b * GT_GROUP_M + r % m_in_band;
    const int nt = r / m_in_band;
    it.row0 = mt * GT_BM;
    it.row_end = p.M;
    it.n0 = nt * GT_BN;
    it.b_row = 0;
  } else {
    const int g = w / tiles_n;
    while (g >= tile_start[cursor + 1]) ++cursor;
    it.row0 = p.group_offs[cursor] + (g - tile_start[cursor]) * GT_BM;
    it.row_end = p.group_offs[cursor + 1];
    it.n0 = (w % tiles_n) * GT_BN;
    it.b_row = cursor * p.b_group_rows;
  }
  return it;
}

template <bool B_KN>
__global__ void __launch_bounds__(GT_THREADS, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
               const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* slabs = smem + GT_STAGES * GT_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(slabs + 8 * GT_SLAB_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + GT_STAGES;
  uint64_t* tmem_full = bars + 2 * GT_STAGES;
  uint64_t* tmem_empty = bars + 2 * GT_STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GT_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* tile_start = reinterpret_cast<int*>(slabs + 8 * GT_SLAB_BYTES + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.N + GT_BN - 1) / GT_BN;
  const int nk1 = (p.K1 + GT_BK - 1) / GT_BK;
  const int nk2 = (p.K2 + GT_BK - 1) / GT_BK;
  const int num_kb = nk1 + nk2;
  const uint64_t budget = p.wait_budget_ns;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GT_STAGES; ++s) {
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
    if (nk2) {
      tma_prefetch_desc(&map_a2);
      tma_prefetch_desc(&map_b2);
    }
    if (p.group_offs != nullptr) {
      int acc = 0;
      tile_start[0] = 0;
      for (int e = 0; e < p.num_groups; ++e) {
        acc += (p.group_offs[e + 1] - p.group_offs[e] + GT_BM - 1) / GT_BM;
        tile_start[e + 1] = acc;
      }
      tile_start[p.num_groups + 1] = 0x7fffffff;     // sentinel for the cursor walk
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles_m = p.group_offs ? tile_start[p.num_groups] : (p.M + GT_BM - 1) / GT_BM;
  const int total_work = tiles_m * tiles_n;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0, cursor = 0;
      uint32_t phase = 0, issued_mask = 0, issued_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const GtItem it = gt_decode(p, w, tiles_m, tiles_n, tile_start, cursor);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, OB_ERR_WAIT_EMPTY, budget)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], GT_STAGE_BYTES);
          uint8_t* a_dst = smem + stage * GT_STAGE_BYTES;
          uint8_t* b_dst = a_dst + GT_A_BYTES;
          if (kb < nk1) {
            tma_load_2d(a_dst, &map_a, &full[stage], kb * GT_BK, it.row0);
            if constexpr (B_KN) {
#pragma unroll
              for (int j = 0; j < GT_BN / 64; ++j)
                tma_load_2d(b_dst + j * (GT_BK * 128), &map_b, &full[stage], it.n0 + 64 * j, it.b_row + kb * GT_BK);
            } else {
              tma_load_2d(b_dst, &map_b, &full[stage], kb * GT_BK, it.b_row + it.n0);
            }
          } else {
            tma_load_2d(a_dst, &map_a2, &full[stage], (kb - nk1) * GT_BK, it.row0);
            tma_load_2d(b_dst, &map_b2, &full[stage], (kb - nk1) * GT_BK, it.n0);
          }
          issued_mask |= 1u << stage;
          issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
          if (++stage == GT_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        for (int s = 0; s < GT_STAGES; ++s)
          if (issued_mask & (1u << s)) {
            int dummy_abort = 0;
            mbar_wait(&full[s], (issued_phase >> s) & 1u, &dummy_abort, p.status, OB_ERR_DRAIN, budget);
          }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_main = make_idesc_bf16(GT_BM, GT_BN, 0, B_KN ? 1 : 0);
      constexpr uint32_t idesc_kmaj = make_idesc_bf16(GT_BM, GT_BN, 0, 0);
      int stage = 0, acc_iter = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const int as = acc_iter & 1;
        if (!mbar_wait(&tmem_empty[as], ((acc_iter >> 1) & 1) ^ 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_EMPTY,
                       budget)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * GT_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, OB_ERR_WAIT_FULL, budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * GT_STAGE_BYTES);
          const uint32_t b_addr = a_addr + GT_A_BYTES;
          const bool kn = B_KN && kb < nk1;
#pragma unroll
          for (int kk = 0; kk < GT_BK / 16; ++kk) {
            // K-major operand: rows 128 B apart, 8-row groups 1024 B apart, 32 B per 16-element k-step.
            // N-major operand: 64-column blocks GT_BK*128 B apart, 8-row (k) groups 1024 B apart, 2048 B per k-step.
            const uint64_t ad = make_smem_desc(a_addr + kk * 32, 16, 1024, 2);
            const uint64_t bd = kn ? make_smem_desc(b_addr + kk * (16 * 128), GT_BK * 128, 1024, 2)
                                   : make_smem_desc(b_addr + kk * 32, 16, 1024, 2);
            umma_bf16(d_tmem, ad, bd, kn ? idesc_main : idesc_kmaj, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == GT_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[as]);
        ++acc_iter;
      }
    }
  } else {
    // Eight warps drain one 128 x 256 accumulator: warp w reads TMEM lanes 32 * (w % 4) .. (the lane quarter a warp may
    // touch) and one 128-column half, 64 columns per round (two loads in flight, one wait), and hands the rows to memory
    // through its shared-memory slab as whole 128-byte row segments.
    const int q = warp & 3;
    const int g = (warp - 2) >> 2;
    uint8_t* slab = slabs + (warp - 2) * GT_SLAB_BYTES;
    int acc_iter = 0, cursor = 0;
    bool ok = true;
    const bool vec_ok = ((p.ldo & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      const GtItem it = gt_decode(p, w, tiles_m, tiles_n, tile_start, cursor);
      const int as = acc_iter & 1;
      if (!mbar_wait(&tmem_full[as], (acc_iter >> 1) & 1, abort_flag, p.status, OB_ERR_WAIT_TMEM_FULL, budget)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row0 = it.row0 + q * 32;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * GT_BN + g * (GT_BN / 2);
      // Both 64-column rounds go to registers (packed bf16) first, so the accumulator is back with the tensor pipe before
      // a single store is issued.  Tiles that end inside a group's rows are masked by hand; all others leave through
      // bulk tensor stores, which clip at the tensor's own bounds.
      uint32_t pk[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int nc = it.n0 + g * (GT_BN / 2) + c * 64;
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
      if (lane == 0) mbar_arrive(&tmem_empty[as]);
      const bool use_tma = p.tma_store != 0 && (p.group_offs == nullptr || row0 + 32 <= it.row_end);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int nc = it.n0 + g * (GT_BN / 2) + c * 64;
        if (nc < p.N)
          store_tile64_packed(slab, pk[c], &map_out, use_tma, nc, row0, p.out, p.ldo, it.row_end - row0, p.N - nc, vec_ok,
                              lane);
      }
      ++acc_iter;
    }
    if (lane == 0) tma_store_wait_all();         // this lane's bulk stores are done before shared memory is given back
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace ob

extern "C" int ob_gemm_tn(const void* a, const void* b, const void* a2, const void* b2, const void* bias, void* out,
                          long long rows_a, int N, int K1, int K2, long long lda, long long ldb, long long lda2,
                          long long ldb2, long long ldo, int b_kn, const int* group_offs, int num_groups,
                          int* status, double wait_budget_s, int num_sms, void* stream) {
  using namespace ob;
  if (rows_a <= 0 || N <= 0 || K1 <= 0) return 0;
  if (rows_a > 0x7fffffffLL - GT_BM) return -40;
  if (group_offs != nullptr && (num_groups < 1 || num_groups > GT_MAX_GROUPS)) return -41;
  if (K2 > 0 && (a2 == nullptr || b2 == nullptr)) return -42;
  const int groups = group_offs ? num_groups : 1;
  CUtensorMap ma, mb, ma2, mb2;
  int rc = make_bf16_map_2d(&ma, a, rows_a, K1, lda, GT_BK, GT_BM);
  if (rc) return rc;
  if (b_kn)
    rc = make_bf16_map_2d(&mb, b, static_cast<long long>(groups) * K1, N, ldb, 64, GT_BK);
  else
    rc = make_bf16_map_2d(&mb, b, static_cast<long long>(groups) * N, K1, ldb, GT_BK, GT_BN);
  if (rc) return rc;
  if (K2 > 0) {
    rc = make_bf16_map_2d(&ma2, a2, rows_a, K2, lda2, GT_BK, GT_BM);
    if (rc) return rc;
    rc = make_bf16_map_2d(&mb2, b2, N, K2, ldb2, GT_BK, GT_BN);
    if (rc) return rc;
  } else {
    ma2 = ma;
    mb2 = mb;
  }
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_tn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM) != cudaSuccess)
      return -43;
    configured = true;
  }
  GemmParams p;
  p.M = static_cast<int>(rows_a);
  p.N = N; p.K1 = K1; p.K2 = K2;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.group_offs = group_offs;
  p.num_groups = num_groups;
  p.b_group_rows = b_kn ? K1 : N;
  p.status = status;
  p.wait_budget_ns = static_cast<unsigned long long>(wait_budget_s * 1e9);
  const long long tiles_n = (N + GT_BN - 1) / GT_BN;
  const long long tiles_m_bound = (rows_a + GT_BM - 1) / GT_BM + (group_offs ? groups : 0);
  const long long total = tiles_m_bound * tiles_n;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  CUtensorMap mo = ma;
  p.tma_store = 0;
  if ((reinterpret_cast<uintptr_t>(out) & 15) == 0 && ((ldo * 2) & 15) == 0 &&
      make_bf16_map_2d(&mo, out, rows_a, N, ldo, 64, 32) == 0)
    p.tma_store = 1;
  if (b_kn)
    gemm_tn_kernel<true><<<grid, GT_THREADS, GT_SMEM, static_cast<cudaStream_t>(stream)>>>(ma, mb, ma2, mb2, mo, p);
  else
    gemm_tn_kernel<false><<<grid, GT_THREADS, GT_SMEM, static_cast<cudaStream_t>(stream)>>>(ma, mb, ma2, mb2, mo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -44;
}
