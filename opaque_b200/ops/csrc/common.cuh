// Shared device helpers for the sm_100a kernels: PTX wrappers for mbarrier, TMA
// (cp.async.bulk.tensor), tcgen05 (TMEM alloc, UMMA issue/commit, TMEM loads),
// bounded waits, Philox-4x32-10 and small vector utilities.
//
// Every wait in this library is bounded: a spin that exceeds its time budget
// records an error code in a caller-provided status word and returns false, so
// a kernel can unwind (drain its own async copies, free TMEM) instead of
// hanging the GPU.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ob {

// ---------------------------------------------------------------------------------------------
// error codes written to the status word (first error wins)
enum : int {
  OB_OK = 0,
  OB_ERR_WAIT_FULL = 1,      // consumer gave up waiting for a TMA stage
  OB_ERR_WAIT_EMPTY = 2,     // producer gave up waiting for a free stage
  OB_ERR_WAIT_TMEM_FULL = 3, // epilogue gave up waiting for an accumulator
  OB_ERR_WAIT_TMEM_EMPTY = 4,
  OB_ERR_WAIT_SCALED = 5,
  OB_ERR_WAIT_PEER = 6,      // a peer's flag did not arrive in time
  OB_ERR_DRAIN = 7,
  OB_ERR_CLAIM = 8,          // a tile-claim word was shared by two launches in flight
};

__device__ __forceinline__ void set_error(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t.reg .b32 R;\n\t"
      "elect.sync R|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` is a CTA-shared word: once any role of the CTA has
// given up, every other wait in the CTA returns false promptly as well.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code, uint64_t budget_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > budget_ns) {
        *abort_flag = 1;
        set_error(status, code);
        return false;
      }
    }
  }
}

// generic-proxy writes to shared memory -> visible to the async proxy (UMMA / TMA reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA: 2-D tiled load, completion on an mbarrier of this CTA.  c0 is the innermost
// coordinate and must keep (c0 * element size) a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The barrier receives one arrival once every UMMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 16 consecutive fp32 columns (half the registers of tmem_ld32 in flight).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format: version field = 1).
//   bits [0,14)  start address >> 4        bits [16,30) leading-dimension byte offset >> 4
//   bits [32,46) stride byte offset >> 4   bits [46,48) version = 1
//   bits [61,64) swizzle: 0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle_code) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(swizzle_code & 7) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
//   [4,6) D fmt = 1 (f32)  [7,10) A fmt = 1 (bf16)  [10,13) B fmt = 1 (bf16)
//   bit 15 A major (1 = MN-major)  bit 16 B major  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// Philox-4x32-10 (Salmon et al.), counter-based: same (key, counter) -> same 4 words.
struct Philox4 {
  uint32_t x, y, z, w;
};
__host__ __device__ __forceinline__ void philox_mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
  const uint64_t p = static_cast<uint64_t>(a) * static_cast<uint64_t>(b);
  hi = static_cast<uint32_t>(p >> 32);
  lo = static_cast<uint32_t>(p);
}
__host__ __device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                          uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    philox_mulhilo(0xD2511F53u, c0, hi0, lo0);
    philox_mulhilo(0xCD9E8D57u, c2, hi1, lo1);
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return Philox4{c0, c1, c2, c3};
}
// Four independent N(0,1) samples for the counter block `blk` (coordinates 4*blk .. 4*blk+3),
// `stream` separates logically different noise draws under the same key.
//
// Box-Muller in fp32.  The radius uses all 32 bits of its uniform, u = (x + 0.5) / 2^32 in (0, 1], so the largest
// magnitude is sqrt(-2 ln 2^-33) = 6.76 standard deviations (two-sided mass beyond it: 1.4e-11); the angle uses 24 bits.
// Logarithm and sine / cosine are the accurate library functions (this header's callers that draw noise are compiled
// without approximate math); sincospif needs no range reduction for an argument in [0, 2).
__device__ __forceinline__ float4 philox_normal4(uint64_t seed, uint64_t blk, uint32_t stream) {
  const Philox4 r = philox4x32_10(static_cast<uint32_t>(blk), static_cast<uint32_t>(blk >> 32), stream, 0u,
                                  static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
  const float s32 = 1.0f / 4294967296.0f, s24 = 1.0f / 16777216.0f;
  // float(x) rounds large x to 24 bits (then u may be exactly 1 and the radius 0); small x, the tail, is exact
  const float u0 = fminf((static_cast<float>(r.x) + 0.5f) * s32, 1.0f);
  const float u2 = fminf((static_cast<float>(r.z) + 0.5f) * s32, 1.0f);
  const float a1 = static_cast<float>(r.y >> 8) * s24;          // angle / 2 pi in [0, 1)
  const float a3 = static_cast<float>(r.w >> 8) * s24;
  const float ra = sqrtf(-2.0f * logf(u0)), rb = sqrtf(-2.0f * logf(u2));
  float sa, ca, sb, cb;
  sincospif(2.0f * a1, &sa, &ca);
  sincospif(2.0f * a3, &sb, &cb);
  return make_float4(ra * ca, ra * sa, rb * cb, rb * sb);
}

// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// fp32 vector reduction into (possibly peer) global memory, system scope.
__device__ __forceinline__ void red_add_v4(float* addr, float4 v) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void red_add_f32(float* addr, float v) {
  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

// v[0 .. 63] += bias[nc .. nc + 63] (bf16 values, the same for every row): one 16-byte load per 8 columns when the
// slice is aligned and inside N (64 scalar loads per thread made the epilogue LSU-bound: 12 % of a 512 x 256 tile).
__device__ __forceinline__ void add_bias64(float* v, const __nv_bfloat16* bias, int nc, int N) {
  if (nc + 64 <= N && (reinterpret_cast<uintptr_t>(bias + nc) & 15) == 0) {
    const uint4* bp = reinterpret_cast<const uint4*>(bias + nc);
#pragma unroll
    for (int j8 = 0; j8 < 8; ++j8) {
      const uint4 pk = __ldg(bp + j8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = __bfloat1622float2(h[t]);
        v[8 * j8 + 2 * t] += f.x;
        v[8 * j8 + 2 * t + 1] += f.y;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 64; ++j)
      if (nc + j < N) v[j] += __bfloat162float(__ldg(bias + nc + j));
  }
}

// ---------------------------------------------------------------------------------------------
// Epilogue stores through the TMA engine.  A warp writes its [32 rows x 64 columns] bf16 tile into a 4 KB shared-memory
// slab in the 128-byte-swizzled layout the tensor map expects (16-byte chunk j of row r at chunk position j ^ (r & 7);
// the slab is 1024-byte aligned), and one lane issues a bulk tensor store.  Rows and columns outside the tensor are
// clipped by the hardware.  Against 16-byte st.global per lane this halves the bytes the SM pushes into the crossbar
// (measured: 266 MB vs 134 MB for a 134 MB output) and takes the stores off the warp's critical path; a drain of a
// 128 x 256 accumulator half by eight warps took 4.4 k clocks with st.global.
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the issuing thread's earlier bulk stores have finished READING shared memory (the slab may be rewritten)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... have finished altogether (before the kernel gives its shared memory back)
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// pk[0 .. 31]: this lane's row of 64 bf16 values, two per register.  `use_tma` is warp-uniform.  Without it (unaligned
// output, or rows that must be masked at a bound the tensor map does not know) the tile leaves through the slab as
// 16-byte st.global row segments, or element by element when even that is not aligned.
__device__ __forceinline__ void store_tile64_packed(uint8_t* slab, const uint32_t* pk, const CUtensorMap* map, bool use_tma,
                                                    int col0, int row0, __nv_bfloat16* out, long long ldo, int rows_valid,
                                                    int cols_valid, bool vec_ok, int lane) {
  if (lane == 0) tma_store_wait_read();
  __syncwarp();
  if (!use_tma && !vec_ok) {
    if (lane < rows_valid) {
      __nv_bfloat16* dst = out + static_cast<long long>(row0 + lane) * ldo + col0;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&pk[j]);
        if (2 * j < cols_valid) dst[2 * j] = h.x;
        if (2 * j + 1 < cols_valid) dst[2 * j + 1] = h.y;
      }
    }
    return;
  }
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<uint4*>(slab + lane * 128 + ((c ^ (lane & 7)) << 4)) =
        make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
  if (use_tma) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map, slab, col0, row0);
      tma_store_commit();
    }
    return;
  }
  __syncwarp();
  const int c = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3);
    const uint4 q = *reinterpret_cast<const uint4*>(slab + r * 128 + ((c ^ (r & 7)) << 4));
    if (r < rows_valid) {
      __nv_bfloat16* dst = out + static_cast<long long>(row0 + r) * ldo + col0 + 8 * c;
      if (8 * c + 8 <= cols_valid) {
        *reinterpret_cast<uint4*>(dst) = q;
      } else if (8 * c < cols_valid) {
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&q);
        for (int j = 0; j < cols_valid - 8 * c; ++j) dst[j] = e[j];
      }
    }
  }
  __syncwarp();
}

}  // namespace ob
