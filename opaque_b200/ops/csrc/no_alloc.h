// Entry point that allocates nothing.  It has no counterpart in the reference library.
//
// Who needs it: code that runs where device memory must not be requested — inside a CUDA-graph capture or a
// memory-pool-locked inference server loop, in a real-time or safety-certified process whose memory plan is fixed at
// start-up, under a host framework that owns the whole device heap and hands none of it to third-party libraries, or
// in an out-of-memory handler.  For such callers `cudaMalloc` (and any library routine that may call it behind the
// scenes, including a tensor framework's caching allocator) is off limits, yet the fused output-head + cross-entropy
// kernel needs scratch memory for its per-tile softmax statistics.
//
// ob_linear_ce_fwd_noalloc is ob_linear_ce_fwd (forward only: losses and log-sum-exps, no stored logits) with that
// scratch taken from a fixed array that lives in the library image itself:
//
//   * Limit: rows * 2 * ceil(N / 256) must not exceed OB_NO_ALLOC_MAX_PARTIALS (2^20 sixteen-byte records = 16 MiB; for
//     example 1024 rows at a vocabulary of 128 256, or 2610 rows at 50 257).  A larger problem is REFUSED with the
//     return code OB_NO_ALLOC_TOO_LARGE and a message readable through ob_no_alloc_last_error(); nothing is launched.
//     Split the rows over several calls instead.
//   * Cost: every GPU on which the library is loaded holds those 16 MiB until the process exits, used or not.
//   * The first call on each device looks the array's device address up once (with that device current) and caches it.
//     Make that first call outside of any stream capture.
//   * All calls share the one array, and it keeps whatever the last call left in it.  Nothing in it has to start at zero:
//     each call writes every record it later reads.  Two calls that overlap on the GPU (different streams, or several
//     host threads launching at once on one device) race on it — serialise them on one stream.
//   * The caller still owns inputs and outputs: hidden [rows, K] and weight [N, K] (bf16, 16-byte aligned rows), labels
//     [rows] (int64), nll [rows] and lse [rows] (fp32; lse may be NULL), all device pointers of the current device.
//   * No cudaMalloc / cudaFree / allocating library routine is called, on the first call or later.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define OB_NO_ALLOC_MAX_PARTIALS (1 << 20)
#define OB_NO_ALLOC_TOO_LARGE (-60)

// Returns 0 on success, OB_NO_ALLOC_TOO_LARGE when the scratch array is too small for (rows, N), another negative code
// for a host-side failure (bad pointer alignment, launch error).  Device-side wait timeouts are reported through
// `status` (may be NULL) as for every tensor-core kernel of this library.
int ob_linear_ce_fwd_noalloc(const void* hidden, const void* weight, const long long* labels, float* nll, float* lse,
                             long long rows, int N, int K, long long ldh, long long ldw, float softcap, float smoothing,
                             long long ignore_index, int* status, double wait_budget_s, int num_sms, void* stream);

// Text of the last refusal / failure of ob_linear_ce_fwd_noalloc on the calling thread ("" if none).
int ob_no_alloc_last_error(char* buf, int len);

#ifdef __cplusplus
}
#endif
