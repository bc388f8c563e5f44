// C entry points of libopaque_b200.so (every function returns 0 on success, a negative
// code on a host-side failure; device-side wait timeouts are reported through `status`).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int ob_wgrad_clip(const void* a, const void* b, int T, int M, int N, long long lda, long long ldb,
                  const float* row_scale, const int* seg_offsets, int num_groups, int splits, float* out,
                  float* const* peer_out, long long shard_elems, const long long* group_out_offset,
                  long long group_stride, long long out_offset, long long ldm, long long ldn, int n_valid,
                  int accumulate, int block_n, int* status, double wait_budget_s, int num_sms, void* stream);

// out[m, n] (+)= sum over examples e of ex_scale[e] * A_e^T B_e, where example e owns rows [e*ex_rows, (e+1)*ex_rows) of
// a [T, M] and b [T, N] (ex_rows a multiple of 64).  The factor is applied to each example's fp32 partial product in
// the epilogue; operands are not modified.  splits > 1 needs accumulate = 1.
int ob_wgrad_clip_pe(const void* a, const void* b, int num_examples, int ex_rows, int M, int N, long long lda,
                     long long ldb, const float* ex_scale, int splits, float* out, float* const* peer_out,
                     long long shard_elems, long long out_offset, long long ldm, int accumulate, int* status,
                     double wait_budget_s, int num_sms, void* stream);
// Direct per-example gradient norms on the same kernel: norm2[e] += || a_e^T b_e ||_F^2 (nothing else is written).
int ob_direct_norm2(const void* a, const void* b, int num_examples, int ex_rows, int M, int N, long long lda, long long ldb,
                    int splits, float* norm2, int* status, double wait_budget_s, int num_sms, void* stream);

int ob_ghost_norm(const void* a, const void* g, const int* ids, int B, int T, int Da, int Dg, long long lda,
                  long long ldg, float* norm2, const int* seg, const int* seg_out, long long total_rows, int* status,
                  double wait_budget_s, int num_sms, void* stream);

// D[M, N] = A[M, K1] op(B) + A2[M, K2] B2[N, K2]^T + bias, bf16 in / bf16 out, fp32 accumulation.  b_kn = 0: B is
// [N, K1] row-major (per group: [groups * N, K1]); b_kn = 1: B is [K1, N] row-major (per group: [groups * K1, N]).
// group_offs (int32 device array [num_groups + 1]) switches on the grouped mode: rows [offs[e], offs[e+1]) use slab e.
int ob_gemm_tn(const void* a, const void* b, const void* a2, const void* b2, const void* bias, void* out,
               long long rows_a, int N, int K1, int K2, long long lda, long long ldb, long long lda2, long long ldb2,
               long long ldo, int b_kn, const int* group_offs, int num_groups, int* status, double wait_budget_s,
               int num_sms, void* stream);

// Dense GEMM on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles):  D = A op1(B) + A2 op2(B2) + bias.
// b_kn / b2_kn = 1: that B operand is stored [K, N] row-major, 0: [N, K].  glu != 0: `b` holds the gate rows and `b_up`
// the up rows of a gated MLP ([N/2, K] each; N counts both), out [M, N/2] = act(gate) * up (glu_act: 0 silu, 1 gelu erf,
// 2 gelu tanh) and the optional out_gate / out_up receive the pre-activations.
int ob_gemm_pair(const void* a, const void* b, const void* b_up, const void* a2, const void* b2, const void* b2_up,
                 const void* bias, void* out, void* out_gate, void* out_up, long long rows_a, int N, int K1, int K2,
                 long long lda, long long ldb, long long lda2, long long ldb2, long long ldo, int b_kn, int b2_kn, int glu,
                 int glu_act, int* status, double wait_budget_s, int num_sms, void* stream);
// Data gradient of a gated MLP's down projection with the activation's backward in the epilogue: dH = dY op(W) stays in
// tensor memory; dGate = dH * up * act'(gate) and dUp = dH * act(gate) are stored (bf16 [M, N], pitch ld_out).  N % 64 == 0.
int ob_gemm_pair_glu_bwd(const void* dy, const void* w, const void* gate, const void* up, void* dgate, void* dup,
                         long long rows_a, int N, int K, long long lddy, long long ldw, long long ld_gu, long long ld_out,
                         int b_kn, int glu_act, int* status, double wait_budget_s, int num_sms, void* stream);
// Same product (store epilogue only) on 256 x 256 pair tiles with double-buffered accumulators: the variant for short K.
int ob_gemm_pair_db(const void* a, const void* b, const void* a2, const void* b2, const void* bias, void* out,
                    long long rows_a, int N, int K1, int K2, long long lda, long long ldb, long long lda2, long long ldb2,
                    long long ldo, int b_kn, int b2_kn, int* status, double wait_budget_s, int num_sms, void* stream);
// Die map of the current device (which SMs share a die, probed by atomic latency; once per device and process).
// ob_pair_init: probes if needed, returns 1000 * (SM pairs on die 0) + (SM pairs on die 1), 0 if no two-die split was
// found; call it outside stream captures.  ob_die_map: smid -> 0 / 1 into out[0 .. n), returns the SM count or 0.
int ob_pair_init(void);
int ob_pair_set_die_aware(int on);   // die-aware tile assignment of the pair GEMMs (default off); returns the old value
int ob_die_map(unsigned char* out, int n);
// Output head fused with cross-entropy statistics on CTA pairs: logits tiles stay in tensor memory, per-tile partials
// (scratch: rows * 2 * ceil(N / 256) float4) are combined in a fixed order into nll[rows], lse[rows]; `logits_out` (optional)
// receives the bf16 soft-capped logits for the backward pass.
int ob_linear_ce_fwd(const void* hidden, const void* weight, const long long* labels, void* logits_out, float* partials,
                     float* nll, float* lse, long long rows, int N, int K, long long ldh, long long ldw, long long ldo,
                     float softcap, float smoothing, long long ignore_index, int* status, double wait_budget_s,
                     int num_sms, void* stream);
// In place on those stored logits: z <- row_weight * d nll / d (raw logits), one read and one write per element.
int ob_linear_ce_dlogits(void* logits, const long long* labels, const float* lse, const float* row_weight, long long rows,
                         int N, long long ld, float softcap, float smoothing, long long ignore_index, void* stream);
unsigned int ob_debug_idesc_bf16(int m, int n, int a_mn_major, int b_mn_major);

// LayerNorm over the last dimension (bf16 in/out, fp32 statistics saved per row).
int ob_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, long long rows,
                     int H, float eps, void* stream);
int ob_layernorm_bwd_dx(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                        long long rows, int H, void* stream);
// out[e, :N] += sum over the rows of example e of g (mode 0), g * (x - mean) * rstd (mode 1) or g * x * rstd (mode 2);
// out row pitch ld_out.  In modes 1 and 2 a non-NULL out2 (row pitch ld_out2) also receives the plain sums of g.
int ob_rows_group_sum(const void* g, const void* x, const float* mean, const float* rstd, int num_examples,
                      int rows_per_example, int N, long long ldg, float* out, long long ld_out, int mode, float* out2,
                      long long ld_out2, void* stream);
// q, k, v gradients [B, heads, T, hd] (strides[9] = batch, head, token stride of each, in elements; head vectors
// contiguous) -> out [B*T, 3*heads*hd] bf16.
int ob_merge_heads3(const void* q, const void* k, const void* v, const long long* strides, void* out, long long B, int T,
                    int heads, int hd, int sms, void* stream);
// out = act(x) (dy == NULL) or dy * act'(x); act: 0 silu, 1 gelu erf, 2 gelu tanh, 3 relu.
int ob_activation(const void* x, const void* dy, void* out, long long numel, int act, int sms, void* stream);

#ifdef __cplusplus
}
#endif
