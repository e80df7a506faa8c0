// C entry points of the kernels (raw pointers + stream); the torch bindings and C callers use these.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- counter.cpp ----
void mb_count_launch(int n);
long long mb_launch_count();
int mb_pdl_enabled(void);      // programmatic dependent launch for the kernels that support it (pdl.cuh); MILES_PDL=0 disables
void mb_set_pdl(int on);

// ---- gemm.cu ----
int mb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                 int a_mn, int b_mn, int out_fp32, int accumulate, const void* bias, int force_bn, int* error_flag,
                 cudaStream_t stream);
int mb_gemm_bf16_splitk(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                        int out_fp32, int accumulate, const void* bias, int split_k, float* ws, int* counters, int* error_flag,
                        cudaStream_t stream);
int mb_gemm_bf16_grouped(const void* A, const void* B, void* C, int M_pad, int N, int K, int num_experts,
                         const int* tile_expert, int b_mn, int out_fp32, int force_bn, int* error_flag, cudaStream_t stream);
// ---- gemm_small.cu: weights on the 128-row MMA side, tokens in tiles of bt ∈ {16, 32, 64} ----
int mb_gemm_small(const void* X, const void* W, void* C, int tokens, int N, int K, long long ldx, long long ldw, long long ldc,
                  int out_fp32, const void* bias, int bt, int split_k, float* ws, int* counters, int* error_flag, cudaStream_t stream);
int mb_gemm_small_grouped(const void* X, const void* W, void* C, int rows, int N, int K, int num_experts, const int* tile_expert,
                          const int* used_rows, int bt, int* error_flag, cudaStream_t stream);
// ---- gemv.cu: ≤ 16 tokens (dense) / ≤ 8 tokens (MoE), no pipeline set-up ----
int mb_gemv(const void* x, const void* residual, const void* norm_w, float eps, const void* W, const void* bias, void* y, long long ldy,
            int out_fp32, void* res_out, void* xn_out, int M, int N, int K, int static_w, cudaStream_t s);
int mb_moe_gemv(const void* x, const void* w13, const void* w2, const int* topk_idx, const float* topk_w, void* act, void* out, int T, int k,
                int E, int expert_offset, int H, int F, cudaStream_t s);
int mb_gemm_bf16_grouped_wgrad(const void* dY, const void* X, void* dW, int M_pad, int N, int K, int num_experts,
                               const int* seg_offsets, int out_fp32, int accumulate, int force_bn, int* error_flag,
                               cudaStream_t stream);

// ---- elementwise.cu ----
int mb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* res_out, float* rstd, long long T, int H,
                   float eps, cudaStream_t s);
int mb_rmsnorm_bwd_blocks(long long T);
int mb_rmsnorm_bwd(const void* x, const void* w, const void* dy, const void* dres, const float* rstd, void* dx, float* dw_partial,
                   void* dw_out, int dw_fp32, long long T, int H, cudaStream_t s);
// RMSNorm backward that allocates nothing.  This entry point has no counterpart in the reference framework, whose
// kernels all take their workspaces from the PyTorch caching allocator; it exists for callers that cannot allocate:
// a C or C++ host without torch, code running under an allocator that is frozen or being snapshotted (the sleep /
// wake-up window in which the trainer's device memory is handed to the rollout engine), and latency-critical paths
// where an allocator call may synchronise the device.
//   * Same arguments and results as mb_rmsnorm_bwd minus `dw_partial`: the partial sums go to a fixed array in device
//     memory (592 × MB_RMSNORM_BWD_STATIC_MAX_H floats ≈ 9.7 MB, one per device, reserved when the module loads).
//   * H > MB_RMSNORM_BWD_STATIC_MAX_H returns MB_ERR_STATIC_SCRATCH_TOO_SMALL; mb_rmsnorm_bwd_static_strerror() gives text.
//   * The first call on each device looks up the array's address with cudaGetSymbolAddress; make that call before any
//     stream capture begins.  Later calls only launch the two kernels.
//   * The array is shared by all calls on a device and keeps its last contents.  Nothing needs to be zeroed: each call
//     writes every element it later reads.  Calls that overlap on one device race on it; the caller serialises them.
#define MB_RMSNORM_BWD_STATIC_MAX_H 4096
#define MB_ERR_STATIC_SCRATCH_TOO_SMALL (-2)
#define MB_ERR_STATIC_SCRATCH_SETUP (-3)
int mb_rmsnorm_bwd_static(const void* x, const void* w, const void* dy, const void* dres, const float* rstd, void* dx, void* dw_out,
                          int dw_fp32, long long T, int H, cudaStream_t s);
const char* mb_rmsnorm_bwd_static_strerror(int code);
int mb_colsum(const float* partial, void* out, int R, int C, int out_fp32, cudaStream_t s);
int mb_swiglu_fwd(const void* in, void* out, long long T, int F, const int* rows_ptr, cudaStream_t s);
int mb_swiglu_bwd(const void* in, const void* dout, void* din, long long T, int F, const int* rows_ptr, cudaStream_t s);
int mb_qk_norm_rope_fwd(const void* q, const void* k, long long q_stride, long long k_stride, const void* qw, const void* kw,
                        const int* positions, void* qo, void* ko, float* q_rstd, float* k_rstd, long long T, int Hq, int Hk, int D,
                        float theta, float eps, cudaStream_t s);
int mb_rope(const void* x, void* y, const int* positions, long long T, int H, int D, long long tok_stride, float theta, int inverse,
            cudaStream_t s);
int mb_qk_norm_rope_cache(const void* q, const void* k, const void* v, long long q_stride, long long k_stride, long long v_stride,
                          const void* qw, const void* kw, const int* positions, void* qo, void* ko, void* kc, void* vc,
                          const long long* slots, long long T, int Hq, int Hk, int D, float theta, float eps, cudaStream_t s);
int mb_qk_norm_rope_bwd_blocks(long long T, int Hn);
int mb_qk_norm_rope_bwd(const void* x, long long x_stride, const void* w, const float* rstd, const void* dy, const int* positions,
                        void* dx, long long dx_stride, float* dw_partial, void* dw_out, long long T, int Hn, int D, float theta,
                        cudaStream_t s);
int mb_kv_cache_write(const void* k, const void* v, long long k_stride, long long v_stride, void* kc, void* vc,
                      const long long* slots, long long T, int row_elems, cudaStream_t s);
int mb_adamw(float* master, const float* grad, float* m, float* v, const float* decay_mask, const float* scale_ptr, void* param_out,
             int out_bf16, long long n, float lr, float b1, float b2, float eps, float wd, int step, cudaStream_t s);

// ---- attention.cu ----
int mb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_seqlens, int batch, int max_seqlen,
                 int total_tokens, long long q_stride, long long k_stride, long long v_stride, int Hq, int Hkv, int D, float scale,
                 int causal, cudaStream_t s);
int mb_flash_bwd_tc(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta, void* dq,
                    void* dk, void* dv, const int* cu_seqlens, int batch, int max_seqlen, int total_tokens, long long q_stride,
                    long long k_stride, long long v_stride, int Hq, int Hkv, float scale, int causal, int* error_flag, cudaStream_t s);
int mb_attn_delta(const void* o, const void* dout, float* delta, int total_tokens, int Hq, int D, cudaStream_t s);
int mb_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse, float* delta,
                 void* dq, void* dk, void* dv, const int* cu_seqlens, int batch, int max_seqlen, int total_tokens, long long q_stride,
                 long long k_stride, long long v_stride, int Hq, int Hkv, int D, float scale, int causal, cudaStream_t s);
int mb_paged_decode(const void* q, const void* kc, const void* vc, const int* block_table, const int* seq_lens, void* out,
                    float* part_o, float* part_ml, int batch, int max_blocks, int block_size, int Hq, int Hkv, int D, float scale,
                    int num_splits, cudaStream_t s);

// ---- attention_tc.cu (tcgen05 forward, head_dim 128) ----
int mb_flash_fwd_tc(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_seqlens, int batch, int max_seqlen,
                    int total_tokens, long long q_stride, long long k_stride, long long v_stride, int Hq, int Hkv, float scale,
                    int causal, int* error_flag, const int* cu_seqlens_k, int total_k_tokens, cudaStream_t s);
int mb_flash_fwd_tc_ctas_per_sm(void);

// ---- debug.cuh: index checks of the debug build (each returns −1 in a build without them) ----
int mb_elementwise_bounds_set_limit(int which, long long value);
int mb_elementwise_bounds_read(long long* out4, int clear);
int mb_moe_bounds_set_limit(int which, long long value);
int mb_moe_bounds_read(long long* out4, int clear);
int mb_paged_bounds_set_limit(int which, long long value);
int mb_paged_bounds_read(long long* out4, int clear);

// ---- moe.cu ----
int mb_router_topk(const float* logits, float* probs, float* topk_w, int* topk_idx, long long T, int E, int K, int normalize,
                   cudaStream_t s);
int mb_moe_align(const int* idx, int n, const int* n_ptr, int E, int expert_offset, int* seg_offsets, int* tile_expert, int* row_src,
                 int* dst_row, int max_rows, cudaStream_t s);
int mb_moe_align_pad(const int* idx, int n, const int* n_ptr, int E, int expert_offset, int* seg_offsets, int* tile_expert,
                     int* row_src, int* dst_row, int max_rows, int pad, cudaStream_t s);
int mb_moe_gather(const void* x, void* x_perm, const int* row_src, const int* seg_offsets, int E, int k, int H, int max_rows,
                  cudaStream_t s);
int mb_moe_combine(const void* y_perm, const float* w, const int* dst_row, void* out, long long T, int k, int H, int identity_rows,
                   cudaStream_t s);
int mb_moe_combine_bwd(const void* dout, const void* y_perm, const float* w, const int* row_src, const int* seg_offsets, int E,
                       void* dy_perm, float* dw, int k, int H, int max_rows, cudaStream_t s);

// ---- misc.cu ----
int mb_sample_logprob_split(const float* logits, const float* temperature, const uint8_t* greedy, const long long* seeds, long long step,
                            long long* tokens, float* logprobs, int B, int V, int parts, float* ws, int* counters, cudaStream_t s);
int mb_decode_advance(const long long* o_tok, const float* o_lp, const int* o_routed, long long* h_tok, float* h_lp, int* h_routed,
                      int routed_per_row, int* tok, int* pos, int* len, const int* block_table, int max_blocks, int block_size,
                      long long* slot, long long* seed, int B, int vocab, int* error_flag, cudaStream_t s);
int mb_sample_logprob(const float* logits, const float* temperature, const uint8_t* greedy, const long long* seeds, long long step,
                      long long* tokens, float* logprobs, int B, int V, cudaStream_t s);
int mb_logit_stats(const float* logits, long long ld, const long long* targets, float* stats, long long R, int Vc, int v0,
                   float inv_temp, int first, cudaStream_t s);
int mb_logit_stats_finish(const float* stats, float* logp, float* ent, float* lse, long long R, cudaStream_t s);
int mb_logit_grad(const float* logits, long long ld, const long long* targets, const float* lse, const float* ent, const float* g_lp,
                  const float* g_ent, void* dlogits, long long ldd, long long R, int Vc, int v0, float inv_temp, cudaStream_t s);

// ---- quant.cu ----
int mb_mxfp8_quant(const void* x, void* q, void* scales, long long numel, cudaStream_t s);
int mb_fp8_block_quant(const void* w, void* q, float* scale_inv, int M, int N, cudaStream_t s);
int mb_int4_fake_quant(const void* x, void* y, float* scales, int M, int N, int bm, int bn, int symmetric, cudaStream_t s);
int mb_block_fake_quant(const void* x, void* y, long long numel, int mode, cudaStream_t s);
int mb_nvfp4_qdq(const void* x, void* y, const float* global_amax, long long numel, int four_over_six, cudaStream_t s);
int mb_absmax(const void* x, float* out, long long numel, cudaStream_t s);

// ---- comm.cu (peer-memory kernels; *_ptrs are host arrays of `world` device addresses, one per rank) ----
int mb_barrier(const long long* flag_ptrs, int rank, int world, int channel, int* epochs, int* err, cudaStream_t s);
int mb_ar_add_rmsnorm(const long long* partial_ptrs, int world, const void* residual, const void* w, void* y, void* res_out,
                      long long T, int H, float eps, cudaStream_t s);
int mb_rs_reduce_sqnorm(const long long* grad_ptrs, int world, int rank, long long lo, long long hi, const float* norm_weight,
                        float* sqnorm, cudaStream_t s);
int mb_adam_allgather(float* master, const float* grad_shard, float* m, float* v, const float* decay_mask, const float* sqnorm,
                      float clip, const long long* param_ptrs, int world, long long lo, long long n, float lr, float b1, float b2,
                      float eps, float wd, int step, cudaStream_t s);
int mb_moe_dispatch(const void* x, const int* topk_idx, long long n_pairs, int k, int H, int e_local, int rank,
                    const long long* recv_x_ptrs, const long long* recv_meta_ptrs, const long long* counter_ptrs, int world,
                    int capacity, int* sent_row, int* err, cudaStream_t s);
int mb_moe_dispatch_signal(const void* x, const int* topk_idx, long long n_pairs, int k, int H, int e_local, int rank,
                           const long long* recv_x_ptrs, const long long* recv_meta_ptrs, const long long* counter_ptrs, int world,
                           int capacity, int* sent_row, int* err, const long long* flag_ptrs, int channel, int* epochs, int* ticket,
                           cudaStream_t s);
int mb_moe_recv_align(const void* meta, int* counter, int capacity, int E, int* seg_offsets, int* tile_expert, int* row_src, int max_rows,
                      int pad, const long long* flag_ptrs, int rank, int world, int channel, const int* epochs, int* err, cudaStream_t s);
int mb_moe_return_signal(const void* y_perm, const int* row_src, const void* meta, const int* seg_offsets, int E, int H, int max_rows,
                         const long long* ret_ptrs, int world, const long long* flag_ptrs, int rank, int channel, int* epochs, int* ticket,
                         cudaStream_t s);
int mb_moe_combine_wait(const void* ret, const float* w, const int* sent_row, void* out, long long T, int k, int H,
                        const long long* flag_ptrs, int rank, int world, int channel, const int* epochs, int* err, cudaStream_t s);
int mb_moe_scatter_known(const void* rows_in, int src_by_pair, const int* topk_idx, const int* sent_row, long long n_pairs, int k,
                         int H, int e_local, const long long* recv_x_ptrs, int world, cudaStream_t s);
int mb_moe_return(const void* y_perm, const int* row_src, const void* meta, const int* seg_offsets, int E, int H, int max_rows,
                  const long long* ret_ptrs, int world, cudaStream_t s);
int mb_recv_expert_ids(const void* meta, int* counter, int capacity, int* expert_ids, int* n_out, int clear_counter, cudaStream_t s);
int mb_sum_rows(const long long* src_ptrs, int world, void* out, long long numel, cudaStream_t s);
int mb_gather_rows(const long long* src_ptrs, int world, void* out, long long bytes_per_rank, cudaStream_t s);
int mb_stats_merge(const long long* stats_ptrs, int world, long long R, float* logp, float* ent, float* lse, cudaStream_t s);

// ---- extra.cu (other model families, quantisation tools) ----
int mb_grouped_rmsnorm(const void* x, int x_fp32, const float* w, float* out, float* rstd, long long T, int n, int C, float eps,
                       cudaStream_t s);
int mb_short_conv(const void* x, int fp32, const float* w, const int* bos, void* y, long long T, int D, int W, cudaStream_t s);
int mb_mhc_mix(const void* x, const void* res, const float* h_res, const float* h_post, void* out, int fp32, long long T, int n, int d,
               cudaStream_t s);
int mb_mhc_aggregate(const void* x, int fp32, const float* pre, float* out, long long T, int n, int d, cudaStream_t s);
int mb_hc_combine(const void* res, const void* y, const float* h_post, void* out, int fp32, long long T, int n, int C, cudaStream_t s);
int mb_act_quant_1x128(const void* x, void* q, void* qdq, float* scales, long long M, int N, int round_scale, cudaStream_t s);
int mb_fp8_dequant(const void* q, const float* scale_inv, const void* e8m0, void* out, long long M, int N, cudaStream_t s);
int mb_gather_rows_host(const void* table_dev, const long long* ids, void* out, long long n, int row_bytes, long long table_rows,
                        cudaStream_t s);

// ---- gemm_mxfp8.cu (block-scaled: e4m3 payload [rows, K] + e8m0 scales [rows, K/32]; K % 128 == 0) ----
int mb_gemm_mxfp8(const void* A, const void* sa, const void* B, const void* sb, void* C, int M, int N, int K, long long ldc,
                  int* error_flag, cudaStream_t stream);
int mb_gemm_mxfp8_grouped(const void* A, const void* sa, const void* B, const void* sb, void* C, int M_pad, int N, int K, int E,
                          const int* tile_expert, long long ldc, int* error_flag, cudaStream_t stream);

// ---- sparse_attn.cu ----
int mb_sparse_attention_fwd(const void* q, const void* k, const void* v, const int* indices, const float* sink, void* out, float* lse,
                            long long T, int H, int Hk, int D, int Dv, int K, long long Tkv, float scale, cudaStream_t s);

// ---- weight_sync.cu (one launch per bucket of tensors; dst may be peer memory) ----
int mb_multi_copy(const long long* table, const long long* prefix, int n, long long total_chunks, cudaStream_t s);
int mb_multi_copy2d(const long long* table, const long long* prefix, int n, long long total_items, int qdq, cudaStream_t s);
int mb_multi_mxfp8(const long long* table, const long long* prefix, int n, long long total_chunks, int qdq, cudaStream_t s);

// ---- gemm_comm.cu ----
int mb_ag_gemm(const long long* xg_ptrs, const void* W, void* Y, int* block_counters, int rows_per_rank, int N, int K, int rank,
               int world, const long long* flag_ptrs, int channel, int epoch, int* error_flag, cudaStream_t s);
int mb_comm_configure(int* err, unsigned long long wait_ns);
int mb_gemm_comm_configure(int* err, unsigned long long wait_ns);
int mb_gemm_rs(const void* X, const void* W, const long long* partial_ptrs, void* out, int* counters, int T, int N, int K, int rank,
               int world, const long long* flag_ptrs, int channel, int epoch, int* error_flag, cudaStream_t s);

#ifdef __cplusplus
}
#endif
