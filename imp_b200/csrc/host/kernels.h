// Declarations of the kernel launchers of this library (defined in the .cu files beside this
// folder) for the host code.  Every launcher returns 0, a negative argument error (-2: the kernel
// does not take this shape), or a cudaError_t; imp_last_error() has the text.
#pragma once

#include <stdint.h>

extern "C" {

const char* imp_last_error(void);
const char* imp_status_string(int code);
int imp_device_arch(void);
int imp_device_sm_count(void);

int imp_embedding(float* out, const void* table, const int* ids, int n_tokens, int d, int vocab, int table_dtype,
                  float scale, int* status, void* stream);
int imp_swiglu(void* out, const void* gate_up, int n_tokens, int F, int block, int dtype, void* stream);
int imp_cast(void* dst, int dst_dtype, const void* src, int src_dtype, int64_t n, void* stream);
int imp_random_fill(void* out, int dtype, int64_t n, uint64_t tensor_seed, int mode, float std, float norm_std,
                    int round_bf16, void* stream);
int imp_tensor_stats(const void* x, int dtype, int64_t n, float* out5, void* stream);

int imp_add_rmsnorm(float* h, const void* branch, const void* w, void* out, const int* rows, int n_out_rows, int d,
                    float eps, float weight_offset, int act_dtype, int w_dtype, int write_h, void* stream);
int imp_add_rmsnorm_split(float* h, const float* part, int64_t split_stride, int n_splits, const void* w, void* out,
                          const int* rows, int n_out_rows, int d, float eps, float weight_offset, int act_dtype,
                          int w_dtype, int write_h, void* stream);
int imp_rmsnorm_rows(const void* x, int64_t x_stride, const void* w, void* out, int64_t out_stride, int n_rows, int d,
                     float eps, float weight_offset, int act_dtype, int w_dtype, void* stream);

int imp_qk_norm_rope_kv_write(void* qkv, int64_t row_stride, int n_tokens, int Hq, int Hkv, int Dh, const void* q_norm_w,
                              const void* k_norm_w, float eps, float weight_offset, int w_dtype, const float* cos_tab,
                              const float* sin_tab, int rot_dim, int max_pos, const int* positions,
                              const int* seq_of_token, const int* block_table, int bt_stride, int n_seqs, void* k_cache,
                              void* v_cache, int page_size, int num_pages, int act_dtype, int* status, void* stream);

int imp_paged_attention_generic(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* k_cache,
                                const void* v_cache, const int* block_table, int bt_stride, const int* seq_of_token,
                                const int* positions, int n_tokens, int n_seqs, int Hq, int Hkv, int Dh, int page_size,
                                int num_pages, float scale, int window, int dtype, int* status, void* stream);

int imp_paged_attention_generic_bias(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* k_cache,
                                     const void* v_cache, const int* block_table, int bt_stride, const int* seq_of_token,
                                     const int* positions, int n_tokens, int n_seqs, int Hq, int Hkv, int Dh, int page_size,
                                     int num_pages, float scale, int window, const float* bias, int n_dist, const float* sink,
                                     int dtype, int* status, void* stream);
int imp_proj_norm_kv_write(void* qk, int64_t row_stride, int n_tokens, int Hq, int Hkv, int Dh, const float* b_q, const float* b_k,
                           const float* w_q, const float* w_k, float eps, float temp_coef, int temp_every, const int* positions,
                           const int* seq_of_token, const int* block_table, int bt_stride, int n_seqs, void* k_cache,
                           void* v_cache, int page_size, int num_pages, int act_dtype, int* status, void* stream);
int imp_add_bias(void* x, int64_t stride, int n_rows, int n_cols, const float* bias, int dtype, void* stream);
int imp_scaled_sum(void* out, const void* x, float a, const void* y, float b, const float* col_bias, float bias_scale, int n_rows,
                   int n_cols, int dtype, void* stream);
int imp_gdr_prepare(const void* proj, int64_t ld, const float* conv_w, int taps, float* conv_state, const int* seq_of_token,
                    const int* q_start, const int* slots, int n_tokens, int n_seqs, int G, int D, int H, int Dv, const float* a_log,
                    const float* dt_bias, float* qn, float* kn, float* vc, float* beta, float* decay, int update_state, int act_dtype,
                    int* status, void* stream);
int imp_gdr_conv_state(const void* proj, int64_t ld, float* conv_state, int taps, int C, const int* q_start, const int* slots,
                       int n_seqs, int act_dtype, void* stream);
int64_t imp_gdr_state_floats(int H, int D, int Dv);
int imp_gdr_scan(const float* qn, const float* kn, const float* vc, const float* beta, const float* decay, float* state, float* out,
                 const int* q_start, const int* slots, int n_seqs, int G, int D, int H, int Dv, void* stream);
int imp_gdr_output(void* y, const float* o, const void* gate, int64_t gate_ld, const float* w, float eps, int n_tokens, int H, int Dv,
                   int act_dtype, void* stream);

int imp_gemm_f32(float* C, int64_t ldc, const float* A, int64_t lda, const float* W, int64_t ldw, int M, int N, int K,
                 void* stream);
int imp_gemm_bf16_plain(void* C, int64_t ldc, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, int M,
                        int N, int K, void* stream);
int imp_gemm_bf16_small_m(void* C, int64_t ldc, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw,
                          int M, int N, int K, void* stream);
int imp_gemm_bf16_stream(void* C, int64_t ldc, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, int M,
                         int N, int K, void* stream);
int imp_gemm_bf16_stream_swiglu(void* C, int64_t ldc, const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N,
                                int K, void* stream);
int imp_gemm_bf16_stream_gated(void* C, int64_t ldc, const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N,
                               int K, int act, void* stream);
int imp_gemm_bf16_tc_splits(int M, int N, int K);
int imp_gemm_bf16_tc_partials(float* scratch, const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N, int K, int* status,
                              void* stream);
int imp_gemm_bf16_tc(void* C, int64_t ldc, int epilogue, const void* A, int64_t lda, const void* W, int64_t ldw, int M,
                     int N, int K, int* status, void* stream);
int64_t imp_gemm_bf16_tc_swap_scratch_floats(int M, int N, int K, int epilogue);
int imp_gemm_bf16_tc_swap(void* C, int64_t ldc, int epilogue, const void* A, int64_t lda, const void* W, int64_t ldw, int M,
                          int N, int K, float* scratch, int* status, void* stream);
int imp_gemm_bf16_tc_swap_splits(int M, int N, int K);
int imp_gemm_bf16_tc_swap_partials(float* scratch, const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N,
                                   int K, int* status, void* stream);
int imp_gemm_bf16_tc_swap_sum(void* C, int64_t ldc, int epilogue, const float* scratch, int M, int N, int splits,
                              void* stream);
int imp_gemm_bf16_tc_qkv_rope(const void* A, int64_t lda, const void* W, int64_t ldw, int M, int K, int Hq, int Hkv, int Dh,
                              const float* q_norm_w, const float* k_norm_w, float eps, const float* cos_tab,
                              const float* sin_tab, int max_pos, const int* positions, const int* seq_of_token,
                              const int* block_table, int bt_stride, int n_seqs, void* q_out, int64_t q_stride,
                              void* k_cache, void* v_cache, int page_size, int num_pages, int* status, void* stream);

int imp_argmax_scratch_words(int n_rows);
int imp_argmax(const float* logits, int64_t ld, int n_rows, int V, int* out, void* scratch, void* stream);
int imp_apply_penalties(float* logits, int64_t ld, int n_rows, int V, const int* history, const int* hist_start,
                        int max_hist, const float* rep, const float* freq, const float* pres, int* counts_scratch,
                        void* stream);
int imp_sample(const float* logits, int64_t ld, int n_rows, int V, const float* temperature, const int* top_k,
               const float* top_p, const float* min_p, const float* uniform, int* out, void* stream);
int imp_sparse_subtract(float* logits, int64_t ld, int n_rows, int V, const int* rows, const int* tokens,
                        const float* values, int n, void* stream);
int imp_typical_filter(float* logits, int64_t ld, int n_rows, int V, const float* typical_p, const float* min_p,
                       void* stream);
int imp_sample_mirostat(const float* logits, int64_t ld, int n_rows, int V, const int* active, const float* temperature,
                        const float* mu, const float* uniform, int* out, float* surprise, void* stream);

// layer norm with the residual sum, and streams whose branches carry a factor per column (layernorm.cu)
int imp_add_layernorm(float* h, const void* branch, const float* col_scale, const void* w, void* out, const int* rows,
                      int n_out_rows, int d, float eps, int act_dtype, int w_dtype, int write_h, void* stream);
int imp_scale_columns(void* x, int64_t stride, int n_rows, int n_cols, const float* s, int dtype, void* stream);
int imp_concat_streams(void* out, const float* h, const void* branch, const float* col_scale, const float* x0, int n_rows,
                       int d, int act_dtype, void* stream);
int imp_add_layernorm_ex(float* h, float h_mult, const void* branch, const float* col_scale, const void* w, const void* bias, void* out,
                         const int* rows, int n_out_rows, int d, float eps, int act_dtype, int w_dtype, int write_h, void* stream);
int imp_add_normed_layernorm(float* h, const void* branch, const void* bw, const void* bb, float eps_b, const void* w, const void* bias,
                             float eps, void* out, const int* rows, int n_out_rows, int d, int act_dtype, int w_dtype, int write_h,
                             void* stream);
int imp_add_normed_layernorm_conv(float* h, const void* branch, const void* bw, const void* bb, float eps_b, const void* w, const void* bias,
                                  float eps, void* out, int n_rows, int d, int act_dtype, int w_dtype, const float* conv_w, int taps,
                                  float* conv_state, const int* seq_of_token, const int* slots, void* stream);
// the general scan over a decaying matrix state and the kernels around it (delta_rule.cu)
int imp_lsr_scan(int mode, const float* kw, const float* q, const float* w, const float* p, const float* z, const float* v,
                 const float* scal, const float* head_decay, float* state, float* out, const int* q_start, const int* slots,
                 int n_seqs, int D, int H, int Dv, void* stream);
int imp_retention_prepare(const void* proj, int64_t ld, int n_tokens, int H, int D, int Dv, float k_scale, float* q, float* kw, float* v,
                          float* scal, int act_dtype, void* stream);
int imp_retention_prepare_ex(const void* proj, int64_t ld, int n_tokens, int H, int D, int Dv, float k_scale, int act, float* q, float* kw,
                             float* v, float* scal, int act_dtype, void* stream);
int imp_lsr_output_row(void* y, const float* o, const void* gate, int64_t gate_ld, const float* w, int gate_act, float eps, int n_tokens,
                       int n, int act_dtype, void* stream);
int imp_gdelta_prepare(const void* proj, int64_t ld, const float* dlog, const float* w0, const float* a_bias, float decay_scale,
                       float unit_eps, int n_tokens, int H, int D, float* q, float* kw, float* w, float* p, float* z, float* v,
                       float* scal, int act_dtype, void* stream);
int imp_gdrc_prepare(const void* proj, int64_t ld, const float* conv_w, int taps, const float* conv_state, const int* seq_of_token,
                     const int* q_start, const int* slots, int n_tokens, int n_seqs, int G, int D, int H, int Dv, const float* dpre,
                     const float* a_log, const float* dt_bias, float unit_eps, float* q, float* kw, float* w, float* v, float* scal,
                     int act_dtype, int* status, void* stream);
int imp_gdr_output_ex(void* y, const float* o, const void* gate, int64_t gate_ld, const float* w, int w_head_stride, int gate_act,
                      float eps, int n_tokens, int H, int Dv, int act_dtype, void* stream);
// attention with normalised, partly rotated, scaled and gated heads; blocks of two mixers (qkv_prepare.cu)
int imp_qkv_prepare(const void* proj, int64_t ld, int n_tokens, int Hq, int Hkv, int D, int Dv, int Dc, const float* q_norm_w,
                    const float* k_norm_w, float eps, int v_norm, const float* inv_freq, int rot, const float* head_mult,
                    const int* positions, const int* seq_of_token, const int* block_table, int bt_stride, int n_seqs, void* q_out,
                    int64_t q_ld, void* k_cache, void* v_cache, int page_size, int num_pages, int act_dtype, int* status,
                    void* stream);
int imp_qkv_prepare_ex(const void* proj, int64_t ld, int n_tokens, int Hq, int Hkv, int D, int Dv, int Dc, const float* q_norm_w,
                       const float* k_norm_w, float eps, int v_norm, const float* inv_freq, int rot, int pairing, int v_share,
                       const float* head_mult, const int* positions, const int* seq_of_token, const int* block_table, int bt_stride,
                       int n_seqs, void* q_out, int64_t q_ld, void* k_cache, void* v_cache, int page_size, int num_pages, int act_dtype,
                       int* status, void* stream);
int imp_diff_combine(void* y, const void* attn, int64_t ld, int n_tokens, int G, int R, int Dc, int Dv, const float* lambda, float eps,
                     float out_scale, int dtype, void* stream);
int imp_head_gate(void* y, int64_t y_ld, const void* g, int64_t g_ld, int n_tokens, int H, int Dv, int dtype, void* stream);
int imp_rms_pair_mean(void* out, const void* a, const float* wa, float ca, const void* b, const float* wb, float cb, int n_rows, int d,
                      float eps, int dtype, void* stream);
int imp_gated_act(void* out, const void* gate_up, int n_tokens, int F, int block, int act, int dtype, void* stream);
int imp_act_rows(void* out, const void* x, int64_t ld, int n_tokens, int n, int act, int dtype, void* stream);
int imp_gather_head_cols(void* dst, const void* src, int n_tokens, int H, int ds, int n, int dtype, void* stream);
// a short causal convolution added to its input; a normalised polynomial as activation (short_conv.cu)
int imp_add_conv(void* out, const void* x, int64_t ld, const float* w, int taps, float* state, const int* seq_of_token, const int* q_start,
                 const int* slots, int n_tokens, int n_seqs, int C, int shift_state, int dtype, int* status, void* stream);
int imp_polynorm(void* out, const void* z, int64_t ld, int n_tokens, int n, const float* coef, float eps, int dtype, void* stream);
// products over groups: per-head matrices, routed experts (grouped_gemm.cu)
int imp_grouped_gemm(void* C, int64_t ldc, int64_t c_group_cols, const void* A, int64_t lda, int64_t a_group_cols,
                     const int* a_rows, const void* W, const void* W2, int64_t w_group_stride, int64_t ldw, const int* seg,
                     int M, int N, int K, int G, int swiglu, int dtype, void* stream);
int imp_transpose_groups(void* dst, const void* src, int G, int R, int Cn, int dtype, void* stream);
// latent attention (latent_attention.cu)
int imp_latent_prepare(const void* proj, int64_t ld, int n_tokens, int q_rank, int kv_rank, int rot, const float* wq,
                       const float* wkv, float eps, void* cq, int64_t cq_ld, const float* cos_tab, const float* sin_tab,
                       int rot_dims, int max_pos, const int* positions, const int* seq_of_token, const int* block_table,
                       int bt_stride, int n_seqs, void* pages, int page_size, int num_pages, int act_dtype, int* status,
                       void* stream);
int imp_latent_query_rope(const void* q, int64_t q_ld, int n_tokens, int H, int D, int rot, void* out, int64_t out_ld, int kv_rank,
                          const float* cos_tab, const float* sin_tab, int rot_dims, int max_pos, const int* positions,
                          int act_dtype, int* status, void* stream);
// the wkv recurrence (wkv.cu)
int imp_wkv_max_head_dim(void);
int imp_wkv_mix(const void* x, int64_t ldx, const float* mu, float* prev_state, const int* seq_of_token, const int* q_start,
                const int* slots, int n_tokens, int n_seqs, int d, void* out, int update_state, int act_dtype, int* status,
                void* stream);
int imp_tanh_inplace(void* x, int64_t n, int dtype, void* stream);
int imp_wkv_scan(const void* r, const void* k, const void* v, int64_t ld, const float* dlog, const float* w0, const float* u,
                 float* state, float* out, const int* q_start, const int* slots, int n_seqs, int H, int D, int act_dtype,
                 void* stream);
int imp_wkv_output(void* y, const float* o, const void* g, int64_t ldg, const float* w, float eps, int n_tokens, int H, int D,
                   int act_dtype, void* stream);
// routed experts (moe.cu)
int imp_moe_route(const void* x, int64_t ldx, int n_tokens, int d, const float* wr, const float* br, int E, int top, const float* wg,
                  int* idx, float* wts, float* gate, int act_dtype, void* stream);
int imp_moe_route_ex(const void* x, int64_t ldx, int n_tokens, int d, const float* wr, const float* br, int E, int top, const float* wg,
                     int* idx, float* wts, float* gate, int score_mode, int n_groups, int keep, float weight_scale, int act_dtype, void* stream);
int imp_moe_sort(const int* idx, int n_tokens, int top, int E, int* seg, int* row_token, int* pair_row, void* stream);
int imp_gather_rows(void* dst, const void* src, int64_t ld, const int* idx, int n_rows, int d, int dtype, void* stream);
int imp_moe_combine(void* out, const void* y, const int* pair_row, const float* wts, int n_tokens, int top, const void* shared,
                    const float* gate, int d, int act_dtype, void* stream);
}

// Epilogues of the tcgen05 products.
enum { TC_OUT_BF16 = 0, TC_OUT_F32 = 1, TC_OUT_SWIGLU = 2, TC_OUT_GEGLU = 4 };   // 2 / 4: act(gate) * up, act silu / gelu (tanh form)
