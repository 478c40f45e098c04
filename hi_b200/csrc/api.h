// C entry points of libhi_b200_kernels.so. Every function enqueues work on `stream` and
// returns 0, a cudaError_t, or one of the HB_ERR_* codes of common.cuh; none of them
// synchronises. dtype codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int hb_feed_tokens(int* tokens, const int* dst, const int* src, const int* sampled, int n, cudaStream_t stream);
int hb_embed_gather(const void* table, int table_dtype, const int* tokens, float* out, int n, int hidden,
                    int vocab, float scale, cudaStream_t stream);
// routed_weight (or null): [n * top_k] factors of the routed rows in the sum (a score that scales the
// experts' outputs). The sum takes x_scale * x; post != 0: the stream takes the normalised row, not the sum.
int hb_add_rmsnorm(float* x, const void* delta, int delta_dtype, const void* delta2, int delta2_dtype,
                   const float* routed, const int* slot_of_entry,
                   const float* routed_weight, int top_k, const void* w, int w_dtype, void* y, int y_dtype, float* y_f32, const int* row_map,
                   int rows, int hidden, float eps, float x_scale, int post, cudaStream_t stream);
int hb_swiglu(const void* in, void* out, int dtype, int rows, int inter, cudaStream_t stream);
int hb_relu2(const void* in, int dtype, void* out, int out_dtype, long long n, cudaStream_t stream);   // max(x, 0)^2
int hb_convert(const void* in, int dtype, void* out, int out_dtype, long long n, cudaStream_t stream);  // a copy in another dtype
int hb_softcap(float* x, float cap, long long n, cudaStream_t stream);                     // cap tanh(x / cap), in place
int hb_moe_combine(const float* y, const int* slot_of_entry, const float* routed_weight, const void* shared,
                   int shared_dtype, float* out,
                   int n, int hidden, int top_k, cudaStream_t stream);

// q_norm_w / k_norm_w (float32 [hd] or null), norm_first, norm_dim (<= hd; 0: hd), rot_mul: an RMS norm of q and
// k with a weight per dim, over the first norm_dim dims of a head, before the rotation (else: the weightless
// norm after it), and a factor on cos and sin; what the lane-per-16-dims kernel cannot take runs in a general one
int hb_qkv_post(const void* qkv, int dtype, const float* inv_freq, int rot_pairs, int interleaved, int qk_norm,
                float qk_eps, int temp_on, float floor_scale, float attn_scale, const float* q_norm_w,
                const float* k_norm_w, int norm_first, int norm_dim, float rot_mul, const float* v_inv_freq,
                int v_pairs, int v_interleaved, const int* positions,
                const int* seq_of_token, const int* block_table, int table_stride, void* q_out, void* k_pages,
                void* v_pages, int page_size, int write_kv, int n_tokens, int nh, int nkv, int hd,
                cudaStream_t stream);

// sink != 0 (every attention entry point): the softmax's denominator has one more term of score 0,
// p_j = e^{s_j} / (1 + sum e^{s_j}); the term has no value. The general kernel and the merge also take
// sink_values (float32 [nh] or null): the term's score is the head's own number instead of 0. The general
// kernel takes softcap (> 0: s <- softcap tanh(s / softcap) after the scale) and slopes (float32 [nh] or null:
// slopes[h] * (query position - key position) is taken off the score after the cap).
int hb_paged_attention(const void* q, int dtype, const void* k_pages, const void* v_pages,
                       const int* block_table, int table_stride, const int* seq_of_token, const int* positions,
                       void* out, int n_tokens, int nh, int nkv, int hd, int page_size, int chunk, int window,
                       float scale, int sink, float softcap, const float* slopes, const float* sink_values,
                       int split_size, int max_splits, float* part_acc, float* part_ml, cudaStream_t stream);

int hb_attention_merge(const float* part_acc, const float* part_ml, void* out, int dtype, int n_rows, int hd,
                       int max_splits, int sink, int nh, const float* sink_values, cudaStream_t stream);
int hb_attention_decode(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                        int table_stride, const int* seq_of_token, const int* positions, void* out, int n_tokens,
                        int nh, int nkv, int hd, int page_size, int chunk, int window, float scale, int sink,
                        const float* head_bias, float softcap, const float* slopes, const float* sink_values,
                        int split_size, int max_splits, float* part_acc, float* part_ml,
                        cudaStream_t stream);   // sink == 2: sigmoid weights with head_bias; plain sums go to part_acc
                                                // softcap, slopes, sink_values: as hb_paged_attention

int hb_attention_decode_tma(const void* q, const void* k_pages, const void* v_pages, int n_pages, const int* block_table,
                            int table_stride, const int* seq_of_token, const int* positions, void* out, int n_tokens,
                            int nh, int nkv, int hd, int page_size, int chunk, int window, float scale, int sink,
                            int split_size, int max_splits, float* part_acc, float* part_ml, int* status,
                            cudaStream_t stream);

// hb_qkv_post, hb_attention_decode_tma and hb_attention_merge in one launch (attention_decode_tma.cu)
int hb_attention_decode_fused(const void* qkv, const float* inv_freq, int rot_pairs, int interleaved, int qk_norm,
                              float qk_eps, int temp_on, float floor_scale, float attn_scale, void* k_pages,
                              void* v_pages, int n_pages, const int* block_table, int table_stride,
                              const int* seq_of_token, const int* positions, void* out, int n_tokens, int nh, int nkv,
                              int hd, int page_size, int chunk, int window, float scale, int split_size,
                              int max_splits, float* part_acc, float* part_ml, int* counters, int* status,
                              const float* q_norm_w, const float* k_norm_w, int norm_first, float rot_mul, int sink,
                              cudaStream_t stream);

// hb_attention_prefill with reshaped scores: softcap, slopes, sink_values as hb_paged_attention
int hb_attention_prefill_reshaped(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                  int table_stride, const int* cu_seqlens, const int* positions, void* out, int n_seqs,
                                  int max_new, int nh, int nkv, int hd, int page_size, int chunk, int window, float scale,
                                  int skip_single, int sink, float softcap, const float* slopes, const float* sink_values,
                                  cudaStream_t stream);
int hb_attention_prefill(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                         int table_stride, const int* cu_seqlens, const int* positions, void* out, int n_seqs,
                         int max_new, int nh, int nkv, int hd, int page_size, int chunk, int window, float scale,
                         int skip_single, int sink, cudaStream_t stream);

// hb_attention_prefill_tc with reshaped scores: softcap, slopes, sink_values as hb_paged_attention
int hb_attention_prefill_tc_reshaped(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                     int table_stride, const int* cu_seqlens, const int* positions, void* out,
                                     int n_tokens, int n_pages, int n_seqs, int max_new, int nh, int nkv, int hd,
                                     int page_size, int chunk, int window, float scale, int skip_single, int sink,
                                     float softcap, const float* slopes, const float* sink_values, int key_splits,
                                     float* part_acc, float* part_ml, int* status, cudaStream_t stream);
int hb_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                            int table_stride, const int* cu_seqlens, const int* positions, void* out, int n_tokens,
                            int n_pages, int n_seqs, int max_new, int nh, int nkv, int hd, int page_size, int chunk,
                            int window, float scale, int skip_single, int sink, const float* head_bias, int key_splits,
                            float* part_acc, float* part_ml, int* status, cudaStream_t stream);   // sink == 2 as above
// sigmoid weights, one block per (query tile, head) over all its keys: the block turns its rows back by their
// positions (values cached rotated: v_inv_freq [v_pairs] or null) and writes `out` (bfloat16) itself
int hb_sigmoid_prefill_tc(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                          int table_stride, const int* cu_seqlens, const int* positions, void* out, int n_tokens,
                          int n_pages, int n_seqs, int max_new, int nh, int nkv, int hd, int page_size, int chunk,
                          int window, float scale, int skip_single, const float* head_bias, const float* v_inv_freq,
                          int v_pairs, int v_interleaved, int* status, cudaStream_t stream);

// mode: bit 0 = scores are the softmax over all experts (clear: the sigmoid of the chosen logit),
// bit 1 = the chosen scores are divided by their sum; bits 8-15 = G, 16-23 = KEEP: only experts of the KEEP best
// of G equal groups of neighbours can be chosen (a group counts as the sum of its two largest sigmoid scores)
int hb_router_topk(const void* x, int x_dtype, const void* w, int w_dtype, int n, int hidden, int experts,
                   int top_k, int mode, float score_scale, float* logits_out, int* ids, float* scores,
                   cudaStream_t stream);    // score_scale: a constant factor on every chosen score
int hb_moe_plan(const int* ids, int n_entries, int experts, int* offsets, int* sorted_entry,
                int* slot_of_entry, int* active, cudaStream_t stream);
int hb_router_plan(const void* x, int x_dtype, const void* w, int w_dtype, int n, int hidden, int experts, int top_k,
                   int mode, float score_scale, float* logits_out, int* ids, float* scores, int* offsets,
                   int* sorted_entry, int* slot_of_entry, int* active, int* counter, cudaStream_t stream);
int hb_moe_gate_up(const void* x, int dtype, const int* sorted_entry, int top_k, const void* w_gate,
                   const void* w_up, const int* offsets, const int* active, int experts, const float* scores,
                   void* act, int n_entries, int inter, int hidden, int few_rows, int activation, cudaStream_t stream);
int hb_moe_down(const void* act, int dtype, const void* w_down, const int* offsets, const int* active, int experts,
                float* y, int n_entries, int hidden, int inter, int few_rows, cudaStream_t stream);

int hb_gather_rows(const void* x, const int* sorted_entry, int top_k, void* xs, int rows, int hidden,
                   cudaStream_t stream);
int hb_moe_gate_up_tc(const void* xs, const int* sorted_entry, const void* w_gate, const void* w_up,
                      const int* offsets, int experts, const float* scores, void* act, int rows, int inter,
                      int hidden, int* status, cudaStream_t stream);
int hb_moe_down_tc(const void* act, const void* w_down, const int* offsets, int experts, float* y, int rows,
                   int hidden, int inter, float* scratch, long long scratch_floats, int* counters, int n_counters,
                   int* status, cudaStream_t stream);
long long hb_moe_down_tc_scratch_floats(int sms);
int hb_moe_up_relu2_tc(const void* xs, const void* w_up, const int* offsets, int experts, void* act, int rows, int inter,
                       int hidden, int* status, cudaStream_t stream);     // act = bfloat16 max(xs W_up^T, 0)^2

int hb_sample_rows(const float* logits, int rows, int vocab, const float* temperatures, const float* uniforms,
                   int* out, cudaStream_t stream);
int hb_sample_rows_parts(const float* logits, int rows, int vocab, int parts, const float* temperatures,
                         const float* uniforms, float* part_val, int* part_idx, float* part_max, float* part_sum,
                         int* counters, int* out, cudaStream_t stream);
int hb_ranked_rows(const float* logits, int rows, int vocab, const float* temperatures, const float* top_ps,
                   const int* top_ks, const float* uniforms, int* out, cudaStream_t stream);
int hb_argmax_rows(const float* logits, int rows, int vocab, int parts, float* part_val, int* part_idx, int* counters,
                   int* out, cudaStream_t stream);

// gated_block.cu: gated sum of two sub-layer results into the stream, the weighted average of all layer
// results so far, and up to two Dynamic Tanh norms of it, in one pass; the xIELU activation
int hb_gated_depth_dyt(const float* x, const void* delta0, int delta0_dtype, const void* gate0, int gate0_dtype,
                       const void* delta1, int delta1_dtype, const void* gate1, int gate1_dtype, float* hist,
                       long long hist_stride, int n_prev, const float* mix, float* z_out, const float* alpha0,
                       const void* w0, const void* b0, void* y0, const float* alpha1, const void* w1, const void* b1,
                       void* y1, int wb_dtype, int y_dtype, const int* row_map, int rows, int width,
                       cudaStream_t stream);
int hb_xielu(const void* in, void* out, int dtype, const float* coef, long long n, cudaStream_t stream);

// latent.cu: RMS-normed latent rows into their pages; a sigmoid gate per (token, head)
int hb_latent_append(const void* in, int dtype, long long in_stride, const void* w, float eps, const int* positions,
                     const int* seq_of_token, const int* block_table, int table_stride, void* pages, int page_size,
                     int rank, int row_len, int n_tokens, const float* inv_freq, int rot_pairs, int interleaved,
                     float rot_mul, cudaStream_t stream);   // rot_mul: a factor on cos and sin
int hb_rope_copy(const void* src, long long src_row, long long src_head, void* dst, long long dst_row,
                 long long dst_head, int dtype, const int* positions, const float* inv_freq, int n_tokens, int heads,
                 int pairs, int interleaved, float rot_mul, cudaStream_t stream);
int hb_rmsnorm_rows(const void* in, int dtype, long long in_stride, const void* w, float eps, void* out, int n_rows,
                    int width, cudaStream_t stream);
int hb_head_gate(const void* in, const void* gate, long long gate_stride, void* out, int dtype, int n_tokens,
                 int heads, int dim, cudaStream_t stream);

// delta_rule.cu: the gated delta rule with a decay per head and key channel
int hb_delta_prep(const void* proj, int proj_dtype, long long ld, int chan_off, int beta_off, const float* taps,
                  float* state, long long state_stride, long long conv_off, const void* a_pre, int a_dtype,
                  const float* dt_bias, const float* a_log, const int* cu_seqlens, const int* seq_of_token,
                  const int* slots, float* q, float* k, float* v, float* beta, float* decay, int n_tokens, int heads,
                  int kvh, int dim, int vdim, int taps_n, int head_decay, cudaStream_t stream);
int hb_gla_prep(const void* proj, int proj_dtype, long long ld, int q_off, int k_off, int v_off, const float* z,
                const float* bias, float tau, float q_scale, float* q, float* k, float* v, float* decay, int n_tokens,
                int qk_cols, int v_cols, cudaStream_t stream);
int hb_delta_conv_update(const void* proj, int proj_dtype, long long ld, int chan_off, float* state,
                         long long state_stride, long long conv_off, const int* cu_seqlens, const int* slots,
                         int n_seqs, int channels, int taps_n, cudaStream_t stream);
int hb_delta_recurrence(const float* q, const float* k, const float* v, const float* beta, const float* decay,
                        float* state, long long state_stride, const int* cu_seqlens, const int* slots, float* out,
                        int n_seqs, int heads, int kvh, int dim, int vdim, int variant, int single_tokens, int plain,
                        cudaStream_t stream);   // variant: 0 chosen by sizes, 1 S in shared memory, 16 / 32 rows a lane
int hb_delta_out_norm(const float* o, const void* gate, int gate_dtype, const void* w, float eps, void* out, int dtype,
                      long long rows, int vdim, int gate_silu, long long gate_stride, int heads, cudaStream_t stream);

// mlstm.cu: the matrix memory of the mLSTM (gates and running maximum; S and n token after token; output norm).
// A request's state row: [heads][vdim + 1][dim] float32 (S column by column, then n), then m [heads] at m_off.
int hb_mlstm_gates(const float* z, const float* bias_i, const float* bias_f, float cap, float* state,
                   long long state_stride, long long m_off, const int* cu_seqlens, const int* slots, float* keep,
                   float* take, float* floor_, int n_seqs, int heads, cudaStream_t stream);
int hb_mlstm_recurrence(const void* proj, int proj_dtype, long long ld, int q_off, int k_off, int v_off, float q_scale,
                        const float* keep, const float* take, float* state, long long state_stride,
                        const int* cu_seqlens, const int* slots, float* o, float* nq, int n_seqs, int heads, int dim,
                        int vdim, int rows_per_lane, cudaStream_t stream);
int hb_mlstm_out_norm(const float* o, const float* nq, const float* floor_, const void* proj, int proj_dtype,
                      long long ld, int g_off, const void* w, int w_dtype, float eps, void* out, int out_dtype,
                      long long n_tokens, int heads, int vdim, cudaStream_t stream);

// seeded random weights: out[i] = value of element first + i of the tensor with `key` (random_fill.cu)
int hb_random_normal(void* out, int dtype, long long n, long long first, unsigned long long key, float scale,
                     cudaStream_t stream);

// canon.cu: the norm's output through a short causal convolution over time per channel, kept float32 between the
// two; what is added to the stream between passes over a range of layers; the mean of two normed mixer outputs.
// update_state: 0 the state stays, 1 a second launch stores the portions' last rows, 2 every request brings exactly
// one row and the convolution kernel moves its state itself
int hb_canon_conv(const float* h, const float* taps_a, const float* taps_b, float* state, long long state_stride,
                  const int* cu_seqlens, const int* seq_of_token, const int* slots, void* out_a, void* out_b, int dtype,
                  int n_tokens, int n_seqs, int width, int taps_n, int update_state, cudaStream_t stream);
int hb_stream_add(float* x, const void* d1, int d1_dtype, const void* d2, int d2_dtype, const float* e,
                  const float* vec, long long rows, int width, cudaStream_t stream);
int hb_rmsnorm_mean2(const void* a, const void* b, int in_dtype, const void* wa, const void* wb, int w_dtype, float eps,
                     void* out, int out_dtype, int rows, int width, cudaStream_t stream);

// sigmoid_attention.cu: weights sigmoid(score + bias[head]), not normalised; values cached rotated and the sum
// turned back (v_inv_freq null: values as they are)
int hb_sigmoid_attention(const void* q, int dtype, const void* k_pages, const void* v_pages, const int* block_table,
                         int table_stride, const int* seq_of_token, const int* positions, const float* head_bias,
                         const float* v_inv_freq, int v_pairs, int v_interleaved, void* out, int n_tokens, int nh,
                         int nkv, int hd, int page_size, int chunk, int window, float scale, int split_size,
                         int max_splits, float* part_acc, cudaStream_t stream);

// the splits of every (token, head) of part_acc [n_tokens * nh][max_splits][hd] added in split order and turned back
int hb_sigmoid_merge(const float* part_acc, const int* positions, const float* v_inv_freq, int v_pairs,
                     int v_interleaved, void* out, int dtype, int n_tokens, int nh, int hd, int max_splits,
                     cudaStream_t stream);

// hyper.cu: a residual stream of n_streams copies per token (float32 [N, S, W]). One launch per sub-layer boundary:
// the result the sub-layer before left (delta, delta2, routed rows) goes into every copy with out_coef * mult while
// the copies are mixed by mix [from, to] (null: the copies stay), then u = sum_s in_coef[s] x_s (null: ones) is RMS
// normed with w into y (and y_f32). x_in: the copies do not exist yet and all equal x_in's row. row_map: only those
// rows, nothing written back.
int hb_hyper_step(float* streams, const float* x_in, const void* delta, int delta_dtype, const void* delta2,
                  int delta2_dtype, const float* routed, const int* slot_of_entry, const float* routed_weight, int top_k,
                  const float* mix, const float* out_coef, float mult, const float* in_coef, const void* w, int w_dtype,
                  float eps, void* y, int y_dtype, float* y_f32, const int* row_map, int rows, int n_streams, int width,
                  cudaStream_t stream);
int hb_hyper_sum(const float* streams, float* out, int rows, int n_streams, int width, cudaStream_t stream);

// mamba2.cu: what surrounds the Mamba-2 recurrence (which is hb_delta_recurrence without its correction term)
int hb_mamba2_prep(const void* proj, int proj_dtype, long long ld, int chan_off, int dt_off, const float* taps,
                   const float* conv_bias, const float* state, long long state_stride, long long conv_off,
                   const float* dt_bias, const float* a_log, const int* cu_seqlens, const int* seq_of_token,
                   const int* slots, float* x, float* v, float* k, float* q, float* decay, int n_tokens, int heads,
                   int groups, int n_state, int vdim, int taps_n, cudaStream_t stream);
int hb_mamba2_out(const float* o, const float* x, const void* z, int z_dtype, long long z_stride, const float* d_skip,
                  const void* w, float eps, void* out, int dtype, int n_tokens, int heads, int vdim, int parts,
                  cudaStream_t stream);

#ifdef __cplusplus
}
#endif
