// C entry points of the kernel library (libferrox_b200.so).  Every function
// enqueues work on `stream` (a cudaStream_t passed as void*) and returns 0, a
// cudaError_t (> 0) from the launch, or one of the negative FX_ERR_* codes of
// common.cuh when it refuses its arguments.  Nothing here allocates or synchronises.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int fx_gemm(const void* A, int a_dtype, long lda, const int* a_rows, const void* W, int w_dtype, long ldw,
            const void* bias, int bias_dtype, void* C, int c_dtype, long ldc, int accumulate, int M, int N, int K,
            const int* group_offsets, int n_groups, long w_group_stride, void* stream);

// Streaming multiprocessors of the current device (asked once).
int fx_sm_count();

// Programmatic dependent launch of the short kernels on (1, default) or off (0); returns the old setting.
int fx_set_pdl(int on);

int fx_embed(const void* table, int dtype, const int* ids, float* out, int n_tokens, int hidden, int vocab,
             int* status, float scale, void* stream);    // out[t] = table[ids[t]] * scale
// h[r] += scale * y[r] and, with a weight w, x_out[r] = rmsnorm(h[r]) * w on the new rows (elementwise.cu)
int fx_scaled_add_norm(float* h, const float* y, float scale, const void* w, int w_dtype, float eps, void* x_out,
                       int x_dtype, int n_rows, int hidden, void* stream);
int fx_rmsnorm(const float* x, const int* rows, const void* w, int w_dtype, float eps, void* out, int out_dtype,
               int n_rows, int hidden, void* stream);
int fx_silu_mul(const void* gu, long ld_in, void* out, long ld_out, int dtype, const int* n_rows_dev, int rows, int n,
                void* stream);
int fx_glu_mul(const void* gu, long ld_in, void* out, long ld_out, int dtype, const int* n_rows_dev, int rows, int n,
               int act, float act_limit, float act_alpha, void* stream);   // act 0: SiLU(gate) * up, 1: ReLU(gate) * up,
                                                                          // 2: the clamped unit (fx_clamped_glu)
int fx_rope_kv_write(void* qkv, int dtype, long ld, const int* positions, const int* token_seq, const int* seq_slot,
                     const float* inv_freq, const float* cos_sin, int rotary_dim, int pairing, void* k_pages, void* v_pages, const int* block_table,
                     int table_width, int page_size, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                     int write_cache, int* status, void* stream);
int fx_moe_combine(float* h, const void* y, int dtype, const int* inv_perm, const float* topk_w, int top_k,
                   const void* shared, const float* shared_gate_logit, long gate_ld, int n_tokens, int hidden,
                   void* stream);
int fx_residual_add(float* h, const void* y, int dtype, long n, void* stream);

int fx_paged_attention(const void* q, long ldq, const void* k_pages, const void* v_pages, int dtype,
                       const int* block_table, int table_width, int page_size, const int* positions,
                       const int* token_seq, const int* seq_slot, void* out, long ldo, int n_tokens, int n_heads,
                       int n_kv_heads, int head_dim, int window, float scale, float softcap, void* stream);

// fx_paged_attention with keys and values of different widths and strides, strided queries and outputs, and an
// optional distance bias slopes[h] * (i - j) taken off the scores (attention_generic.cu)
int fx_paged_attention_ex(const void* q, long ldq, long ldqh, const void* k_pages, const void* v_pages, long ldk, long ldv,
                          int dtype, const int* block_table, int table_width, int page_size, const int* positions,
                          const int* token_seq, const int* seq_slot, void* out, long ldo, long ldoh, int n_tokens,
                          int n_heads, int n_kv_heads, int key_dim, int value_dim, int window, float scale, float softcap,
                          const float* slopes, int keep_first, const float* sinks, int value_share, void* stream);
// sinks (optional, one per head): exp(sinks[h]) joins the softmax's denominator once.  value_share >= 1: that many
// consecutive key heads read one value head (the value pages hold n_kv_heads / value_share heads).

// the same operation in bfloat16 on the tensor cores (attention_general_mma.cu); items: int32 [n_items, 5] = (first flat
// token, tokens, entry, first query head, heads) or nullptr (one token a tile, n_items = tokens)
int fx_general_attention_ok(int key_dim, int value_dim, int alias);
int fx_general_attention(const void* q, long ldq, long ldqh, const void* k_pages, const void* v_pages, long ldk, long ldv,
                         const long* kv_strides, const int* block_table, int table_width, int page_size, const int* positions,
                         const int* token_seq, const int* seq_slot, const int* items, int n_items, void* out, long ldo,
                         long ldoh, int n_heads, int n_kv_heads, int key_dim, int value_dim, int window, float scale,
                         const float* slopes, int n_splits, float* part_o, float* part_ml, int keep_first, float softcap,
                         const float* sinks, int value_share, void* stream);

int fx_prefill_attention_tc(const void* q, long ldq, int n_tokens, const void* k_pages, const void* v_pages, int n_pages,
                            const int* block_table, int table_width, int page_size, const int* items, int n_items,
                            const int* seq_slot, void* out, long ldo, int n_heads, int n_kv_heads, int head_dim,
                            int window, float scale, int* status, float* part_o, float* part_ml, const int* merges,
                            int n_merges, void* stream);
int fx_prefill_attention(const void* q, long ldq, const void* k_pages, const void* v_pages, const int* block_table,
                         int table_width, int page_size, const int* tiles, int n_tiles, const int* seq_slot, void* out,
                         long ldo, int n_heads, int n_kv_heads, int head_dim, int window, float scale, float softcap,
                         void* stream);

// Routing extras (the last three arguments before the stream of the four routing entry points): choice_bias, one
// number per expert added to sigmoid(logit) for the choice only (mode bit 1; nullptr: none); weight_scale, a factor on
// the final weights; renorm_eps, added to the sum the kept scores are divided by (mode bit 0).
int fx_router_topk(const float* logits, long ld, int n_tokens, int n_experts, int top_k, int renorm, int* ids,
                   float* weights, const float* choice_bias, float weight_scale, float renorm_eps, void* stream);
int fx_moe_align(const int* ids, int n_tokens, int top_k, int n_experts, int* scratch, int* offsets, int* src_token,
                 int* inv_perm, int* active, int n_slots, void* stream);

// The four product kernels below, gated form with a bias: `bias` holds the gate rows' values at [0, N) and the up
// rows' at [gate_up_offset, gate_up_offset + N): C = act(gate + b_gate) * (up + b_up).
int fx_gemm_tc(const void* X, long ldx, const void* W, long ldw, long w_group_stride, int w_rows, const void* bias,
               int bias_dtype, void* C, int c_dtype, long ldc, int accumulate, int M, int N, int K, int gated,
               int gate_up_offset, float act_limit, float act_alpha, const int* group_offsets, int n_groups, int* status,
               void* stream);
int fx_gemm_tc_swap(const void* X, long ldx, const void* W, long ldw, long w_group_stride, int w_rows, const void* bias,
                    int bias_dtype, void* C, int c_dtype, long ldc, int accumulate, int M, int N, int K, int gated,
                    int gate_up_offset, float act_limit, float act_alpha, const int* group_offsets, int n_groups, int tokens_per_tile, int weights_first,
                    int k_splits, float* partials, int* status, void* stream);
int fx_gemm_tc2(const void* X, long ldx, const void* W, long ldw, int w_rows, const void* bias, int bias_dtype, void* C,
                int c_dtype, long ldc, int accumulate, int M, int N, int K, int gated, int gate_up_offset, float act_limit,
                float act_alpha, int* status, void* stream);
int fx_moe_combine_norm(float* h, const void* y, int dtype, const int* inv_perm, const float* topk_w, int top_k,
                        const void* shared, const float* shared_gate_logit, long gate_ld, int n_tokens, int hidden,
                        const void* norm_w, int norm_w_dtype, float eps, void* x_out, void* stream);
int fx_gather_rows(const void* x, long ldx, const int* rows, void* out, long ldo, int dtype, int n_rows, int width,
                   void* stream);
// out[r] = w * x[rows[r]], w the routing weight of the (token, rank) pair in place r of the expert order
int fx_gather_rows_scaled(const void* x, long ldx, const int* rows, const int* inv_perm, const float* weights, int top_k,
                          void* out, long ldo, int dtype, int n_rows, int width, void* stream);
int fx_route(const float* logits, long ld, int n_tokens, int n_experts, int top_k, int renorm, int* ids, float* weights,
             int* scratch, int* offsets, int* src_token, int* inv_perm, int* active, int n_slots,
             const float* choice_bias, float weight_scale, float renorm_eps, void* stream);
int fx_route_small(const float* logits, long ld, int n_tokens, int n_experts, int top_k, int renorm, int* ids, float* weights,
                   int* offsets, int* src_token, int* inv_perm, int* active, int n_slots, const float* choice_bias,
                   float weight_scale, float renorm_eps, void* stream);
int fx_route_fused(const void* X, long ldx, const void* W, long ldw, int n_tokens, int n_route, int n_experts, int hidden,
                   int top_k, int renorm, float* logits, long ldl, int* ids, float* weights, int* offsets, int* src_token,
                   int* inv_perm, int* active, int n_slots, void* xp_out, long ldxp, const float* choice_bias,
                   float weight_scale, float renorm_eps, void* stream);
int fx_rope_table(const int* positions, const float* inv_freq, int n_tokens, int half, float* cos_sin, float magnitude,
                  void* stream);   // cos and sin times `magnitude`
// A few tokens against a plain matrix that fits the shared memory of all SMs together (gemm_slab.cu): every block asks
// for its whole slab of W before it waits for the kernel before it on the stream, which therefore must not have written W.
// C[t, n] (+)= sum_k X[t, k] W[n, k] (+ bias[n]); bfloat16 X and W, K a multiple of 128, C bfloat16 or float32.
int fx_gemm_slab_ok(int N, int K, int n_tokens);
int fx_gemm_slab(const void* X, long ldx, const void* W, long ldw, const void* bias, int bias_dtype, void* C,
                 int c_dtype, long ldc, int accumulate, int n_tokens, int N, int K, int* status, void* stream);

int fx_gemm_skinny(const void* X, long ldx, const int* x_rows, const void* W, long ldw, long w_group_stride,
                   const void* bias, int bias_dtype, void* C, int c_dtype, long ldc, int accumulate, int n_tokens,
                   int N, int K, int gated, int gate_up_offset, float act_limit, float act_alpha, const int* group_offsets,
                   const int* active_groups,
                   int n_slots, int tokens_hint, int c_transposed, void* stream);
int fx_decode_split_mma(const void* q, long ldq, const void* k_pages, const void* v_pages, const int* block_table,
                        int table_width, int page_size, const int* positions, const int* token_seq, const int* seq_slot,
                        float* part_acc, float* part_ml, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                        int window, float scale, int split_len, int n_splits, int fresh_positions, float softcap,
                        void* stream);
int fx_decode_split_tma(const void* q, long ldq, const void* k_pages, const void* v_pages, int n_pages,
                        const int* block_table, int table_width, int page_size, const int* positions,
                        const int* token_seq, const int* seq_slot, float* part_acc, float* part_ml, int n_tokens,
                        int n_heads, int n_kv_heads, int head_dim, int window, float scale, int split_len,
                        int n_splits, int* status, void* out, long ldo, int* counters, int fresh_positions,
                        int store_new, int write_pages, const float* cos_sin, void* stream);
// n_pages > 0 (the number of pages behind k_pages / v_pages) lets bfloat16 take the TMA kernel; status: the step's
// status word (may be null).
// fresh_positions: 0 makes no assumption about the kernel launched before this one on the stream: nothing is read until
// it has finished.  N > 0 is the caller's promise that that kernel wrote, of everything this call reads, only the
// queries and the keys and values of at most the last N positions of each request (positions, token_seq, seq_slot and
// the block table are older); the bfloat16 kernels then fetch tiles of older keys while that kernel still runs.  A
// promise that does not hold gives stale keys without any error.
// store_new = 1 (bfloat16, head sizes in steps of 64, pages of a multiple of 64 positions, one token a request; else
// refused): `q` is the step's fused [q | k | v] rows as projected, and the kernel does the rotary kernel's work
// itself: it rotates the queries (split-half pairs over the whole head; cos_sin [tokens][head_dim / 2][2] from
// fx_rope_table, or null for no rotation), and rotates and stores each token's own key and value (into the pages only
// if write_pages).  The kernel before it must then not write the pages at all.
int fx_decode_attention(const void* q, long ldq, const void* k_pages, const void* v_pages, int n_pages, int dtype,
                        const int* block_table, int table_width, int page_size, const int* positions,
                        const int* token_seq, const int* seq_slot, void* out, long ldo, float* part_acc,
                        float* part_ml, int n_tokens, int n_heads, int n_kv_heads, int head_dim, int window,
                        float scale, int split_len, int n_splits, int* status, int* counters, int fresh_positions,
                        int store_new, int write_pages, const float* cos_sin, float softcap, void* stream);
// attention_prep.cu: what mixers with normed queries and keys, a query temperature, keys and values of different
// widths, or a latent cache do between their projections and the attention kernel
int fx_qk_norm_store(void* qkv, int dtype, long ld, const int* positions, const int* token_seq, const int* seq_slot,
                     const void* wq, const void* wk, int w_dtype, float eps, float temp_coef, int temp_every, void* k_pages,
                     void* v_pages, const int* block_table, int table_width, int page_size, int n_tokens, int n_heads,
                     int n_kv_heads, int key_dim, int value_dim, int write_cache, int* status, float v_eps, void* stream);
int fx_latent_prep(void* q, long ldq, const void* dkv, long ld_dkv, int dtype, const int* positions,
                   const int* token_seq, const int* seq_slot, const void* wc, int w_dtype, float eps, const float* cos_sin,
                   int rot_dims, void* q_plain, void* q_full, void* pages, const int* block_table, int table_width,
                   int page_size, int n_tokens, int n_heads, int plain_dim, int rot_dim, int rank, int write_cache,
                   int* status, int pairing, void* stream);   // q_plain == nullptr: q's rotated parts are turned where they
                                                              // lie; pairing 1: neighbours, 0: halves
int fx_rmsnorm_rows(const void* x, int x_dtype, long ldx, const void* w, int w_dtype, float eps, void* out, int out_dtype,
                    long ldo, int n_rows, int n, void* stream);
int fx_heads_to_tokens(const void* in, long in_ldt, long in_ldh, const void* gate, long ldg, void* out, long ldo, int dtype,
                       int n_tokens, int n_heads, int width, int gate_per_head, void* stream);

// softcap c > 0 (fx_paged_attention, fx_prefill_attention, fx_decode_attention): the scaled scores pass through
// c * tanh(s / c) before the softmax; 0: none.  The kernels that stream pages by TMA take no cap: fx_decode_attention
// goes to the others, and callers do not give a capped layer to fx_prefill_attention_tc.

// out[i] = mean + stdev * z_i, z the standard normal stream of `key` (random_init.cu; the host restates the rule
// bit for bit).  dtype: FX_F32 or FX_BF16.
int fx_random_normal(void* out, int dtype, long n, unsigned long long key, double mean, double stdev, void* stream);

int fx_argmax(const float* logits, long ld, int n_rows, int vocab, int* out, void* stream);
int fx_sample_or(const float* scores, long lds, float* work, long ld, int n_rows, int vocab, const float* temperature,
                 const int* top_k, const float* top_p, const float* draw, const int* use_sample, const int* instead,
                 int* out, void* stream);
int fx_repetition_penalty(float* work, long ld, int n_rows, int vocab, const int* history, const int* hist_offsets,
                          const float* penalty, void* stream);
int fx_sample(float* work, long ld, int n_rows, int vocab, const float* temperature, const int* top_k,
              const float* top_p, const float* draw, int* out, void* stream);

// Layer norm without bias (layernorm.cu): out = (x - mean) / sqrt(var + eps) * w over rows of the 32-bit residual
// stream (`rows` optional: which rows; out may be x itself).  fx_layernorm_residual: z = s1 y1 (+ s2 y2);
// h += ln(z) w_post; and, if w_next is given, x_out = ln(h) w_next on the new rows.  fx_scale: x *= scale.
int fx_layernorm(const float* x, const int* rows, const void* w, int w_dtype, const void* bias, int b_dtype, float eps,
                 void* out, int out_dtype, int n_rows, int hidden, void* stream);
int fx_layernorm_residual(float* h, const void* y1, int y1_dtype, float s1, const void* y2, int y2_dtype, float s2,
                          const void* w_post, int wp_dtype, float eps, const void* w_next, int wn_dtype, float eps_next,
                          void* x_out, int x_dtype, int n_rows, int hidden, void* stream);
int fx_scale(float* x, long n, float scale, void* stream);

// Mixers with a matrix state per (request, head) (linear_state.cu).  The state is [slots, H, V, D] 32-bit.
int fx_delta_prep(const void* proj, int dtype, long ldp, const void* conv_w, int cw_dtype, int taps, const float* tail,
                  const float* ba, long ldba, const float* a_log, const float* dt_bias, const int* token_seq,
                  const int* seq_slot, float* out, float* beta, float* g, int n_tokens, int G, int D, int H, int V,
                  int update_tail, void* stream);
// update_tail = 1: the caller's promise that every entry of the step brings exactly one token; the kernel then moves
// the convolution's tail on itself and fx_conv_tail_update is not needed.
int fx_conv_tail_update(const void* proj, int dtype, long ldp, int channels, int taps, float* tail, const int* token_seq,
                        const int* seq_slot, int n_tokens, int n_entries, void* stream);
int fx_state_scan(const void* q, long ldq, const void* k, long ldk, const void* v, long ldv, int dtype, int act,
                  const float* g, long g_ld, const float* beta, float* state, float* out, long ldo, const int* token_seq,
                  const int* seq_slot, int n_tokens, int n_entries, int H, int G, int D, int V, void* stream);
int fx_set_scan_lanes(int lanes);   // lanes that share a state column, fixed for measurements (0: the launcher's choice)
int fx_gated_group_norm(const float* x, const void* gate, int gate_dtype, long ldg, const void* w, int w_dtype, float eps,
                        int act, void* out, int out_dtype, int n_tokens, int groups, int width, long w_stride,
                        void* stream);

// The generalized delta rule (general_delta.cu).  fx_general_delta_prep: per (token, head) the unit key
// u = k / sqrt(sum k^2 + 1e-6), a u with a = sigmoid(a_pre + a_bias), and the decay
// w = exp(-rate * sigmoid(w2 . tanh(w1_out) + w0)), from 32-bit rows.  fx_general_delta_scan: over every entry's
// tokens in order, S <- diag(w) S - (a u)(u^T S) + k v^T (both terms read the old S), out = S^T r; state
// [slots, H, D(value), D(key)] 32-bit.
int fx_general_delta_prep(const float* k, long ldk, const float* a_pre, long lda, const float* w1_out, long ldw1,
                          const void* w2, int w2_dtype, const void* w0, int w0_dtype, const void* a_bias, int ab_dtype,
                          float rate, float* u, float* au, float* w, int n_tokens, int H, int D, int rank, void* stream);
int fx_general_delta_scan(const float* r, long ldr, const float* k, long ldk, const float* v, long ldv, const float* u,
                          const float* au, const float* w, float* state, float* out, long ldo, const int* token_seq,
                          const int* seq_slot, int n_tokens, int n_entries, int H, int D, void* stream);

// The input convolution of a mixer (input_conv.cu): out[t] = x[t] + sum_j w[:, j] x[t - taps + 1 + j] over the
// tokens of a request, the inputs before the step from tail [slots, taps - 1, channels] (32-bit, oldest first).
// update_tail: every entry brings exactly one token and the kernel moves the tail on itself.
int fx_input_conv(const void* x, int dtype, long ldx, const void* w, int w_dtype, int taps, float* tail,
                  const int* token_seq, const int* seq_slot, void* out, long ldo, int n_tokens, int channels,
                  int update_tail, int add_input, void* stream);   // add_input 0: out[t] = the sum alone
// out[t] = table[ids[t]] + pos_table[positions[t]] in 32 bits; status 1: an id outside the vocabulary, 4: a position
// outside the table.
int fx_embed_pos(const void* table, int dtype, const int* ids, const void* pos_table, int pos_dtype, const int* positions,
                 float* out, int n_tokens, int hidden, int vocab, int n_positions, int* status, void* stream);
// x <- cap * tanh(x / cap), 32-bit, in place.
int fx_softcap(float* x, long n, float cap, void* stream);
// x <- max(x, 0)^2 in place, rows of `n` elements with row stride ld.
int fx_relu_square(void* x, int dtype, long ld, int rows, int n, void* stream);

// The matrix memory of an mLSTM mixer (mlstm.cu): gates capped and taken to the logarithm, a running maximum, the
// state S [slots, H, V, D], a normaliser n [slots, H, Z, D] and the maximum m [slots, H, Z], Z =
// fx_mlstm_column_blocks(D, V) copies of both; q, k [tokens, H*D], v [tokens, H*V] and gates [tokens, >= 2H] (input
// gates, then forget gates, before bias and cap) are 32-bit rows.
int fx_mlstm_column_blocks(int D, int V);
int fx_mlstm_scan(const float* q, long ldq, const float* k, long ldk, const float* v, long ldv, const float* gates,
                  long ldg, const void* i_bias, const void* f_bias, int bias_dtype, float cap, float q_scale, float* S,
                  float* n, float* m, float* out, long ldo, const int* token_seq, const int* seq_slot, int n_tokens,
                  int n_entries, int H, int D, int V, int copies, void* stream);   // copies: Z as the state holds it

// diff_attention.cu.  fx_conv_rotary_store: a short causal convolution on every channel of the projected
// [q | k | v] rows (no input added), rotation of the first rot_dims elements of every q and k head by cos_sin
// [tokens][rot_dims / 2][2], q into q_out, k and v into pages of their own head counts and widths.
// fx_diff_combine: out[t, h] = rms(a1 - lambda a2) * post, the two maps of head h = g * group + hg being rows
// (2 g) * group + hg and (2 g + 1) * group + hg of attn.
int fx_conv_rotary_store(const void* proj, int dtype, long ldp, const void* w, int w_dtype, int taps, float* tail,
                         const int* positions, const int* token_seq, const int* seq_slot, const float* cos_sin,
                         int rot_dims, int pairing, void* q_out, long ldq, void* k_pages, void* v_pages,
                         const int* block_table, int table_width, int page_size, int n_tokens, int n_q_heads,
                         int n_k_heads, int head_dim, int n_v_heads, int value_dim, int write_cache, int update_tail,
                         int* status, void* stream);
int fx_diff_combine(const void* attn, long lda, void* out, long ldo, int dtype, int n_tokens, int n_heads, int group,
                    int value_dim, float lambda, float eps, float post, void* stream);

#ifdef __cplusplus
}
#endif
