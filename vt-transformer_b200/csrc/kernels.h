// Launchers of the hand-written kernels.  Plain pointers and sizes; every launcher
// enqueues on `stream` and returns cudaGetLastError().  `status` points at two ints on
// the device (code, detail), see common.cuh; it may be null.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace vtb {

enum DType : int { kF32 = 0, kBF16 = 1 };

// out[t, :] = float(table[ids[t], :]).  hidden % 8 == 0.
cudaError_t launch_embedding(int table_dtype, const void* table, const int* ids, float* out, int n_tokens,
                             int hidden, int vocab, float scale, int* status, cudaStream_t stream);
// logits = cap * tanh(scale * logits / cap) in place; cap 0 applies the scale alone
cudaError_t launch_logits_scale_cap(float* logits, long long n, float scale, float cap, cudaStream_t stream);

// For r in 0..n_rows: t = rows ? rows[r] : r; v = x[t] (+ delta[t], written back to x[t]);
// out[r] = weight * v * rsqrt(mean(v^2) + eps).  x float, weight float, delta/out of out_dtype.  Instead of
// delta: parts [n_parts, n_tokens, hidden] float, the unadded shares of a delta, added in the order of their index.
cudaError_t launch_rmsnorm(int out_dtype, float* x, const void* delta, const float* parts, int n_parts,
                           const float* weight, float eps, void* out, const int* rows, int n_rows, int n_tokens,
                           int hidden, int* status, const float* post_weight, float post_eps, float post_mult, cudaStream_t stream,
                           int groups = 1, float x_scale = 1.f, int write_normed = 0);

// The same with the mean taken off: out[r] = weight * (v - mean(v)) * rsqrt(mean((v - mean(v))^2) + eps).
cudaError_t launch_layernorm(int out_dtype, float* x, const void* delta, const float* parts, int n_parts,
                             const float* weight, float eps, void* out, const int* rows, int n_rows, int n_tokens,
                             int hidden, int* status, const float* post_weight, float post_eps, float post_mult, cudaStream_t stream);

// out[t, :] = a N(z) + b N(z^2) + c N(z^3) + e for every row of z [n_tokens, inter], N(y) = y / sqrt(mean(y^2) + eps),
// (a, b, c, e) = coef[0..3].  out may be z.  inter % 8 == 0; the means are over the first n_mean columns, the rest being
// zero padding.
cudaError_t launch_polynorm(int dtype, const void* z, const float* coef, float eps, void* out, int n_tokens, int inter,
                            int n_mean, cudaStream_t stream);

// Gated linear attention over the tokens of every (sequence, head) in order (recurrent.cu).  y [tokens, stride] holds
// q, k [heads * dim], v [heads * v_dim] and the low-rank gate's input [rank] at the given columns; a2 [heads * dim,
// rank] and a2_bias are float; state [state_rows, heads, dim, v_dim] float is read at rows[sequence] and left as after
// the sequence's last token; out [tokens, heads * v_dim] float.  A sequence without tokens is left alone.  most_threads > 0
// says that the step is a long walk of few sequences: CTAs of 256 threads, a head's column blocks spread over several
// CTAs; it changes no result.
cudaError_t launch_gla_scan(int dtype, const void* y, int stride, int q_col, int k_col, int v_col, int low_col, int rank,
                            const float* a2, const float* a2_bias, float inv_tau, float q_scale, float* state,
                            int state_rows, const int* cu_q, const int* rows, int n_seqs, float* out, int heads, int dim,
                            int v_dim, int most_threads, int* status, cudaStream_t stream);
// The generalized delta rule in the same manner; a_col: the removal rate's projection, low_col: the decay's low-rank
// input (tanh is applied to it), w2 [heads * dim, rank], w0 and a_bias float; state [state_rows, heads, dim, dim].
cudaError_t launch_delta_scan(int dtype, const void* y, int stride, int r_col, int k_col, int v_col, int a_col, int low_col,
                              int rank, const float* w2, const float* w0, const float* a_bias, float decay_rate,
                              float key_eps, float* state, int state_rows, const int* cu_q, const int* rows, int n_seqs,
                              float* out, int heads, int dim, int most_threads, int* status, cudaStream_t stream);
// out[t, out_col + h v_dim + i] = out_scale * o[t, h, i] * rsqrt(mean_i o[t, h, :]^2 + eps) * w * act(y[t, gate_col + h v_dim + i]);
// w = weight[i], or weight[h v_dim + i] with weight_per_channel; act 0: silu, 1: sigmoid.  token_seq (may be null): rows
// of padding tokens (< 0) become zero.
cudaError_t launch_head_norm_gate(int dtype, const float* o, const void* y, int y_stride, int gate_col, const float* weight,
                                  int weight_per_channel, float eps, int act, void* out, int out_stride, int out_col,
                                  float out_scale, const int* token_seq, int n_tokens, int heads, int v_dim, cudaStream_t stream);

// Recurrences with one decay a head (recurrent_gated.cu), in the manner of the scans above: q, k, v and the gates' inputs are
// columns of y; the state is read at rows[sequence] and left as after the sequence's last token; out [tokens, heads * v_dim].
// The delta rule with one decay a head: q and k [kv_heads * dim], v [heads * v_dim] pass a causal convolution over time
// (conv_* [channels, taps], the last tap the present token's; the inputs before the step's first token from tail
// [state_rows, taps - 1, 2 kv_heads dim + heads v_dim], oldest first; null with one tap) and silu; q and k are divided head
// by head by sqrt(sum(.^2) + key_eps), q times q_scale; beta = sigmoid(y[b_col + h]), g = exp(-exp(a_log[h]) softplus(y[a_col + h]
// + dt_bias[h])); S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  state [state_rows, heads, dim, v_dim].
cudaError_t launch_gated_delta_scan(int dtype, const void* y, int stride, int q_col, int k_col, int v_col, int b_col, int a_col,
                                    const float* conv_q, const float* conv_k, const float* conv_v, int taps, const float* a_log,
                                    const float* dt_bias, float key_eps, float q_scale, float* state, int state_rows, const float* tail,
                                    const int* cu_q, const int* rows, int n_seqs, float* out, int heads, int kv_heads, int dim, int v_dim,
                                    int most_threads, int* status, cudaStream_t stream);
// tail [state_rows, kept, channels] takes the last `kept` inputs of every channel after the step (the step's last tokens, and
// before them what it held); the channels are up to four groups of columns [c_i, c_i + w_i) of y, one after the other.
cudaError_t launch_conv_tail_update(int dtype, const void* y, int stride, int c0, int w0, int c1, int w1, int c2, int w2, int c3, int w3,
                                    float* tail, int state_rows, int kept, int channels, const int* cu_q, const int* rows, int n_seqs,
                                    int* status, cudaStream_t stream);
// The matrix memory with exponential gates: i = cap tanh((y[i_col + h] + i_bias[h]) / cap), f = log sigmoid(cap tanh((y[f_col + h] +
// f_bias[h]) / cap)); m' = max(f + m, i); S <- exp(f + m - m') S + exp(i - m') k v^T, n likewise with k alone;
// o = S^T q / (max(|n . q|, exp(-m')) + den_eps), q times q_scale.  state [state_rows, heads, dim + 1, v_dim + 1]: S beside n (the
// last column), m at [dim, 0].
cudaError_t launch_memory_scan(int dtype, const void* y, int stride, int q_col, int k_col, int v_col, int i_col, int f_col,
                               const float* i_bias, const float* f_bias, float gate_cap, float q_scale, float den_eps, float* state,
                               int state_rows, const int* cu_q, const int* rows, int n_seqs, float* out, int heads, int dim, int v_dim,
                               int most_threads, int* status, cudaStream_t stream, float* snap);
// (snap [sequences, heads, dim + 1]: scratch for n and m as they are before the step, used where a head's columns lie on several CTAs)
// out = sum_i s_i w_i p_i / sqrt(mean(p_i^2) + eps), row by row, for n (1 to 4) float parts [tokens, width]; 32-bit.
cudaError_t launch_normed_sum(int n, const float* p0, const float* p1, const float* p2, const float* p3, const float* w0, const float* w1,
                              const float* w2, const float* w3, float s0, float s1, float s2, float s3, float eps, float* out,
                              int n_tokens, int width, cudaStream_t stream);
// x += other, element by element (float).
cudaError_t launch_add_rows(float* x, const float* other, long long n, cudaStream_t stream);

// The general attention (attention_general.cu).  Prepare: q [heads * dim] and k [kv_heads * dim] at their columns of y
// are rotated (pairs (i, i + half) of each head's first 2 half dimensions, angle position * freq[i]) and, with
// norm_eps >= 0, divided head by head by sqrt(mean(.^2) + norm_eps); q is written back, k and v [kv_heads * v_dim] go
// into k_cache [pages, kv_heads, page_size, dim] and v_cache [pages, v_heads, page_size, v_dim] if store.  The norm
// multiplies by q_weight / k_weight [dim] where given, and comes before the rotation with norm_first.  whole: the mean
// square is over all heads of q together (and of k), the weights are [heads * dim] and [kv_heads * dim], before the
// rotation.  rot_mult multiplies cos and sin.  qt_coef c != 0: q is multiplied by 1 + c ln((position + 1) / qt_every + 1)
// (integer division), last of all.
cudaError_t launch_attention_prepare(int dtype, void* y, int stride, int q_col, int k_col, int v_col, const int* positions,
                                     const int* token_seq, const float* freq, int half, float norm_eps, void* k_cache,
                                     void* v_cache, const int* block_table, int table_stride, int n_seqs, int n_pages,
                                     int n_tokens, int heads, int kv_heads, int dim, int v_dim, int page_size, int store,
                                     int* status, int v_heads, const float* q_weight, const float* k_weight, int norm_first,
                                     cudaStream_t stream, int whole = 0, float rot_mult = 1.f, float qt_coef = 0.f, int qt_every = 1);
// Token t at position p sees keys j <= p with j > p - window or j < keep_first (window > 0) and j / chunk == p / chunk
// (chunk > 0).  maps 2: q [heads, 2, dim], k_cache [pages, kv_heads * 2, page_size, dim], v_cache [pages, kv_heads, ..];
// out = out_scale * o / sqrt(mean(o^2) + sub_eps) with o = a_1 - lam * a_2, the two maps' attentions over the same values.
// softcap c > 0: a score becomes c tanh(score / c).  gate_mode 1: head h's result times sigmoid(y[t, gate_col + h]); 2: its
// element i times sigmoid(y[t, gate_col + h v_dim + i]).
cudaError_t launch_attention_general(int dtype, const void* y, int stride, int q_col, void* out, int out_stride, int out_col,
                                     float out_scale, const void* k_cache, const void* v_cache, const int* positions,
                                     const int* token_seq, const int* block_table, int table_stride, int n_seqs, int n_pages,
                                     int n_tokens, int heads, int kv_heads, int dim, int v_dim, int page_size, int window,
                                     int chunk, float scale, int* status, int keep_first, int maps, float lam, float sub_eps,
                                     cudaStream_t stream, const float* sinks = nullptr, int v_stride = 0, float softcap = 0.f,
                                     int gate_mode = 0, int gate_col = 0);

// Attention over paged rows that all heads share (attention_latent.cu), bfloat16 on the tensor cores: head h's query
// [key] at q_col + h * key of q; a row's first v_dim numbers are its value; out[t, out_col + h * v_dim + :].  sinks [heads]
// or null: exp(sink_h) joins the softmax's denominator.  tiles [n_tiles, 2] (sequence, first token), or null for a step
// of single tokens; a tile holds attention_latent_tile_rows() / min(heads, that) tokens.  A step of single tokens may cut every
// sequence's keys into n_splits (up to 16) runs with a CTA each, merged by a second kernel through part
// [n_splits, n_tokens, heads, v_dim + 2] float32.
bool attention_latent_supports(int key, int v_dim);
int attention_latent_tile_rows();
cudaError_t launch_attention_latent(const void* q, int q_stride, int q_col, void* out, int out_stride, int out_col, const void* pages,
                                    const int* cu_q, const int* q_start, const int* block_table, int table_stride, const int* tiles,
                                    int n_tiles, int n_pages, int heads, int key, int v_dim, int page_size, float scale,
                                    const float* sinks, int n_splits, float* part, int n_tokens, cudaStream_t stream);

// Differential attention on the tensor cores (attention_diff.cu), bfloat16: the two maps of attention_general with
// maps 2, for the sizes that attention_diff_supports names.  tiles [n_tiles, 2] (sequence, first token), or null for a
// step of single tokens (n_tiles = sequences).
bool attention_diff_supports(int dim, int v_dim, int heads, int kv_heads);
int attention_diff_tile_rows();
cudaError_t launch_attention_diff(const void* y, int y_stride, int q_col, void* out, int out_stride, int out_col, float out_scale,
                                  const void* k_cache, const void* v_cache, const int* cu_q, const int* q_start,
                                  const int* block_table, int table_stride, const int* tiles, int n_tiles, int tokens_per_tile,
                                  int n_pages, int heads, int kv_heads, int dim, int v_dim, int page_size, int window,
                                  int keep_first, float scale, float lam, float sub_eps, int* status, cudaStream_t stream);

// Retention (recurrent.cu): S <- decay[h] S + (k_scale k_t) v_t^T, o_t = S^T q_t for every (sequence, head), q and k
// rotated (pairs (i, i + half), angle positions[t] * freq[i], 32-bit) while they are staged.
cudaError_t launch_retention_scan(int dtype, const void* y, int stride, int q_col, int k_col, int v_col, const float* decay,
                                  float k_scale, const float* freq, int half, const int* positions, float* state, int state_rows,
                                  const int* cu_q, const int* rows, int n_seqs, float* out, int heads, int dim, int v_dim,
                                  int most_threads, int* status, float* ends, int end_rows, cudaStream_t stream, int act = 0);
// A long walk cut into segments (see recurrent.cu): rows[i] = -(n + 1) above starts segment i from zeros and leaves its
// last state in ends[n].  Carry: for split sequence s with later segments first .. first + count - 1 of lengths seg_len:
// starts[n] = the state before later segment n, and the request's row gets the last state.  Fix: tiles (later segment,
// first token, tokens <= 32, the segment's first token): out[t] += decay^(t - t0 + 1) starts[n]^T q_t.
cudaError_t launch_retention_carry(float* state, int state_rows, const float* ends, float* starts, const int* seq_row,
                                   const int* seq_first, const int* seq_count, const int* seg_len, int n_split, const float* decay,
                                   int heads, int dim, int v_dim, int* status, cudaStream_t stream);
cudaError_t launch_retention_fix(int dtype, const void* y, int stride, int q_col, const int* positions, const float* freq, int half,
                                 const float* starts, const int* tiles, int n_tiles, const float* decay, float* out, int heads, int dim,
                                 int v_dim, cudaStream_t stream, int act = 0);

// Mixture of experts (experts.cu): for each row of logits [n_tokens, experts] the `top` largest choose the experts, the
// softmax over the chosen logits weighs them; act[t, e * inter + i] *= weight of e (0 where e was not chosen), for
// act [n_tokens, act_stride] of `dtype`.
// The logits are given, or (x not null) formed in the kernel: logits[t, e] = x[t, :] . router[e, :] in 32-bit, x of `dtype`
// [n_tokens, width], router float [experts, width].
cudaError_t launch_route_experts(int dtype, const float* logits, const void* x, const float* router, int width, int n_tokens, int experts,
                                 int top, void* act, int act_stride, int inter, cudaStream_t stream, int mode = 0, float scale = 1.f);
// The grouped form: ids / weights [n_tokens, top] of each token's picks; lists [experts, list_stride] of the picks (flat
// index t * top + k) of every expert in rising order and counts [experts]; sorted [n_picks, width] the input rows by
// expert and where [n_picks] each pick's row; out[t] = sum_k weights[t, k] * y[where[t * top + k]] (+ shared_y[t]).
cudaError_t launch_route_topk(int x_dtype, const float* logits, const void* x, const float* router, int width, int n_tokens, int experts,
                              int top, int* ids, float* weights, cudaStream_t stream, int mode = 0, float scale = 1.f);
cudaError_t launch_expert_lists(const int* ids, int n_picks, int experts, int list_stride, int* lists, int* counts, cudaStream_t stream);
cudaError_t launch_gather_picks(int dtype, const void* x, int width, const int* lists, int list_stride, const int* counts, int experts,
                                int top, int n_picks, void* sorted, int* where, cudaStream_t stream);
cudaError_t launch_combine_picks(int dtype, const void* y, int width, const int* where, const float* weights, int top, int n_tokens,
                                 const void* shared_y, void* out, cudaStream_t stream);

// Layers with a latent for each token (latent.cu).
// Token shift: out[t] = x[t] + (x[t - 1] - x[t]) * mu [width]; before a sequence's first token of the step comes the row
// state[rows[seq]] (float [state_rows, width]), which then takes the sequence's last row of the step.
cudaError_t launch_token_shift(int out_dtype, const float* x, const float* mu, float* state, int state_rows, const int* cu_q,
                               const int* rows, const int* token_seq, int n_seqs, void* out, int n_tokens, int width, int* status,
                               cudaStream_t stream);
// The two latents of a token: y[t, q_col : q_col + q_rank] normed (root mean square, q_weight) into cq [tokens, cq_stride];
// y[t, kv_col : kv_col + kv_rank] normed (k_weight) and the rot_dim numbers behind it rotated (pairs (2i, 2i + 1), i < half,
// angle positions[t] * freq[i], cos and sin times mult) into the token's row of pages [n_pages, 1, page_size, kv_rank + rot_dim].
cudaError_t launch_latent_prepare(int dtype, const void* y, int stride, int q_col, int q_rank, int kv_col, int kv_rank, int rot_dim,
                                  const float* q_weight, const float* k_weight, float eps, const float* freq, int half, float mult,
                                  const int* positions, const int* token_seq, const int* block_table, int table_stride, int n_seqs,
                                  int n_pages, int page_size, void* cq, int cq_stride, void* pages, int store, int n_tokens, int* status,
                                  cudaStream_t stream);
// out[t, out_col + h out_head + j] = sum_i x[t, x_col + h x_head + i] m[h, i, j] (m [heads, inner, outer] of m_dtype), 32-bit sums.
// mode 1: the `tail` numbers behind a head's inputs are rotated like the shared key part and copied behind its outputs;
// mode 2: the output is multiplied by sigmoid(gate[t, gate_col + h outer + j]) (gate may be null).
cudaError_t launch_head_matmul(int dtype, int m_dtype, const void* x, int x_stride, int x_col, int x_head, const void* m, int heads,
                               int inner, int outer, void* out, int out_stride, int out_col, int out_head, int n_tokens, int mode,
                               int tail, const float* freq, int half, float mult, const int* positions, const int* token_seq,
                               const void* gate, int gate_stride, int gate_col, cudaStream_t stream);
// out = z > 0 ? ap z^2 + z / 2 : an (exp(z) - 1 - z) + z / 2, element by element.
cudaError_t launch_xielu(int dtype, const void* z, void* out, long long n, float ap, float an, cudaStream_t stream);
// out[t, i] = g sigmoid(alpha g) (u + 1), g = min(gate, lim), u = clamp(up, -lim, lim); lim = limit2 from column `split` on.
cudaError_t launch_gate_clamp(int dtype, const void* gu, void* out, int n_tokens, int inter, int interleave, float alpha, float limit,
                              int split, float limit2, cudaStream_t stream);

// dst[t, dst_col + i] = scale * src[t, i] for src [n_tokens, n] and dst [n_tokens, dst_stride], the product in 32-bit.
// dst[t, dst_col + h v_dim + i] = scale * src[t, h v_dim + i] * sigmoid(y[t, gate_col + (mode 1: h; mode 2: h v_dim + i)]);
// mode 0: no gate (scale_into).
cudaError_t launch_gate_into(int dtype, const void* src, const void* y, int y_stride, int gate_col, int mode, void* dst, int n_tokens,
                             int heads, int v_dim, int dst_stride, int dst_col, float scale, cudaStream_t stream);
cudaError_t launch_scale_into(int dtype, const void* src, void* dst, int n_tokens, int n, int dst_stride, int dst_col, float scale,
                              cudaStream_t stream);

// out[t, i] = silu(gate) * up.  interleave 0: gate = gu[t, i], up = gu[t, inter + i].  interleave 8: gate and up
// columns alternate in runs of 8 (g0..g7, u0..u7, g8.., ...): gate = gu[t, 16 (i / 8) + i % 8], up 8 further.
// inter % 8 == 0.
cudaError_t launch_silu_mul(int dtype, const void* gu, void* out, int n_tokens, int inter, int interleave,
                            cudaStream_t stream);

// Rotates q (in place) and k by the token's position and stores k and v into the pages.
// qkv [n_tokens, (heads + 2 kv_heads) * head_dim]; cos_sin [max_pos, head_dim / 2] of (cos, sin);
// k_cache, v_cache [pages, kv_heads, page_size, head_dim]; token_seq[t] < 0 marks padding.
// store == 0 rotates q only.
cudaError_t launch_rope_store(int dtype, void* qkv, const int* positions, const float2* cos_sin, int max_pos,
                              void* k_cache, void* v_cache, const int* token_seq, const int* block_table,
                              int table_stride, int n_seqs, int n_pages, int n_tokens, int heads, int kv_heads,
                              int head_dim, int page_size, int rotate, int store, int* status, cudaStream_t stream);

// C[M, N] = A[M, K] W[N, K]^T (+ bias[N]) with 32-bit multiply-adds in a fixed order (no tensor cores).
// (in, out) dtypes: (float, float), (bfloat16, bfloat16), (bfloat16, float).  k % 4 == 0.
cudaError_t launch_gemm_simt(int in_dtype, int out_dtype, const void* a, const void* w, const float* bias, void* c,
                             int m, int n, int k, cudaStream_t stream);

// Attention of every token over the paged keys of its sequence, one warp for a (token, head).
// q is read from qkv [n_tokens, qkv_stride] at column head * head_dim; out [n_tokens, heads * head_dim].
// Token t at position p of sequence s sees keys j with max(0, p - window + 1) <= j <= p (window <= 0: all).
cudaError_t launch_attention_simt(int dtype, const void* qkv, int qkv_stride, void* out, const void* k_cache,
                                  const void* v_cache, const int* positions, const int* token_seq,
                                  const int* block_table, int table_stride, int n_seqs, int n_pages, int n_tokens,
                                  int heads, int kv_heads, int head_dim, int page_size, int window, float scale,
                                  int* status, cudaStream_t stream);

// out[M, N] = x[M, K] w[N, K]^T (+ bias) for M <= 64 rows of bfloat16 x: the weight-streaming kernel.
// out is bfloat16 or float.  k % 8 == 0.
cudaError_t launch_gemm_skinny(int out_dtype, const void* x, const void* w, const float* bias, void* out, int m, int n,
                               int k, cudaStream_t stream);

// out[M, N] = x[M, K] w[N, K]^T (+ bias) with tcgen05.mma fed by TMA, accumulators in tensor memory.
// bfloat16 x and w, out bfloat16 or float, any M and N, k % 8 == 0.  status receives kStatusWaitTimeout
// if a bounded wait inside the kernel runs out.  scratch (floats) and counters (ints, zero before the
// first launch; the kernel leaves them zero) let a small batch cut k over several CTAs; without them
// k is not cut.  Launches that share them must not overlap on the GPU.
// epilogue 0: out[M, N] = sums + bias.  epilogue 1 (bfloat16 out, no bias, N % 16 == 0): the rows of w are
// gate and up rows interleaved in runs of 8 (g0..g7, u0..u7, g8.., ...) and out[M, N / 2] = silu(gate) * up.
// epilogue 2 (float out, M <= 256): k is cut into gemm_tc_shares(M, N, K) shares and out[share, M, N] takes each
// share's sums as they are (the bias with share 0); the kernel that reads them adds them (launch_rmsnorm).
// NextProduct: the product that the stream runs after this one (its matrix [n, k] of bfloat16, which no kernel writes, and its
// epilogue).  A kernel that streams weights for a small batch asks the first `bytes` of what that product will read
// into L2 once its own last load is on its way, so that HBM has work between the two kernels.  A hint: it changes no result.
struct NextProduct {
    const void* w;
    int n, k, epilogue;
    long long bytes;
};
int gemm_tc_shares(int m, int n, int k);
cudaError_t launch_gemm_tc(int out_dtype, const void* x, const void* w, const float* bias, void* out, int m, int n, int k,
                           int epilogue, float* scratch, long long scratch_floats, int* counters, int n_counters,
                           int* status, cudaStream_t stream, const NextProduct* next = nullptr);
// The same product for many rows of x with a tile of 256 rows of x by `bn` (256 or 192) rows of w to a pair of CTAs
// (tcgen05.mma.cta_group::2): bfloat16 out, epilogue 0 (bias) or 1 (SiLU(gate) * up).
cudaError_t launch_gemm_tc_pair(const void* x, const void* w, const float* bias, void* out, int m, int n, int k, int epilogue,
                                int bn, float* scratch, long long scratch_floats, int* counters, int n_counters, int* status,
                                cudaStream_t stream);

// In the three tensor-core attention launchers `chunk` > 0 adds the mask of chunks to the causal mask and the window: a
// token at position p sees key j only if j / chunk == p / chunk (chunks are counted from position 0 of the sequence).
// Tensor-core attention over the paged cache (bfloat16).  A tile is 16 * warps rows, row r being
// (token r / group, head r % group); `tiles` lists (sequence, first token) pairs, or is null when
// every sequence is one tile (single-token steps).  warps is 1 or 4.  With n_splits > 1 the keys of a
// tile are cut into n_splits runs whose partial results go to part_o [splits, tokens, heads, head_dim]
// and part_ml [splits, tokens, heads, 2] and are merged by a second kernel.
bool attention_mma_supports(int head_dim, int heads, int kv_heads, int warps);
cudaError_t launch_attention_mma(const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache,
                                 const int* cu_q, const int* q_start, const int* block_table, int table_stride,
                                 const int* tiles, int n_tiles, int n_pages, int n_tokens, int heads, int kv_heads,
                                 int head_dim, int page_size, int window, float scale, int warps, int n_splits,
                                 float* part_o, float* part_ml, int* status, cudaStream_t stream, int chunk = 0, const float* sinks = nullptr, float softcap = 0.f);

// Attention of prompt portions on tcgen05 tensor cores with the scores in tensor memory (head size 128):
// tiles of 128 rows of (token, head of the group) as in launch_attention_mma with 8 warps.
bool attention_tc_supports(int head_dim, int heads, int kv_heads);
cudaError_t launch_attention_tc(const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache,
                                const int* cu_q, const int* q_start, const int* block_table, int table_stride,
                                const int* tiles, int n_tiles, int n_pages, int heads, int kv_heads, int head_dim,
                                int page_size, int window, float scale, int* status, cudaStream_t stream, int chunk = 0,
                                const float* sinks = nullptr);

// Attention of single-token steps: every sequence brings tokens_per_tile = 16 / group tokens at most (one in a
// decode step).  Grid (sequences, kv_heads, n_splits), four warps a CTA.  With n_splits > 1 the runs' results
// pass through part_o [splits, tokens, heads, head_dim] and part_ml [splits, tokens, heads, 2], and
// counters [sequences * kv_heads] (zero before the first launch; left zero) tells the last CTA to merge.
// fuse_rope 1 (one token a sequence): q and k in qkv are still unrotated and the token's k and v are not in
// the cache; the kernel rotates q and k by cos_sin [max_pos, head_dim / 2] (null: no rotation) and, with
// store_kv, writes the token's k and v into their page: no rotation kernel has to run before it.  With fuse_rope,
// q, k and v may come as qkv_shares [n_shares, tokens, qkv_stride] float, the unadded shares of the product that
// made them (launch_gemm_tc, epilogue 2), instead of qkv: they are added where they are read.
// long_runs 1: the caller expects a warp to stream many blocks of keys (long contexts); head sizes 64 and 128 then
// fetch them as boxes of a tensor map, which arrive later than cp.async copies but cost far fewer instructions.
cudaError_t launch_attention_decode(const void* qkv, int qkv_stride, void* out, const void* k_cache, const void* v_cache,
                                    const int* cu_q, const int* q_start, const int* block_table, int table_stride,
                                    int n_seqs, int n_pages, int n_tokens, int heads, int kv_heads, int head_dim,
                                    int page_size, int window, float scale, int n_splits, float* part_o, float* part_ml,
                                    int* counters, int fuse_rope, const float2* cos_sin, int max_pos, int store_kv,
                                    const float* qkv_shares, int n_shares, int long_runs, int run_blocks, int* status,
                                    cudaStream_t stream, int chunk = 0);

// out[r] = index of the largest logit of row r (the lowest index among equals).
cudaError_t launch_argmax(const float* logits, int* out, int n_rows, int vocab, cudaStream_t stream);

// Sampling of one token for each row of float logits [n_rows, vocab]:
// temperature[r] <= 0 or top_k[r] == 1: argmax.  Else p = softmax(logits / temperature) restricted to the
// top_k[r] largest (top_k <= 0: all) and then to the smallest set of largest p whose sum reaches top_p[r];
// the token is the first index, in index order, at which the running sum of the kept p exceeds u[r] * total.
cudaError_t launch_sample(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                          const float* u, int* out, int n_rows, int vocab, cudaStream_t stream);

}  // namespace vtb
