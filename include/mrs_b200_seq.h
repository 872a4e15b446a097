/* mrs_b200_seq.h — C ABI of the sequence-mixer kernels (libmrs_b200_seq.so): multi-stream residuals
 * (hyper-connections), single residuals with Dynamic Tanh or RMS norms (the latter with a depth-weighted average over
 * the layers' results), gated linear recurrences with a per-sequence f32 state (linear attention with decay, selective
 * state spaces, matrix memories, per-row forget gates that also write), short causal convolutions, windowed attention
 * over a paged cache with unequal key and value head sizes, attention over cached low-rank latents, grouped-limited
 * expert routing and the expert feed-forward.
 *
 * Conventions: raw device pointers, caller-owned memory, stream-ordered, no allocation and no host
 * synchronisation; every function returns 0 or a cudaError (negative: a bad argument).  `dtype` is the storage
 * type of activations and of the paged cache (MRS_SEQ_BF16 / MRS_SEQ_F32); residual streams, states, norm
 * weights and every per-head constant are f32.
 *
 * A step's batch is a flat run of `n_tok` tokens from `n_seq` sequences: cu_tok[n_seq + 1] are the token
 * offsets, past[s] the tokens that sequence s already has in the cache / state, slot[s] its state slot.  A
 * sequence with past == 0 starts from a zero state whatever its slot holds. */
#ifndef MRS_B200_SEQ_H
#define MRS_B200_SEQ_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum { MRS_SEQ_BF16 = 1, MRS_SEQ_F32 = 2 };
enum { MRS_SEQ_ACT_NONE = 0, MRS_SEQ_ACT_SILU = 1, MRS_SEQ_ACT_GELU_TANH = 2, MRS_SEQ_ACT_SIGMOID = 3, MRS_SEQ_ACT_GELU_ERF = 4,
       MRS_SEQ_ACT_RELU_SQ = 5 };
/* How a gated feed-forward joins its two halves.  act != MRS_SEQ_GLU_CAPPED: act(gate) * up.  MRS_SEQ_GLU_CAPPED:
 * g = min(gate, limit), u = clamp(up, -limit, limit), result g * sigmoid(slope * g) * (u + shift). */
enum { MRS_SEQ_GLU_CAPPED = 100 };
typedef struct {
  int act;
  float limit, slope, shift;
} mrs_seq_glu_rule;

/* ---- residual streams ------------------------------------------------------------------------------ */
/* streams[t][s][:] = table[ids[t]][:] for every stream s (streams f32 [n_tok, n_streams, width]). */
int mrs_seq_embed_streams(const void *table, int dtype, const int32_t *ids, float *streams, int n_tok, int n_streams,
                          int width, int64_t stream);
/* out[r] = rms_norm(sum_s w_in[s] * streams[row(r)][s]) * (unit_offset + norm_w); rows: token of each output row
 * (NULL: all tokens in order).  w_in NULL: plain sum of the streams. */
int mrs_seq_streams_read_norm(const float *streams, const float *w_in, const float *norm_w, float eps, float unit_offset,
                              const int32_t *rows, void *out, int dtype, int n_rows, int n_streams, int width,
                              int64_t stream);
/* streams[t][r] <- sum_s w_mix[s][r] * streams[t][s] + w_out[r] * y[t], all r from the old values; when next_out is
 * given, the next sublayer's read + norm (as above, with next_in / next_norm_w) runs in the same pass. */
int mrs_seq_streams_write(float *streams, const float *w_mix, const float *w_out, const void *y, int dtype, int n_tok,
                          int n_streams, int width, const float *next_in, const float *next_norm_w, float eps,
                          float unit_offset, void *next_out, int64_t stream);

/* ---- single residual with Dynamic Tanh norms -------------------------------------------------------- */
/* A norm without statistics: dyt(z)[c] = tanh(alpha * z[c]) * weight[c] + bias[c]; alpha is ONE f32 on the device.
 * out[r] = dyt(x[row(r)]) for the f32 residual x [n_tok, width]; rows NULL: all tokens in order. */
int mrs_seq_tanh_norm_rows(const float *x, const int32_t *rows, const float *alpha, const float *weight, const float *bias,
                           void *out, int dtype, int n_rows, int width, int64_t stream);
/* One pass over the residual, every part optional (NULL: skipped), in this order:
 *   x <- x + dyt_post(y)        (y: a sublayer's output, activation type)
 *   x <- x + extra              (extra f32 [n_tok, width])
 *   next_out <- dyt_next(x)     (the next sublayer's input, activation type) */
int mrs_seq_residual_tanh_norm(float *x, const void *y, int dtype, const float *post_alpha, const float *post_weight,
                               const float *post_bias, const float *extra, const float *next_alpha, const float *next_weight,
                               const float *next_bias, void *next_out, int n_tok, int width, int64_t stream);

/* ---- single residual with RMS norms, scaled sublayer outputs and a depth-weighted average ------------ */
/* out[t][:] = table[ids[t]][:] * scale (f32). */
int mrs_seq_embed_scaled(const void *table, int dtype, const int32_t *ids, float scale, float *out, int n_tok, int width,
                         int64_t stream);
/* out[t][:] = table[ids[t]][:] * scale + pairs[row][:] (f32): a token embedding plus a hashed embedding of the (previous
 * token, token) pair, row = (previous * mul_prev + token * mul_cur) mod buckets, or row `buckets` (the table's last) for a
 * sequence's first token.  The previous token of a portion's first token comes from prev_state[slot] (int32 per state slot),
 * which is then set to the portion's last token.  cu_tok / past / slot / seq_of_tok describe the step's sequences. */
int mrs_seq_embed_pair(const void *table, const void *pairs, int dtype, const int32_t *ids, float scale, int64_t buckets,
                       int64_t mul_prev, int64_t mul_cur, int32_t *prev_state, const int32_t *cu_tok, const int32_t *past,
                       const int32_t *slot, const int32_t *seq_of_tok, float *out, int n_tok, int width, int64_t stream);
/* One pass per token over an f32 residual, every part optional (NULL: skipped), in this order:
 *   v = src[t] + mult * y[t]                       (y: a sublayer's output, activation type; NULL: v = src[t]; with post_w, y[t]
 *                                                    is first RMS-normed: y / sqrt(mean(y^2) + eps) * post_w — a norm after the
 *                                                    sublayer as well as before it)
 *   v += add_vec                                    (f32 [width], the same for every token; NULL: nothing)
 *   dst[t] = v                                      (dst may be src)
 *   v = sum_(j < n_hist) mix[j] * hist[j][t]        (hist f32 [n_hist][n_tok][width] with entry stride hist_stride floats;
 *                                                    an entry may be dst, which then already holds this token's v)
 *   mixed[t] = v
 *   next_out[t] = v / sqrt(mean(v^2) + eps) * next_w   (the next sublayer's input, activation type)
 * With hist = the embedding output followed by every layer's result so far this is the depth-weighted average of
 * DenseFormer-style models; without it, the plain pre-norm residual step with a multiplier. */
typedef struct {
  const float *src;
  float *dst;
  const void *y;
  float mult;
  const float *hist;
  int64_t hist_stride;
  int n_hist;
  const float *mix;
  float *mixed;
  const float *next_w;
  float eps;
  void *next_out;
  int dtype, n_tok, width;
  const float *post_w;
  const float *add_vec;
} mrs_seq_rms_residual_args;
int mrs_seq_rms_residual(const mrs_seq_rms_residual_args *args, int64_t stream);

/* ---- elementwise / norms --------------------------------------------------------------------------- */
/* x[t][c] = act(x[t][c]) in place for c < cols (row stride ld) */
int mrs_seq_activate_cols(void *x, int64_t ld, int dtype, int n_tok, int cols, int act, int64_t stream);
/* out[t][c] = act(x[t][c]) * x[t][half + c]   (x [n_tok, 2 * half]) */
int mrs_seq_glu_split(const void *x, void *out, int dtype, int n_tok, int half, int act, int64_t stream);
/* the same with any joining rule */
int mrs_seq_glu_join(const void *x, void *out, int dtype, int n_tok, int half, const mrs_seq_glu_rule *rule, int64_t stream);
/* gate[t][c] = lower[c] + (1 - lower[c]) * sigmoid(raw[t][c] + bias[c]) in f32: a forget gate bounded from below.  raw is
 * columns of an activation tensor (row stride raw_ld); gate f32 [n_tok, cols]. */
int mrs_seq_bounded_gate(const void *raw, int64_t raw_ld, int dtype, const float *bias, const float *lower, int n_tok, int cols,
                         float *gate, int64_t stream);
/* gate[t][c] = sigmoid(raw[t][c] + bias[c])^power in f32, as exp(power * log_sigmoid(.)): a decay per channel whose
 * logarithm is a softened log-sigmoid (power = 1 / temperature). */
int mrs_seq_power_gate(const void *raw, int64_t raw_ld, int dtype, const float *bias, float power, int n_tok, int cols, float *gate,
                       int64_t stream);
/* Root-mean-square norm of f32 rows in `groups` equal parts, times weight, with a gate read from an activation
 * tensor (row stride gate_ld): gate_first != 0: norm(x * act(gate)) * w; else norm(x) * w * act(gate).  The result,
 * times out_scale, goes to out[t * out_ld + c]. */
int mrs_seq_gated_group_norm(const float *x, const void *gate, int64_t gate_ld, const float *weight, void *out, int64_t out_ld,
                             float out_scale, int dtype, int n_tok, int cols, int groups, float eps, int gate_act,
                             int gate_first, int64_t stream);

/* ---- short causal convolution + step sizes ---------------------------------------------------------- */
/* Per channel c < channels: y[t][c] = act(bias[c] + sum_j taps[c][j] * x[t - (n_taps-1) + j][c]) over the tokens of
 * one sequence; inputs before the portion come from conv_state[slot][n_taps-1][channels] (zeros when past == 0),
 * which is then advanced to the last n_taps-1 inputs.  x is read from in[t * in_ld + col0 + c]. */
int mrs_seq_causal_conv(const void *in, int64_t in_ld, int col0, int dtype, const float *taps, const float *bias, int channels,
                        int n_taps, int act, float *conv_state, const int32_t *cu_tok, const int32_t *past,
                        const int32_t *slot, const int32_t *seq_of_tok, int n_seq, int n_tok, void *out, int64_t stream);
/* step[t][h] = softplus(raw[t][h] + bias[h]); decay[t][h] = exp(-exp(a_log[h]) * step[t][h]);  raw at
 * in[t * in_ld + col0 + h]. */
int mrs_seq_ssm_steps(const void *in, int64_t in_ld, int col0, int dtype, const float *bias, const float *a_log, int heads,
                      int n_tok, float *step, float *decay, int64_t stream);

/* ---- gated linear recurrence ---------------------------------------------------------------------- */
/* Per head h (keys / queries shared by heads / qk_groups neighbouring heads):
 *   S_t = a_t S_(t-1) + b_t k_t v_t^T     (S f32 [dk, dv], kept in state[slot][h])
 *   o_t = S_t^T q_t + skip[h] v_t         (o f32 [n_tok, heads * dv])
 * a_t = decay_tok[t][h] (or decay_head[h] when decay_tok is NULL), b_t = scale_tok[t][h] (1 when NULL), skip NULL: 0.
 * decay_vec f32 [n_tok, heads, dk] (then decay_tok and decay_head are NULL and qk_groups == heads): every state row has its
 * own decay, S_t = diag(f_t) S_(t-1) + k_t v_t^T; with k NULL the key is the decay's complement, S_t = diag(f_t) S_(t-1) +
 * (1 - f_t) v_t^T; seg_decay then holds one product per state row, f32 [n_seq * n_segs, heads, dk].
 * q_scale: a constant factor on the queries, applied in f32 as they are read (0: none).
 * q, k: [n_tok, qk_groups, dk] with row strides q_ld / k_ld; v: [n_tok, heads, dv] with row stride v_ld; `act` is
 * applied to q, k and v as they are read.
 * Long portions can run as n_segs segments of seg_len tokens side by side (n_segs > 1): the caller provides
 * seg_state f32 [n_seq * n_segs, heads, dk, dv] and seg_decay f32 [n_seq * n_segs, heads] as scratch; every segment is
 * first advanced from a zero state, the segments are chained (with the slot's state) into true start states, then
 * every segment runs again from its start and writes its outputs.  n_segs <= 1: one pass. */
typedef struct {
  const void *q, *k, *v;
  int64_t q_ld, k_ld, v_ld;
  int dtype, act;
  int heads, qk_groups, dk, dv;
  const float *decay_tok, *decay_head, *scale_tok, *skip;
  float *state;
  const int32_t *cu_tok, *past, *slot;
  int n_seq, n_tok;
  float *out;
  float *seg_state, *seg_decay;
  int seg_len, n_segs;
  const float *decay_vec;
  float q_scale;
} mrs_seq_scan_args;
int mrs_seq_linear_scan(const mrs_seq_scan_args *args, int64_t stream);

/* ---- stabilised matrix memory (mLSTM) ---------------------------------------------------------------- */
/* Gates of a matrix memory with a running maximum, per token t and head h, from raw gate pre-activations
 * raw_in / raw_forget f32 [n_tok, heads] (row stride raw_ld) that already hold their biases:
 *   i = cap tanh(raw_in / cap), f = logsigmoid(cap tanh(raw_forget / cap))   (cap <= 0: no soft cap)
 *   m_t = max(f + m_(t-1), i);  keep[t][h] = exp(f + m_(t-1) - m_t);  take[t][h] = exp(i - m_t);  m_tok[t][h] = m_t
 * m is carried per sequence in m_state f32 [n_slots, heads] and starts at 0 when past == 0.  keep / take are the
 * decay_tok / scale_tok of mrs_seq_linear_scan. */
int mrs_seq_mlstm_gates(const float *raw_in, const float *raw_forget, int64_t raw_ld, float cap, int heads, float *m_state,
                        const int32_t *cu_tok, const int32_t *past, const int32_t *slot, int n_seq, int n_tok, float *keep,
                        float *take, float *m_tok, int64_t stream);
/* vaug[t][h][0:dv] = v[t][h][:], vaug[t][h][dv] = 1, vaug[t][h][dv+1:dvp] = 0: with these values the scan's column dv
 * carries the normaliser n_t = keep n_(t-1) + take k_t and its output column dv is n_t . q_t. */
int mrs_seq_append_ones(const void *v, int64_t v_ld, int dtype, int heads, int dv, int dvp, int n_tok, void *vaug, int64_t stream);
/* o f32 [n_tok, heads, dvp] from the scan over augmented values: per head
 *   y = q_scale o[0:dv] / (max(|q_scale o[dv]|, exp(-m_tok)) + 1e-6);  y <- y / rms(y) (eps) * weight[h][:] * sigmoid(gate[h][:])
 * gate: activation type, row stride gate_ld; out: activation type [n_tok, heads * dv] with row stride out_ld. */
int mrs_seq_mlstm_out_norm(const float *o, int dvp, const float *m_tok, float q_scale, const void *gate, int64_t gate_ld,
                           const float *weight, float eps, int heads, int dv, void *out, int64_t out_ld, int dtype, int n_tok,
                           int64_t stream);

/* ---- windowed attention over a paged cache --------------------------------------------------------- */
/* Per-head RMS norm of q and k (both in place) with weights shared by the heads (NULL: no norm), then k and v of the new
 * tokens go to their cache slots.  Cache: k_cache [n_slots, kv_heads, dk], v_cache [n_slots, kv_heads, dv]
 * (slot = page * page_size + offset), storage type `dtype`. */
int mrs_seq_qk_norm_store(void *q, int64_t q_ld, void *k, int64_t k_ld, const void *v, int64_t v_ld, int dtype,
                          const float *q_norm_w, const float *k_norm_w, float eps, int heads, int kv_heads, int dk, int dv,
                          void *k_cache, void *v_cache, const int64_t *slot_of_tok, int n_tok, int64_t stream);
/* out[t][h] = softmax_j(scale * q_t . k_j) v_j over the cached positions j of t's sequence with
 * 0 <= pos(t) - j < window (window <= 0: every earlier position), times out_scale.  pages [n_seq, pages_ld].
 * tok_index (NULL: all n_tok tokens in order) lists the tokens to run: n_tok is then its length. */
int mrs_seq_window_attention(const void *q, int64_t q_ld, const void *k_cache, const void *v_cache, int dtype, int heads,
                             int kv_heads, int dk, int dv, float scale, int window, const int32_t *pages, int pages_ld,
                             int page_size, const int32_t *seq_of_tok, const int32_t *pos_of_tok, const int32_t *tok_index,
                             int n_tok, void *out, int64_t out_ld, float out_scale, int64_t stream);
/* The general forms of the two calls above.
 * prepare: norm_mode 0 none, 1 per head (weights [dk], shared by the heads), 2 over the whole projection at once
 * (weights [heads * dk] and [kv_heads * dk]); then rotation of the first rot_dims entries of every q / k head in pairs
 * (i, i + rot_dims / 2) by cos_sin f32 [n_tok, rot_dims / 2, 2] (NULL: none); q and k change in place, k and v go to their
 * cache slots.  v NULL: the values are the keys as projected (before norm and rotation; needs dv == dk). */
enum { MRS_SEQ_QK_NORM_NONE = 0, MRS_SEQ_QK_NORM_HEAD = 1, MRS_SEQ_QK_NORM_WHOLE = 2 };
typedef struct {
  void *q, *k;
  const void *v;
  int64_t q_ld, k_ld, v_ld;
  int dtype, norm_mode;
  const float *q_norm_w, *k_norm_w;
  float eps;
  int heads, kv_heads, dk, dv;
  int rot_dims;
  const float *cos_sin;
  void *k_cache, *v_cache;
  const int64_t *slot_of_tok;
  int n_tok;
} mrs_seq_attn_prepare_args;
int mrs_seq_attention_prepare(const mrs_seq_attn_prepare_args *args, int64_t stream);
/* cos_sin[t][i] = mag * (cos, sin)(pos_of_tok[t] * freq[i]), i < half; the angle and its cos / sin in double. */
int mrs_seq_rotation_table(const int32_t *pos_of_tok, const double *freq, int n_tok, int half, float mag, float *cos_sin,
                           int64_t stream);
/* attention: position i sees j <= i with i - j < window (window <= 0: all) or j < keep_first; sink f32 [heads] (NULL:
 * none) adds exp(sink[h]) to the softmax denominator — a key without a value whose score is not scaled. */
typedef struct {
  const void *q;
  int64_t q_ld;
  const void *k_cache, *v_cache;
  int dtype, heads, kv_heads, dk, dv;
  float scale;
  int window, keep_first;
  const float *sink;
  const int32_t *pages;
  int pages_ld, page_size;
  const int32_t *seq_of_tok, *pos_of_tok, *tok_index;
  int n_tok;
  void *out;
  int64_t out_ld;
  float out_scale;
  int64_t k_row, v_row;   /* elements between the cache rows of neighbouring slots; 0: kv_heads * dk / kv_heads * dv.  Values that
                             are a column range of the key rows: v_cache = k_cache + first column, v_row = k_row. */
  int pool;               /* > 0 (needs window > 0, keep_first 0): besides its window a position sees one averaged key / value per
                             block of `pool` positions that lies wholly before the window (mrs_seq_pool_blocks makes them) */
  int64_t pool_base;      /* cache row of the first averaged entry: block b of a sequence sits at row
                             pool_base + page * ceil(page_size / pool) + (b - first block that starts in the page) */
  int v_shared;           /* != 0: every head reads value columns [0, dv) of a row, whatever its key/value head — with dv = all
                             value heads side by side, head h's weights are applied to every value head */
  int out_f32;            /* != 0: out is f32 whatever the activation type */
  int64_t out_head;       /* elements between the heads of an output row; 0: dv.  With v_shared, a call may cover a column range of
                             the value heads (v_cache advanced to it) and write the same range of every head's output */
} mrs_seq_paged_attention_args;
int mrs_seq_paged_attention(const mrs_seq_paged_attention_args *args, int64_t stream);
/* Averaged cache entries for attention over pooled blocks: for every token of the step whose position ends a block of `pool`
 * positions, the mean (f32 sum / pool) of the block's cached rows is written to the block's row (see pool_base above), in the
 * k cache over k_cols columns and in the v cache over v_cols columns.  Run after the step's keys and values are stored. */
int mrs_seq_pool_blocks(void *k_cache, void *v_cache, int dtype, int64_t k_row, int64_t v_row, int k_cols, int v_cols, int pool,
                        int64_t pool_base, const int32_t *pages, int pages_ld, int page_size, const int32_t *seq_of_tok,
                        const int32_t *pos_of_tok, int n_tok, int64_t stream);
/* Attention weights mixed across heads after the softmax, applied through linearity: a f32 [n_tok, heads, kv_heads * dv]
 * holds, per head g, its weights applied to EVERY value head (mrs_seq_paged_attention with v_shared); out[t][h][:] =
 * act(gate[t][h][:]) * sum_g mix[h][g] * a[t][g][value head of h][:].  mix f32 [heads, heads]; gate: activation type, row
 * stride gate_ld, NULL: none. */
int mrs_seq_mix_heads(const float *a, const float *mix, const void *gate, int64_t gate_ld, int gate_act, void *out, int64_t out_ld,
                      int dtype, int heads, int kv_heads, int dv, int n_tok, int64_t stream);
/* x[t][c] *= act(gate[t][c / group]) for c < cols: a gate per entry (group 1) or per head (group = head size). */
int mrs_seq_gate_cols(void *x, int64_t x_ld, const void *gate, int64_t gate_ld, int dtype, int cols, int group, int act, int n_tok,
                      int64_t stream);
/* The long portions of a step on tensor cores (bf16, dk = dv = d of 64 or 128, q / out rows 16-byte aligned), with the same
 * window / keep_first / sink rule: queries are the portion's fresh rows of q, keys and values are read from the pages (the
 * portion's own, stored by the preparation, and everything cached before).  portions [n][4]: first row inside q / out,
 * row count, positions cached before the portion, row of `pages`; longest = the largest row count. */
int mrs_seq_prompt_attention(const void *q, int64_t q_ld, const void *k_cache, const void *v_cache, void *out, int64_t out_ld,
                             const int32_t *portions, int n_portions, int longest, const int32_t *pages, int pages_ld,
                             int page_size, int heads, int kv_heads, int d, float scale, int window, int keep_first,
                             const float *sink, int64_t stream);
/* The same with averaged blocks before the window (pool > 0, rows pool_base.. of the caches as for mrs_seq_paged_attention;
 * needs window > 0 and keep_first 0) and / or with every head's weights applied to every value head (every_value_head != 0:
 * out is then f32 [n_tok, heads, kv_heads * d] with row stride out_ld floats — the input of mrs_seq_mix_heads). */
int mrs_seq_prompt_attention_pooled(const void *q, int64_t q_ld, const void *k_cache, const void *v_cache, void *out, int64_t out_ld,
                                    const int32_t *portions, int n_portions, int longest, const int32_t *pages, int pages_ld,
                                    int page_size, int heads, int kv_heads, int d, float scale, int window, int keep_first,
                                    const float *sink, int pool, int64_t pool_base, int every_value_head, int64_t stream);
/* ---- attention through a shared latent ----------------------------------------------------------------- */
/* Per token, from the columns of one projection y (row stride y_ld, activation type), any part optional:
 *   q_out[t] = rms_norm(y[t][q_col : q_col + q_rank]) * q_norm_w                      (the query latent, activation type)
 *   cache[slot(t)][0 : kv_rank] = rms_norm(y[t][kv_col : kv_col + kv_rank]) * kv_norm_w   (the key/value latent)
 *   cache[slot(t)][kv_rank : kv_rank + rot_dim] = turn(y[t][kv_col + kv_rank : ...])     (the key part all heads share)
 * turn: entries (2i, 2i + 1), i < rot_dims / 2, rotate by cos_sin[t][i] (f32 [n_tok, rot_dims / 2, 2]); the rest pass.
 * cache rows are cache_row elements apart.  q_rank 0: no query part; kv_rank 0: no cache part.  kv_out (optional): the normed
 * key/value latent also goes to kv_out[t][0 : kv_rank] (row stride kv_out_ld), for callers that decompress keys and values
 * of the step's own tokens with a matrix product. */
typedef struct {
  const void *y;
  int64_t y_ld;
  int dtype;
  int q_col, q_rank;
  const float *q_norm_w;
  void *q_out;
  int64_t q_out_ld;
  int kv_col, kv_rank, rot_dim, rot_dims;
  const float *kv_norm_w;
  const float *cos_sin;
  float eps;
  void *cache;
  int64_t cache_row;
  const int64_t *slot_of_tok;
  int n_tok;
  void *kv_out;
  int64_t kv_out_ld;
} mrs_seq_latent_prepare_args;
int mrs_seq_latent_prepare(const mrs_seq_latent_prepare_args *args, int64_t stream);
/* out[t][h][0:dims] = in[t][h][0:dims] with entries (2i, 2i + 1), i < rot_dims / 2, rotated by cos_sin[t][i], the rest
 * copied.  in / out: activation type, row strides in_ld / out_ld, head strides in_head / out_head (elements). */
int mrs_seq_rotate_pairs(const void *in, int64_t in_ld, int64_t in_head, void *out, int64_t out_ld, int64_t out_head, int dtype,
                         int heads, int dims, int rot_dims, const float *cos_sin, int n_tok, int64_t stream);

/* The long portions of a step on tensor cores, in the absorbed form: q [n_tok, heads, kv_rank + rot_dim] (row stride q_ld) holds
 * per head [W_uk^T q_plain | q_rot]; the cached rows (cache_row elements apart) are at once the keys (all kv_rank + rot_dim
 * columns) and the values (the first kv_rank columns) of every head; out [n_tok, heads, kv_rank] (row stride out_ld).
 * Position i sees j with 0 <= i - j < window (window <= 0: every earlier position).  portions / longest / pages as for
 * mrs_seq_prompt_attention; portions NULL: every sequence of the step is one portion (cu_tok / past as for the scan,
 * n_portions = n_seq, page-table row = sequence), decoded tokens included.  bf16; kv_rank and kv_rank + rot_dim multiples of 8; mrs_seq_latent_attention_fits tells
 * whether the sizes fit the kernel's shared memory (else: mrs_seq_paged_attention with row strides). */
int mrs_seq_latent_attention_fits(int kv_rank, int rot_dim);
int mrs_seq_latent_attention(const void *q, int64_t q_ld, const void *cache, int64_t cache_row, void *out, int64_t out_ld,
                             const int32_t *portions, const int32_t *cu_tok, const int32_t *past, int n_portions, int longest,
                             const int32_t *pages, int pages_ld, int page_size, int heads, int kv_rank, int rot_dim, float scale,
                             int window, int64_t stream);

/* x[r][c] *= scale for r < rows, c < cols (row stride ld) */
int mrs_seq_scale_rows(void *x, int64_t ld, int dtype, int rows, int cols, float scale, int64_t stream);

/* ---- mixture of experts ---------------------------------------------------------------------------- */
/* scores = softmax(logits) over n_experts; choice = scores + correction (NULL: 0); experts form n_groups equal
 * groups of neighbours, a group's score is its largest choice, only the keep_groups best groups stay eligible; the
 * `top` eligible experts with the largest choice are taken, their weights are their scores (renormalised to sum 1
 * when renorm != 0).  experts / weights: [n_tok, top]. */
int mrs_seq_moe_route(const float *logits, const float *correction, int n_tok, int n_experts, int n_groups, int keep_groups,
                      int top, int renorm, int32_t *experts, float *weights, int64_t stream);
/* The same rule with its choices open: scores = softmax over the experts (score_fn 0) or sigmoid of each logit (1); a
 * group's score is the sum of its group_top largest choices (1: the largest); the weights are the chosen scores
 * (renormalised when renorm != 0) times weight_scale. */
enum { MRS_SEQ_SCORE_SOFTMAX = 0, MRS_SEQ_SCORE_SIGMOID = 1 };
int mrs_seq_moe_route_scored(const float *logits, const float *correction, int n_tok, int n_experts, int n_groups, int keep_groups,
                             int top, int renorm, int score_fn, int group_top, float weight_scale, int32_t *experts,
                             float *weights, int64_t stream);
/* Small batches: hidden[t][k][:] = act(gate_up[e][0:ff] x_t) * (gate_up[e][ff:2ff] x_t), e = experts[t][k]
 * (gate_up [n_experts, 2 * ff, width]), then out[t] = sum_k weights[t][k] * down[e] hidden[t][k]
 * (down [n_experts, width, ff]). */
int mrs_seq_moe_gate_up(const void *x, const void *gate_up, int dtype, const int32_t *experts, int n_tok, int top, int width,
                        int ff, int act, void *hidden, int64_t stream);
int mrs_seq_moe_down(const void *hidden, const void *down, int dtype, const int32_t *experts, const float *weights, int n_tok,
                     int top, int width, int ff, void *out, int64_t stream);
/* mrs_seq_moe_gate_up with any joining rule */
int mrs_seq_moe_gate_up_rule(const void *x, const void *gate_up, int dtype, const int32_t *experts, int n_tok, int top, int width,
                             int ff, const mrs_seq_glu_rule *rule, void *hidden, int64_t stream);
/* The plain rule: the `top` experts with the largest logits, weights = softmax over the chosen logits alone. */
int mrs_seq_moe_route_top_softmax(const float *logits, int n_tok, int n_experts, int top, int32_t *experts, float *weights,
                                  int64_t stream);
/* Experts without a gate: hidden[t][k][:] = act(up[e] x_t), up [n_experts, ff, width]; followed by mrs_seq_moe_down. */
int mrs_seq_moe_up(const void *x, const void *up, int dtype, const int32_t *experts, int n_tok, int top, int width, int ff,
                   int act, void *hidden, int64_t stream);
/* Large batches: rows sorted by expert.  counts[e] rows per expert, order[i] = the (token, k) pair (as token * top + k) at
 * sorted row i; gather copies x rows into sorted order, combine sums the experts' outputs back per token in k order. */
int mrs_seq_moe_sort(const int32_t *experts, int n_pairs, int n_experts, int32_t *counts, int32_t *order, int64_t stream);
int mrs_seq_moe_gather(const void *x, int dtype, const int32_t *order, int n_pairs, int top, int width, void *sorted,
                       int64_t stream);
int mrs_seq_moe_combine(const void *sorted_y, int dtype, const int32_t *order, const float *weights, int n_tok, int top,
                        int width, int32_t *scratch_inverse, void *out, int64_t stream);

#ifdef __cplusplus
}
#endif
#endif
