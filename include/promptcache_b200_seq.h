/*
 * promptcache_b200 -- C ABI of the sequence-batch kernels (libpromptcache_b200_seq.so).
 *
 * These kernels serve models whose step runs a BATCH of sequences as one concatenated token matrix over a pool of
 * per-sequence slots: attention layers keep K/V rows per slot, recurrent layers keep a state per slot.  Each mechanism
 * is one entry point whose constants are parameters, so that several model designs can share them:
 *
 *   pcs_embed            token embedding times a scale into the 32-bit residual stream
 *   pcs_rmsnorm          RMS norm of 32-bit rows, result in the compute type
 *   pcs_gate_norm_add    x += ls * w * rms(y * sigmoid(g))   (gated sublayer result, output norm, layer scale, residual sum),
 *                        optionally followed by the next sublayer's input norm
 *   pcs_xielu            xIELU activation
 *   pcs_qk_prep          whole-projection RMS norm of q and k, position-dependent query temperature, value mixing with an
 *                        earlier layer's values, append of K/V rows to the slot pool
 *   pcs_attn             causal attention over the slot pool with distinct key and value widths, grouped heads, an optional
 *                        logarithmic distance bias and an optional sink term in the softmax denominator
 *   pcs_mlstm_gates      capped input / forget gate pre-activations of a matrix-memory recurrent layer
 *   pcs_mlstm_scan       the stabilised matrix-memory recurrence with its per-head output norm and output gate
 *   pcs_embed_bigram     token embedding plus a row of a hashed (previous token, token) table
 *   pcs_norm_conv        residual sum, RMS norm (one weight per channel or one number) and a short causal convolution over
 *                        time whose last inputs are carried in the slot pool
 *   pcs_rope_kv_prep     rotation of a leading part of every query / key head by position (arbitrary frequency table),
 *                        unit-RMS values, append of K/V rows to the slot pool
 *   pcs_moe_route        router of a mixture of experts: softmax or sigmoid scores, choice with a correction and group limits
 *   pcs_moe_rows_*       the chosen experts' feed-forward (gated, or one up-projection) for a handful of rows (weights streamed once)
 *   pcs_moe_plan/_gemm   the same for many rows: rows sorted by expert, grouped tensor-core products
 *   pcs_moe_combine      weighted sum of expert results, pass-through experts and a gated shared expert into the residual
 *   pcs_silu_mul         silu(gate) * up;  pcs_glu_mul: the same with the activation as a parameter
 *   pcs_depth_mix        weighted sum of the results of all earlier layers (depth-weighted average), with the next norm
 *   pcs_latent_prep      low-rank attention: norms of the query and key/value latents, rotation of the shared key part, append
 *                        of [latent | rotated part] rows to the slot pool
 *   pcs_latent_q         rotation of the queries' rotated part; with latent-space queries, their packing beside it
 *   pcs_latent_expand    per-head key / value rows from up-projected latents and the pool's rotated parts, into a dense pool
 *   pcs_head_gate        out[t, h, :] = o[t, h, :] * sigmoid(g[t, h])
 *   pcs_gla_decay        per key channel log decay  logsigmoid(A2 a + b) / tau  of a gated linear-attention layer
 *   pcs_gla_scan         S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, per-head output norm and silu gate
 *   pcs_add_layer_norm   residual sum of up to three sublayer results and layer norms (weight, no bias) of the new stream with
 *                        one or two weight vectors, for layers whose sublayers run side by side on the same input
 *   pcs_gru_scan         element-wise gated recurrence whose gates read only the current token, S_t = (1 - z_t) S_(t-1) + z_t c_t,
 *                        with its silu output gate
 *   (pcs_attn with `talk`: every (query, key) pair's scores of all heads are mixed by an [H, H] matrix before the softmax)
 *
 * All tensor arguments are DEVICE pointers; `dtype` selects the compute / storage type of activations, weights and K/V
 * rows: PCS_BF16 or PCS_F32 (true 32-bit everywhere).  The residual stream, norms' statistics, attention scores and
 * weights, gates and recurrent state are 32-bit floats in both modes.  Calls are asynchronous on `stream`.
 *
 * The batch is described by int32 arrays on the device:
 *   tok_seq[t]   batch entry of token t          tok_pos[t]   position of token t inside its sequence
 *   seq_slot[b]  pool slot of entry b            seq_pos0[b]  rows / tokens the slot already holds
 *   seq_len[b]   new tokens of entry b           seq_off[b]   index of its first token in the concatenated matrix
 */
#ifndef PROMPTCACHE_B200_SEQ_H_
#define PROMPTCACHE_B200_SEQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PCS_ABI_VERSION 4
#define PCS_BF16 0
#define PCS_F32 1

enum { PCS_OK = 0, PCS_ERR_INVALID = -1, PCS_ERR_UNSUPPORTED = -2, PCS_ERR_CUDA = -3 };

int pcs_version(void);
const char* pcs_last_error(void);
int64_t pcs_launch_count(void);

/* out[t, :] = table[ids[t], :] * scale        (out fp32 [n, width]; ids int64) */
int pcs_embed(const void* table, const int64_t* ids, float* out, int n_tokens, int width, int vocab, float scale, int dtype,
              void* stream);

/* out[r, :] = x[rows ? rows[r] : r, :] / sqrt(mean(x^2) + eps) * w      (x fp32, w and out in `dtype`) */
int pcs_rmsnorm(const float* x, const int32_t* rows, const void* w, void* out, int n_rows, int width, float eps, int dtype,
                void* stream);

/* x[r, :] += ls * (w_offset + w) * rms(y[r, :] * sigmoid(g[r, :]))   (g may be NULL: no gate; ls may be NULL: no layer scale)
 * then, if next_w != NULL, h_out[r, :] = rms(x[r, :]) * (w_offset + next_w).  y and g are `dtype` with row strides in elements
 * (y is fp32 when y_f32 is set).  w_offset is 0 for plain weights and 1 for weights stored around zero; the sum is formed in
 * 32-bit. */
typedef struct pcs_gna_params {
  float* x;
  const void* y;
  const void* g;
  int64_t y_stride, g_stride;
  const void* w;
  const void* ls;
  const void* next_w;
  void* h_out;
  int n_rows, width;
  float eps;
  int dtype;
  float w_offset;
  int y_f32;
} pcs_gna_params;
int pcs_gate_norm_add(const pcs_gna_params* p, void* stream);

/* xIELU: z > 0: softplus(a[0]) z^2 + z/2;  z <= 0: (1/2 + softplus(a[1])) (exp(z) - 1 - z) + z/2.   `a` holds two `dtype` numbers. */
int pcs_xielu(const void* z, int64_t z_stride, void* out, int64_t out_stride, const void* a, int n_rows, int width, int dtype,
              void* stream);

typedef struct pcs_qkprep_params {
  const void* qkv;          /* [n_tokens, row_stride]: q at q_off, k at k_off, v at v_off (biases already added) */
  int64_t row_stride;
  int32_t q_off, k_off, v_off;
  const void* q_norm_w;     /* [H*dim] or NULL (no query norm) */
  const void* k_norm_w;     /* [Hkv*dim] or NULL */
  float eps;
  int32_t n_heads, n_kv_heads, dim, vdim;
  float temp_coef;          /* q *= 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1); temp_every <= 0: none */
  int32_t temp_every;
  void* q_out;              /* [n_tokens, H*dim] */
  void* k_pool;             /* [slots, Hkv, cap, dim] */
  void* v_pool;             /* [slots, Hkv, cap, vdim] */
  int32_t cap;
  const void* v_first_pool; /* value pool of the layer whose values are mixed in, or NULL */
  const void* v_lambda;     /* one `dtype` number: v = (1 - lambda) v + lambda v_first */
  const int32_t* tok_seq;
  const int32_t* tok_pos;
  const int32_t* seq_slot;
  int32_t n_tokens, dtype;
} pcs_qkprep_params;
int pcs_qk_prep(const pcs_qkprep_params* p, void* stream);

typedef struct pcs_attn_params {
  const void* q;            /* [n_tokens, H*dim] */
  const void* k_pool;
  const void* v_pool;
  void* out;                /* [n_tokens, H*vdim] */
  int32_t n_heads, n_kv_heads, dim, vdim, cap;
  float scale;
  const float* bias_r1;     /* [H] or NULL: score -= r1[h] * ln(1 + r2[h] * (i - j)) */
  const float* bias_r2;
  int32_t sink;             /* 1: the softmax denominator has one more term, exp(sink_logit[h]) (exp(0) without sink_logit), that carries no value */
  const int32_t* tok_seq;
  const int32_t* tok_pos;
  const int32_t* seq_slot;
  const int32_t* seq_pos0;
  const int32_t* seq_len;
  const int32_t* seq_off;
  int32_t n_tokens, n_seqs, max_len, dtype;   /* max_len: host upper bound of the new tokens of one entry */
  int32_t impl;             /* 0 = automatic, 1 = the plain kernel */
  int32_t max_keys;         /* host upper bound of the keys one token sees (sizes the split of the keys); 0: one split */
  float* workspace;         /* fp32 scratch of pcs_attn_workspace_floats() elements, or NULL (one split) */
  int64_t workspace_floats;
  float softcap;            /* > 0: score = softcap * tanh(score / softcap), after the scale and before the bias */
  int32_t window;           /* > 0: query i sees key j only if i - j < window or j < keep_first */
  int32_t keep_first;       /* the first keys of a sequence that stay visible beyond the window */
  int32_t v_row_stride;     /* elements between the value rows of neighbouring keys; 0: vdim.  With a stride the values may be a
                               leading part of the key rows themselves (v_pool == k_pool, v_row_stride == dim) */
  const float* sink_logit;  /* [H] or NULL */
  const int32_t* pool_slot; /* [n_seqs] or NULL: overrides seq_slot (a dense pool that is indexed by the batch entry) */
  const float* talk;        /* [H, H] or NULL: the scaled scores of a (query, key) pair are mixed across heads before the mask and
                               the softmax, score'[h] = sum_g talk[h, g] * score[g].  Not with a bias, a cap or a sink. */
  const void* out_gate;     /* [n_tokens, out_gate_stride] `dtype` or NULL: out[t, c] *= sigmoid(out_gate[t, c]) over all H * vdim columns
                               (an element-wise output gate, applied where the result is normalised; only with `talk`) */
  int64_t out_gate_stride;
} pcs_attn_params;
/* scratch the key split of pcs_attn needs for n_tokens tokens */
int64_t pcs_attn_workspace_floats(int n_tokens, int n_heads, int vdim);
int pcs_attn(const pcs_attn_params* p, void* stream);

/* ig = cap * tanh((w_i h + b_i) / cap);  fg = logsigmoid(cap * tanh((w_f h + b_f) / cap))    (fp32 [n_tokens, heads]) */
int pcs_mlstm_gates(const void* h, int64_t h_stride, const void* w_i, const void* w_f, const float* b_i, const float* b_f,
                    float* ig, float* fg, int n_tokens, int width, int heads, float cap, int dtype, void* stream);

/* out[m, n] = sum_k x[m, k] w[n, k] + bias[n] for 1 to 8 rows (decoding): the weights are streamed once, sums are fp32.
   k, the row stride of x and the pointers of x and w must be multiples of 16 bytes. */
int pcs_linear_rows(const void* x, int64_t x_stride, const void* w, const void* bias, void* out, int64_t out_stride, int m, int n, int k,
                    int dtype, void* stream);

typedef struct pcs_mlstm_params {
  const void* proj;         /* [n_tokens, row_stride]: q at q_off, k at k_off, v at v_off, output-gate pre-activation at g_off */
  int64_t row_stride;
  int32_t q_off, k_off, v_off, g_off;
  const float* ig;          /* [n_tokens, heads] log input gate  */
  const float* fg;          /* [n_tokens, heads] log forget gate */
  const void* norm_w;       /* [heads*vdim] */
  void* out;                /* [n_tokens, heads*vdim] */
  float* s_pool;            /* [slots, heads, dim, vdim] */
  float* n_pool;            /* [slots, heads, dim] */
  float* m_pool;            /* [slots, heads] */
  int32_t heads, dim, vdim;
  float q_scale;            /* dim^(-1/2) */
  float eps;
  const int32_t* seq_slot;
  const int32_t* seq_pos0;
  const int32_t* seq_len;
  const int32_t* seq_off;
  int32_t n_seqs, dtype;
  int32_t max_len;          /* host upper bound of the new tokens of one entry */
  int32_t impl;             /* 0 = automatic, 1 = token by token with the state in shared memory, 2 = token by token (registers
                               where the sizes allow): never the chunkwise tensor-core kernel */
  float* o_raw;             /* fp32 scratch of n_tokens*heads*vdim + n_seqs*heads*(dim+1) elements: the recurrence's result before
                               the per-head norm, and the new n / m of every entry until they are committed */
  int32_t n_tokens, reserved;
} pcs_mlstm_params;
int pcs_mlstm_scan(const pcs_mlstm_params* p, void* stream);

/* out[t, :] = table[ids[t], :] + pair[r, :], r = (prev_ids[t] * mul_prev + ids[t] * mul_cur) mod buckets, or r = buckets (the
 * table's last row) where prev_ids[t] < 0 (a sequence's first token).  out fp32 [n, width]; pair [buckets + 1, width]. */
int pcs_embed_bigram(const void* table, const void* pair, const int64_t* ids, const int64_t* prev_ids, float* out, int n_tokens,
                     int width, int vocab, int64_t buckets, int64_t mul_prev, int64_t mul_cur, int dtype, void* stream);

/* Per token t:  x[t] += y_mult * y[t]  (y may be NULL),  u[t] = x[t] / sqrt(mean(x[t]^2) + eps) * g,
 *               h_out[t] = u[t] + sum_{j < taps} conv_w[j, :] * u[t - taps + 1 + j]        (conv_w NULL: h_out = u)
 * u of tokens before the sequence's start is zero; u of tokens of earlier steps comes from `tail`, which holds the last
 * taps - 1 inputs of every slot twice: a step reads copy seq_par[b] and writes copy 1 - seq_par[b] (the caller alternates
 * seq_par from step to step), so no block reads what another one writes.  y and conv_w together are not supported (the
 * convolution reads neighbouring rows of x, which other blocks would be updating).  h_out NULL: only the sum. */
typedef struct pcs_normconv_params {
  float* x;                 /* [n_tokens, width] */
  const void* y;            /* [n_tokens, y_stride] `dtype`, or NULL */
  int64_t y_stride;
  float y_mult;
  const void* g;            /* `dtype`: g_len == 1 one number for all channels, else [width] */
  int32_t g_len;
  float eps;
  const void* conv_w;       /* [taps, width] `dtype` (tap-major: a tap's weights of neighbouring channels are one load), or NULL */
  int32_t taps;
  float* tail;              /* [slots, 2, taps - 1, width] fp32 */
  void* h_out;              /* [n_tokens, width] `dtype`, or NULL */
  const int32_t* tok_seq;
  const int32_t* tok_pos;
  const int32_t* seq_slot;
  const int32_t* seq_pos0;
  const int32_t* seq_len;
  const int32_t* seq_par;
  int32_t n_tokens, width, dtype, reserved;
} pcs_normconv_params;
int pcs_norm_conv(const pcs_normconv_params* p, void* stream);

typedef struct pcs_rope_params {
  const void* qkv;          /* [n_tokens, row_stride]: q at q_off, k at k_off, v at v_off */
  int64_t row_stride;
  int32_t q_off, k_off, v_off;   /* k_off < 0: the layer has no keys and values of its own (it reads another layer's rows) */
  int32_t n_heads, n_kv_heads, dim, vdim;
  const double* freqs;      /* [rot_dims / 2] angular frequencies: coordinate pair i of a head turns by pos * freqs[i] */
  int32_t rot_dims;         /* leading coordinates of every head that are rotated (even, <= dim); the rest pass unchanged */
  int32_t interleaved;      /* 1: pairs (2i, 2i+1); 0: pairs (i, i + rot_dims/2) */
  int32_t v_unit_rms;       /* 1: every value head is divided by sqrt(mean(v^2) + eps) before it is cached */
  float eps;
  void* q_out;              /* [n_tokens, H*dim] */
  void* k_pool;             /* [slots, Hkv, cap, dim] */
  void* v_pool;             /* [slots, Hkv, cap, vdim] */
  int32_t cap;
  const int32_t* tok_seq;
  const int32_t* tok_pos;
  const int32_t* seq_slot;
  int32_t n_tokens, dtype;
  const void* q_norm_w;     /* [dim] `dtype` or NULL: every query head is divided by sqrt(mean(q^2) + eps) and multiplied by this, */
  const void* k_norm_w;     /* [dim] or NULL: the same for every key head; both before the rotation, in 32-bit */
} pcs_rope_params;
int pcs_rope_kv_prep(const pcs_rope_params* p, void* stream);

/* Router of a mixture of experts, per token: z = w_router h (32-bit sums), s = softmax(z) over all n_outputs (or sigmoid(z), see
 * score_fn), choice scores c = s + correction.  Outputs form n_groups equal groups of neighbours; a group's score is its largest c
 * (or the sum of its group_best largest); only outputs of
 * the keep_groups best groups can be chosen; the `top` largest c among them are chosen (ties: the lower index).
 * idx[t, k] = the k-th choice, wgt[t, k] = s of it (not renormalised).  shared_gate[t] = sigmoid(w_sg . h) when w_sg is given. */
typedef struct pcs_route_params {
  const void* h;            /* [n_tokens, h_stride] `dtype` */
  int64_t h_stride;
  const void* w_router;     /* [n_outputs, width] `dtype` */
  const float* correction;  /* [n_outputs] or NULL */
  const void* w_sg;         /* [width] `dtype` or NULL */
  int32_t n_tokens, width, n_outputs, top, n_groups, keep_groups;
  int32_t* idx;             /* [n_tokens, top] */
  float* wgt;               /* [n_tokens, top] */
  float* shared_gate;       /* [n_tokens] or NULL */
  int32_t dtype;
  int32_t renorm;           /* 1: wgt is divided by the sum over the token's choices (the softmax over the chosen logits alone) */
  const float* bias;        /* [n_outputs] or NULL: added to z before the softmax */
  int32_t score_fn;         /* 0: s = softmax(z) over all outputs; 1: s = sigmoid(z), every output by itself */
  int32_t group_best;       /* a group's score is the sum of its group_best largest choice scores (0 or 1: its largest) */
  float wgt_scale;          /* every weight is multiplied by this at the end (0 counts as 1) */
  float renorm_eps;         /* with renorm: wgt / (sum + renorm_eps) */
} pcs_route_params;
int pcs_moe_route(const pcs_route_params* p, void* stream);

/* The gated activation of a feed-forward: PCS_GLU_SILU  silu(g) * u;   PCS_GLU_CLAMPED_SWISH  g' = min(g, limit),
 * u' = clamp(u, -limit, limit), g' * sigmoid(alpha * g') * (u' + 1).  A NULL pointer means PCS_GLU_SILU. */
#define PCS_GLU_SILU 0
#define PCS_GLU_CLAMPED_SWISH 1
/* Activations of a feed-forward WITHOUT a gate branch (one up-projection): the weights are [n_experts, ff, width], a "gu" matrix
 * holds ff columns, and the second argument of the activation does not exist.
 *   PCS_ACT_RELU2     max(z, 0)^2            PCS_ACT_GELU_ERF   z/2 * (1 + erf(z / sqrt 2)) */
#define PCS_ACT_RELU2 2
#define PCS_ACT_GELU_ERF 3
typedef struct pcs_glu_act {
  int32_t kind;
  float alpha, limit;
} pcs_glu_act;

/* The chosen experts for a handful of rows.  Pair p = (token p / top, choice p % top), expert e = idx[p]; e >= n_experts is a
 * pass-through output and is skipped.  w_gu [n_experts, 2*ff, width] (gate rows, then up rows), w_down [n_experts, width, ff].
 *   pcs_moe_rows_up:    act[p, :] = silu(W_gate_e h) * (W_up_e h)        act `dtype` [pairs, ff]
 *   pcs_moe_rows_down:  y[p, :]  = W_down_e act[p, :]                    y fp32 [pairs, width]
 * With an activation that has no gate branch (PCS_ACT_*) w_gu is [n_experts, ff, width] and act[p, :] = act(W_up_e h). */
int pcs_moe_rows_up(const void* h, int64_t h_stride, const void* w_gu, const int32_t* idx, void* act, int n_pairs, int top, int n_experts,
                    int ff, int width, const pcs_glu_act* glu, int dtype, void* stream);
int pcs_moe_rows_down(const void* act, const void* w_down, const int32_t* idx, float* y, int n_pairs, int n_experts, int ff, int width,
                      int dtype, void* stream);

/* Many rows: pairs are sorted by expert on the device.  `plan` is int32 scratch of pcs_moe_plan_ints(n_pairs, n_experts)
 * elements; pcs_moe_plan_part(part, ...) gives the offset of part 0: the experts' cumulative row ends [n_experts] (16-byte
 * aligned), 1: per row tile (expert, first sorted row, rows), 2: the sorted pair list [n_pairs], 3: every pair's sorted row
 * [n_pairs] (-1 for a pass-through choice).  plan[0] is the number of row tiles. */
int64_t pcs_moe_plan_ints(int n_pairs, int n_experts);
int pcs_moe_plan_part(int part, int n_pairs, int n_experts);
int pcs_moe_plan(const int32_t* idx, int n_pairs, int n_experts, int32_t* plan, void* stream);
/* out[r, :] = h[sorted pair r / top, :] for the rows in use (bfloat16, width a multiple of 8): the left operand of a grouped product */
int pcs_moe_gather(const void* h, int64_t h_stride, const int32_t* plan, void* out, int n_pairs, int top, int n_experts, int width,
                   void* stream);
/* stage 0: act[sorted row, :] = silu(W_gate_e h[pair / top]) * (W_up_e h[pair / top])   (bf16 [n_pairs, ff])
 * stage 1: y[pair, :] = W_down_e act[sorted row, :]                                      (fp32 [n_pairs, width])
 * bfloat16 only; ff and width multiples of 8. */
int pcs_moe_gemm(int stage, const void* a, int64_t a_stride, const void* w, const int32_t* plan, void* out, int n_pairs, int top,
                 int n_experts, int ff, int width, const pcs_glu_act* glu, void* stream);

/* x[t] += mult * ( sum_k wgt[t,k] * (idx[t,k] < n_experts ? y[row(t*top + k)] : h[t]) + (ys ? shared_gate[t] * ys[t] : 0) )
 * row(p) = y_row ? y_row[p] : p;  y is fp32 (y_dtype PCS_F32) or `dtype`. */
typedef struct pcs_combine_params {
  float* x;                 /* [n_tokens, width] */
  const void* y;            /* [rows, width] */
  const int32_t* idx;
  const float* wgt;
  const void* h;            /* [n_tokens, h_stride] `dtype`: what pass-through outputs hand on */
  int64_t h_stride;
  const void* ys;           /* [n_tokens, ys_stride] `dtype` or NULL: the shared expert's result */
  int64_t ys_stride;
  const float* shared_gate; /* [n_tokens] or NULL (ys is added as it is) */
  float mult;
  int32_t n_tokens, width, top, n_experts, dtype, y_dtype;
  const int32_t* y_row;     /* [n_tokens * top] or NULL */
  int32_t overwrite;        /* 1: x = mult * (...) instead of x += (x need not be initialised) */
} pcs_combine_params;
int pcs_moe_combine(const pcs_combine_params* p, void* stream);

/* out[r, c] = silu(gu[r, c]) * gu[r, ff + c]     (gu `dtype` [n_rows, gu_stride], out `dtype` [n_rows, ff]) */
int pcs_silu_mul(const void* gu, int64_t gu_stride, void* out, int n_rows, int ff, int dtype, void* stream);
/* out[r, c] = glu(gu[r, c], gu[r, ff + c]) */
int pcs_glu_mul(const void* gu, int64_t gu_stride, void* out, int n_rows, int ff, const pcs_glu_act* glu, int dtype, void* stream);

/* Depth-weighted average: out[r, :] = sum_{j < n_terms} coef[j] * xs[j][row(r), :], row(r) = rows ? rows[r] : r, where xs[j] is the
 * fp32 matrix at xs + j * term_stride elements.  x_out (fp32 [n_rows, width]) may be NULL; when next_w is given,
 * h_out[r, :] = rms(out[r, :]) * (w_offset + next_w)  (`dtype`).  The sum runs over j in increasing order.
 * With y (a sublayer's result, `dtype` or fp32, [*, y_stride]) the newest term first takes its residual sum,
 * xs[n_terms - 1][row, :] += (w_offset + y_w) * rms(y[row, :]), as pcs_gate_norm_add would have done (every row at most once). */
typedef struct pcs_depthmix_params {
  const float* xs;
  int64_t term_stride;
  int32_t n_terms;
  const float* coef;        /* [n_terms] */
  const int32_t* rows;      /* [n_rows] or NULL */
  float* x_out;
  const void* next_w;       /* [width] `dtype` or NULL */
  void* h_out;              /* [n_rows, width] `dtype` */
  float w_offset, eps;
  int32_t n_rows, width, dtype;
  int32_t y_f32;            /* y is fp32 */
  const void* y;            /* or NULL */
  int64_t y_stride;
  const void* y_w;          /* [width] `dtype` */
} pcs_depthmix_params;
int pcs_depth_mix(const pcs_depthmix_params* p, void* stream);

/* Low-rank (latent) attention.  `proj` holds per token the query latent (q_rank numbers at cq_off) and the key/value latent
 * followed by the key part that is rotated (kv_rank + rot_dim numbers at ckv_off).
 *   cq_out[t]                       = rms(query latent) * cq_norm_w                              [n_tokens, q_rank]
 *   pool[slot, pos, 0:kv_rank]      = rms(key/value latent) * ckv_norm_w
 *   pool[slot, pos, kv_rank: ...]   = the rotated part turned by pos (pairs (i, i + rot_dim/2), cos and sin times rot_mult)
 * pool is [slots, cap, kv_rank + rot_dim]. */
typedef struct pcs_latent_prep_params {
  const void* proj;
  int64_t row_stride;
  int32_t cq_off, ckv_off, q_rank, kv_rank, rot_dim;
  const void* cq_norm_w;    /* [q_rank] */
  const void* ckv_norm_w;   /* [kv_rank] */
  float eps;
  const double* freqs;      /* [rot_dim / 2] */
  float rot_mult;
  void* cq_out;
  void* pool;
  int32_t cap;
  const int32_t* tok_seq;
  const int32_t* tok_pos;
  const int32_t* seq_slot;
  int32_t n_tokens, dtype;
} pcs_latent_prep_params;
int pcs_latent_prep(const pcs_latent_prep_params* p, void* stream);

/* Queries of latent attention.  q [n_tokens, H * (dim + rot_dim)], per head [dim plain | rot_dim rotated].
 *   q_lat == NULL:  the rotated part of every head is turned by the token's position in place (q_out == q) or into q_out
 *                   (same layout, plain part copied).
 *   q_lat != NULL:  q_out [n_tokens, H * (kv_rank + rot_dim)] gets per head [q_lat[t, h, :] | rotated part], where
 *                   q_lat[t, h, c] sits at q_lat + t * lat_tok_stride + h * lat_head_stride + c. */
typedef struct pcs_latent_q_params {
  const void* q;
  void* q_out;
  const void* q_lat;
  int64_t lat_tok_stride, lat_head_stride;
  int32_t n_heads, dim, rot_dim, kv_rank;
  const double* freqs;
  float rot_mult;
  const int32_t* tok_pos;
  int32_t n_tokens, dtype;
} pcs_latent_q_params;
int pcs_latent_q(const pcs_latent_q_params* p, void* stream);

/* Per-head rows for attention over expanded keys and values.  kv [n_ctx, H * (dim + vdim)]: for context token n (entry
 * ctx_seq[n], position ctx_pos[n]) the plain key parts of all heads, then the values of all heads.
 *   k_dense[b, h, pos, :] = [kv[n, h * dim ...] | pool[seq_slot[b], pos, kv_rank : kv_rank + rot_dim]]     [B, H, cap_dense, dim + rot_dim]
 *   v_dense[b, h, pos, :] = kv[n, H * dim + h * vdim ...]                                                   [B, H, cap_dense, vdim] */
typedef struct pcs_latent_expand_params {
  const void* kv;
  int64_t kv_stride;
  const void* pool;
  int32_t cap, kv_rank, rot_dim, n_heads, dim, vdim;
  void* k_dense;
  void* v_dense;
  int32_t cap_dense;
  const int32_t* ctx_seq;
  const int32_t* ctx_pos;
  const int32_t* seq_slot;
  int32_t n_ctx, dtype;
} pcs_latent_expand_params;
int pcs_latent_expand(const pcs_latent_expand_params* p, void* stream);

/* rows of the latent pool (the first `width` numbers of each) for the context tokens, as one matrix: out[n, :] = pool[seq_slot[ctx_seq[n]], ctx_pos[n], 0:width] */
int pcs_latent_gather(const void* pool, int cap, int row_width, int width, void* out, const int32_t* ctx_seq, const int32_t* ctx_pos,
                      const int32_t* seq_slot, int n_ctx, int dtype, void* stream);

/* out[t, h * vdim + c] = o[t * o_tok_stride + h * o_head_stride + c] * sigmoid(g[t * g_stride + h])       (out contiguous) */
int pcs_head_gate(const void* o, int64_t o_tok_stride, int64_t o_head_stride, const void* g, int64_t g_stride, void* out, int n_tokens,
                  int n_heads, int vdim, int dtype, void* stream);

/* Gated linear attention.  log decay per key channel: ld[t, c] = logsigmoid(sum_r a2[c, r] * a[t, r] + a2_b[c]) / tau   (fp32
 * [n_tokens, n_channels]); `a` is `dtype` [n_tokens, a_stride] with `rank` numbers per token, a2 `dtype` [n_channels, rank]. */
int pcs_gla_decay(const void* a, int64_t a_stride, const void* a2, const float* a2_b, float* ld, int n_tokens, int n_channels, int rank,
                  float tau, int dtype, void* stream);

/* Per entry and head, token by token:  S <- diag(exp(ld_t)) S + k_t v_t^T,  o_t = S^T (q_t * q_scale);  then
 * out[t, h, :] = o_t / sqrt(mean(o_t^2) + eps) * norm_w * silu(g[t, h, :])   (norm_w [vdim], shared by the heads).
 * S is fp32 [slots, heads, dim, vdim] in the slot pool; an entry whose slot holds no tokens starts from zero. */
typedef struct pcs_gla_params {
  const void* proj;         /* [n_tokens, row_stride]: q at q_off, k at k_off, v at v_off, the gate's pre-activation at g_off */
  int64_t row_stride;
  int32_t q_off, k_off, v_off, g_off;
  const float* ld;          /* [n_tokens, heads * dim] log decays */
  const void* norm_w;       /* [vdim] `dtype` */
  void* out;                /* [n_tokens, heads * vdim] `dtype` */
  float* s_pool;
  int32_t heads, dim, vdim;
  float q_scale, eps;
  const int32_t* seq_slot;
  const int32_t* seq_pos0;
  const int32_t* seq_len;
  const int32_t* seq_off;
  int32_t n_seqs, n_tokens, dtype, max_len;
  int32_t impl;             /* 0 = automatic, 1 = the kernel with the state in shared memory */
  float* o_raw;             /* fp32 scratch [n_tokens, heads * vdim] */
} pcs_gla_params;
int pcs_gla_scan(const pcs_gla_params* p, void* stream);

/* Residual sum and layer norm (weight, no bias) of the 32-bit stream.  Per row r (row(r) = rows ? rows[r] : r):
 *   x[row, :] += sum_i y_mult[i] * y[i][row, :]          (n_addends <= 3 sublayer results, `dtype` or fp32; not with `rows`)
 *   mu = mean(x[row]), var = mean((x[row] - mu)^2)        (two passes over the row, 32-bit)
 *   h1[r, :] = (x[row] - mu) / sqrt(var + eps) * w1;  h2[r, :] likewise with w2   (each may be NULL) */
typedef struct pcs_addln_params {
  float* x;                 /* [*, width] */
  const int32_t* rows;      /* [n_rows] or NULL */
  const void* y[3];
  int64_t y_stride[3];
  float y_mult[3];
  int32_t y_f32[3];
  int32_t n_addends;
  const void* w1;           /* [width] `dtype` */
  void* h1;                 /* [n_rows, width] `dtype` */
  const void* w2;
  void* h2;
  int32_t n_rows, width;
  float eps;
  int32_t dtype;
} pcs_addln_params;
int pcs_add_layer_norm(const pcs_addln_params* p, void* stream);

/* Element-wise gated recurrence whose gates read only the current token (no dependence on the state).  Per entry and channel c:
 *   z_t = sigmoid(proj[t, z_off + c]),  u_t = proj[t, x_off + c],  cand_t = u_t >= 0 ? u_t + 1/2 : sigmoid(u_t)
 *   S_t = (1 - z_t) S_(t-1) + z_t cand_t                         (32-bit; an entry whose slot holds no tokens starts from zero)
 *   out[t, c] = S_t * silu(proj[t, g_off + c])
 * A block takes 32 channels of one entry; the entry's tokens are cut into segments that are scanned side by side (each as the
 * pair (product of 1 - z, sum) of an affine map), joined in order, and scanned again from their true starts. */
typedef struct pcs_gru_params {
  const void* proj;         /* [n_tokens, row_stride] `dtype`, biases already added */
  int64_t row_stride;
  int32_t z_off, x_off, g_off, width;
  void* out;                /* [n_tokens, width] `dtype` */
  float* s_pool;            /* [slots, width] */
  const int32_t* seq_slot;
  const int32_t* seq_pos0;
  const int32_t* seq_len;
  const int32_t* seq_off;
  int32_t n_seqs, n_tokens, max_len, dtype;
} pcs_gru_params;
int pcs_gru_scan(const pcs_gru_params* p, void* stream);

/* The same recurrence in chunks of `chunk` tokens (prompts).  The step's entries are cut into chunks (an entry's last one may
 * be short); chunk c holds tokens chunk_first[c] .. chunk_first[c] + chunk_len[c] - 1 of the concatenated matrix.  With B_i the
 * running sum of the log decays inside a chunk (per key channel) and e its last token:
 *   pcs_gla_chunk_prep   qd[c, h, i, :] = q_i * q_scale * exp(B_i)        kd[c, h, i, :] = k_i * exp(B_e - B_i)     (fp32 [chunks, H, chunk, dim])
 *                        g[c, h, :] = exp(B_e)                            vf[c, h, i, :] = v_i                      (fp32; rows past the chunk are zero)
 *                        a[c, h, i, s] = sum_d q_i[d] k_s[d] exp(B_i[d] - B_s[d]) for s <= i, else 0     (fp32 [chunks, H, chunk, chunk]; every exponent <= 0)
 *   (the caller forms u[c, h] = kd[c, h]^T vf[c, h], fp32 [chunks, H, dim, vdim], with a matrix product)
 *   pcs_gla_chunk_scan   per entry, over its chunks in order: u[c] is replaced by the state S the chunk starts from, S <- g[c] * S + u[c];
 *                        S starts from the pool (zero for an entry whose slot holds no tokens) and returns there
 *   (the caller forms o[c, h] = qd[c, h] S[c, h] + a[c, h] vf[c, h], fp32 [chunks, H, chunk, vdim])
 *   pcs_gla_chunk_out    out[t, h, :] = o_t / sqrt(mean(o_t^2) + eps) * norm_w * silu(g[t, h, :]), o_t = o[tok_row[t] / chunk, h, tok_row[t] % chunk, :] */
typedef struct pcs_gla_chunk_params {
  const void* proj;
  int64_t row_stride;
  int32_t q_off, k_off, v_off, g_off;
  const float* ld;
  int32_t heads, dim, vdim, chunk;
  float q_scale, eps;
  const int32_t* chunk_first;  /* [n_chunks] */
  const int32_t* chunk_len;    /* [n_chunks] */
  int32_t n_chunks, n_tokens, dtype, n_seqs;
  float* qd;
  float* kd;
  float* g;
  float* vf;
  float* a;
  float* u;                    /* [n_chunks, H, dim, vdim]: the chunks' own sums on entry of the scan, their start states after it */
  float* s_pool;
  const int32_t* seq_slot;
  const int32_t* seq_pos0;
  const int32_t* seq_chunk0;   /* [n_seqs] first chunk of the entry */
  const int32_t* seq_chunks;   /* [n_seqs] number of its chunks */
  const float* o;              /* [n_chunks, H, chunk, vdim] */
  const int32_t* tok_row;      /* [n_tokens]: chunk index * chunk + place in the chunk */
  const void* norm_w;
  void* out;
} pcs_gla_chunk_params;
int pcs_gla_chunk_prep(const pcs_gla_chunk_params* p, void* stream);
int pcs_gla_chunk_scan(const pcs_gla_chunk_params* p, void* stream);
int pcs_gla_chunk_out(const pcs_gla_chunk_params* p, void* stream);

#ifdef __cplusplus
}
#endif
#endif
