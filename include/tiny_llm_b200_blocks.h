/*
 * tiny_llm_b200_blocks.h - C ABI of libtiny_llm_b200_blocks.so: building blocks for decoder layers with
 * unquantised (bf16 or fp32) weights on B200 (sm_100a): row-wise norms with a residual stream kept in fp32,
 * rotary positions in both pair layouts, paged latent (low-rank) key/value storage, latent attention with an
 * optional sliding window over ragged batches, gated activations and a top-k mixture-of-experts feed-forward.
 *
 * Conventions are those of tiny_llm_b200.h: plain device pointers and sizes, the caller owns every buffer, a
 * launcher never allocates, frees or synchronises and enqueues on `stream` (a cudaStream_t passed as void*);
 * 0 on success, a negative TL_E* code otherwise with the text in tlb_last_error().  `dtype` (TL_F32 | TL_BF16)
 * names the storage type of activations, weights and the cache; sums, norms, softmax, router logits and the
 * residual stream are fp32 in both.
 *
 * A ragged batch is a flat list of T tokens; token t belongs to sequence row tok_seq[t] of the step's block
 * table and sits at position tok_pos[t] of that sequence.
 */
#ifndef TINY_LLM_B200_BLOCKS_H
#define TINY_LLM_B200_BLOCKS_H

#include <stddef.h>
#include <stdint.h>

#include "tiny_llm_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

int tlb_abi_version(void);
const char *tlb_last_error(void);
long long tlb_launch_count(void);

/* x32[t,:] = table[ids[t],:] (fp32 residual stream) and h[t,:] = the same row in `dtype`. */
int tlb_embed_rows(const int32_t *ids, const void *table, float *x32, void *h, int tokens, int vocab, int dim, int dtype,
                   void *stream);

/* Row-wise RMS norm with optional layer scale and residual accumulation:
 *   n = y / sqrt(mean(y^2) + eps) * (w + weight_offset)          (* scale, if scale != NULL)
 *   residual != NULL: residual += n (fp32, in place), h = residual rounded to `dtype` (if h != NULL)
 *   residual == NULL: h = n rounded to `dtype`.
 * y is fp32 when y_is_f32, else `dtype`; w and scale are `dtype`. */
int tlb_norm_residual(const void *y, int y_is_f32, const void *w, float weight_offset, const void *scale, float eps, float *residual,
                      void *h, int rows, int dim, int dtype, void *stream);

/* End of a sublayer, fused with the next norm: residual += a (+ b, if b != NULL) in fp32, then, if w != NULL,
 * h = residual / rms(residual) * w rounded to `dtype`.  a_row != 0: `a` is one row [dim] added to every row. */
int tlb_add_norm(float *residual, const float *a, int a_row, const float *b, const void *w, float eps, void *h, int rows, int dim, int dtype,
                 void *stream);

/* y = coef * (a / rms(a) * wa + b / rms(b) * wb); a, b, y fp32 [rows, dim], wa, wb `dtype` [dim]. */
int tlb_norm_mix2(const float *a, const void *wa, const float *b, const void *wb, float coef, float eps, float *y, int rows, int dim, int dtype,
                  void *stream);

/* Rotary positions, in place, on `dims` entries starting at `first` within every head of x [rows, heads] (strides in
 * elements).  interleaved = 0: pair (i, i + dims/2); 1: pair (2i, 2i+1).  angle = tok_pos[row] * base^(-2i/dims) / factor
 * (factor 1 = none: linear scaling of the positions). */
int tlb_rope_rows(void *x, long long row_stride, long long head_stride, int first, int heads, int dims, int interleaved, double base,
                  double factor, const int32_t *tok_pos, int rows, int dtype, void *stream);
/* The same angles as fp32 tables cos_out, sin_out [rows, dims / 2], for kernels that rotate in fp32 on their way into a
 * recurrence (tlb_decay_scan). */
int tlb_rope_table(const int32_t *tok_pos, int rows, int dims, double base, double factor, float *cos_out, float *sin_out, void *stream);

/* Latent cache append: for every token, the first `rank` entries of down[t,:] are RMS-normed (plain weight) and the last
 * `rot` entries rotated by the token's position; both are stored at the token's slot of slab [pages, page_size, rank+rot]
 * found through block_table [*, max_pages] (row tok_seq[t], page tok_pos[t] / page_size). */
int tlb_latent_append(const void *down, const void *norm_w, float eps, int rank, int rot, int rot_dims, int interleaved, double base,
                      const int32_t *tok_pos, const int32_t *tok_seq, const int32_t *block_table, int max_pages, int num_pages,
                      int page_size, void *slab, int tokens, int dtype, void *stream);

/* The append with two more things for a fused q|dkv projection: the token's row of `down` is down_stride elements apart
 * (it may be a slice of a wider row), and, when q != NULL, the same launch rotates `rot_dims` entries from q_first in each
 * of q_heads query heads of q[t,:] (q_stride / q_head_stride in elements) in place, with the angles of the shared key part. */
int tlb_latent_prepare(const void *down, long long down_stride, const void *norm_w, float eps, int rank, int rot, int rot_dims, int interleaved,
                       double base, const int32_t *tok_pos, const int32_t *tok_seq, const int32_t *block_table, int max_pages, int num_pages,
                       int page_size, void *slab, void *q, long long q_stride, int q_heads, int q_head_stride, int q_first, int tokens, int dtype,
                       void *stream);

/* Latent (absorbed multi-query) attention over the paged latent cache.  Query row (t, h) is the concatenation of
 * q_lat[t,h,0:rank] and q_rot[t,h,0:rot] (two pointers with token / head strides in elements); key j of the token's
 * sequence is slab row j (rank + rot entries), value j its first `rank` entries.  Token t sees keys j <= tok_pos[t] and,
 * with window > 0, tok_pos[t] - j < window.  out[t,h,0:rank] = softmax(scale * q.k) . values.
 * tiles [num_tiles, 3] int32: first flat token, token count (1..TLB_ATTENTION_TILE_TOKENS, consecutive positions of one
 * sequence), block-table row. */
#define TLB_ATTENTION_TILE_TOKENS 4
int tlb_latent_attention(const void *q_lat, long long ql_token, long long ql_head, const void *q_rot, long long qr_token,
                         long long qr_head, const void *slab, int num_pages, int page_size, int rank, int rot,
                         const int32_t *block_table, int max_pages, const int32_t *tiles, int num_tiles, const int32_t *tok_pos,
                         int heads, int window, float scale, void *out, long long o_token, long long o_head, const float *sink, int dtype,
                         void *stream);
/* sink [heads] fp32 (or NULL): one more term exp(sink[h]) in head h's softmax denominator, without a key or a value and
 * not scaled. */

/* The same on the tensor cores, for the bf16 cache: 32 query rows per CTA = tile_tokens consecutive tokens x min(heads, 32)
 * heads, with tile_tokens = tlb_latent_attention_mma_tile_tokens(heads) the most tokens a tile may hold.  Needs
 * rank <= 512, (rank + rot) % 8 == 0, page_size % 32 == 0 (tlb_latent_attention_mma_supported). */
int tlb_latent_attention_mma_tile_tokens(int heads);
int tlb_latent_attention_mma_supported(int rank, int rot, int page_size);
int tlb_latent_attention_mma(const void *q_lat, long long ql_token, long long ql_head, const void *q_rot, long long qr_token,
                             long long qr_head, const void *slab, int num_pages, int page_size, int rank, int rot,
                             const int32_t *block_table, int max_pages, const int32_t *tiles, int num_tiles, const int32_t *tok_pos,
                             int heads, int window, float scale, void *out, long long o_token, long long o_head, int splits,
                             void *workspace, size_t workspace_bytes, const float *sink, void *stream);
/* splits > 1 cuts every tile's key range over that many CTAs (flash decoding: few query rows, long contexts) and a second
 * launch merges the partial sums; workspace: tlb_latent_attention_mma_workspace(...) bytes, no initialisation needed. */
size_t tlb_latent_attention_mma_workspace(int num_tiles, int heads, int rank, int splits);

/* Grouped-query softmax attention over a paged cache whose row (one token) is [kv_heads * dk keys | kv_heads * dv values].
 * q [T, heads, dk] and out [T, heads, dv] are views with token / head strides in elements.  Token t sees key j <= tok_pos[t]
 * and, mask 1: tok_pos[t] - j < mask_size (sliding window); mask 2: j / mask_size == tok_pos[t] / mask_size (chunks counted
 * from position 0); mask 0: all.  score = scale * q.k, then softcap * tanh(score / softcap) when softcap > 0; sink != 0 adds
 * exp(0) to the softmax's denominator; gate != NULL multiplies head h's output by sigmoid(gate[t * g_token + h]).
 * tiles [num_tiles, 3] as for latent attention, cut to at most tlb_paged_attention_tile_tokens(heads, kv_heads) tokens. */
int tlb_paged_attention_tile_tokens(int heads, int kv_heads);
int tlb_paged_attention(const void *q, long long q_token, long long q_head, const void *slab, int num_pages, int page_size, int dk, int dv,
                        int heads, int kv_heads, const int32_t *block_table, int max_pages, const int32_t *tiles, int num_tiles,
                        const int32_t *tok_pos, int mask, int mask_size, float scale, float softcap, int sink, const void *gate,
                        long long g_token, void *out, long long o_token, long long o_head, const float *head_bias, int weights, int dtype,
                        void *stream);
/* head_bias [heads] fp32 (or NULL): with sink != 0 the sink's term is exp(head_bias[h]) instead of exp(0).  weights 1: no
 * softmax, a visible key weighs sigmoid(score + head_bias[h]) and nothing is normalised over the keys (no sink, no cap). */
/* The same on the tensor cores, for the bf16 cache: 32 query rows per CTA = tile_tokens consecutive tokens x the query heads
 * of one key/value head (up to 32), tile_tokens = tlb_paged_attention_mma_tile_tokens(heads, kv_heads) the most tokens a tile
 * may hold.  Needs dk, dv multiples of 8 up to 256 and page_size % 32 == 0 (tlb_paged_attention_mma_supported). */
int tlb_paged_attention_mma_tile_tokens(int heads, int kv_heads);
int tlb_paged_attention_mma_supported(int dk, int dv, int kv_heads, int page_size);
int tlb_paged_attention_mma(const void *q, long long q_token, long long q_head, const void *slab, int num_pages, int page_size, int dk, int dv,
                            int heads, int kv_heads, const int32_t *block_table, int max_pages, const int32_t *tiles, int num_tiles,
                            const int32_t *tok_pos, int mask, int mask_size, float scale, float softcap, int sink, const void *gate,
                            long long g_token, void *out, long long o_token, long long o_head, int splits, void *workspace,
                            size_t workspace_bytes, const float *head_bias, int weights, void *stream);
/* splits > 1 cuts every tile's key range over that many CTAs (few query rows, long key ranges) and a second launch merges the
 * partial sums; workspace: tlb_paged_attention_mma_workspace(...) bytes, no initialisation needed. */
size_t tlb_paged_attention_mma_workspace(int num_tiles, int heads, int kv_heads, int dv, int splits);
/* Before that attention: per-head RMS norm (plain weight [dk]) of the queries in place (q_norm != NULL) and of the keys
 * (k_norm != NULL), and the token's keys and values stored at its slot of the cache (k != NULL). */
int tlb_kv_prepare(void *q, long long q_token, long long q_head, int heads, const void *q_norm, const void *k, long long k_token, long long k_head,
                   const void *v, long long v_token, long long v_head, int kv_heads, int dk, int dv, const void *k_norm, float eps,
                   const int32_t *tok_pos, const int32_t *tok_seq, const int32_t *block_table, int max_pages, int num_pages, int page_size,
                   void *slab, int tokens, int dtype, void *stream);

/* The same step for attention whose queries and keys are RMS-normed over the WHOLE projection (all heads of a token as one
 * row; q_norm [heads * dk], k_norm [kv_heads * dk], NULL = no norm) and then rotated on the first rot_dims entries of every
 * head (pairs (2i, 2i+1) if interleaved, else (i, i + rot_dims/2); rot_dims 0 = no rotation): q [T, heads * dk] rows q_token
 * apart, changed in place; k [T, kv_heads * dk] and v [T, kv_heads * dv] (NULL: queries only) go to the token's slot. */
int tlb_qk_whole_prepare(void *q, long long q_token, int heads, const void *q_norm, const void *k, long long k_token, const void *v, long long v_token,
                          int kv_heads, int dk, int dv, const void *k_norm, float eps, int rot_dims, int interleaved, double base, const int32_t *tok_pos,
                          const int32_t *tok_seq, const int32_t *block_table, int max_pages, int num_pages, int page_size, void *slab,
                          const float *rope_cos, const float *rope_sin, int tokens, int dtype, void *stream);
/* rope_cos, rope_sin [T, rot_dims / 2] fp32 (tlb_rope_table of this step's tokens), or NULL: the kernel evaluates the angles itself. */

/* Linear attention with a decay, state in fp32 slots.  Per sequence and head S [dk, dv]:
 *   alpha = sigmoid(z + z_bias)^(1 / tau) per key channel, or (head_decay != NULL; z may be NULL) the fixed head_decay[head];
 *   S <- diag(alpha) S + k v^T;  out = S^T (q_scale * q)
 * rope_dims > 0: the first rope_dims entries of every head of q and k are rotated first, in fp32, by the angles tabulated
 * per flat token in rope_cos, rope_sin [T, rope_dims / 2] (pairs (2i, 2i+1) if rope_interleaved, else (i, i + rope_dims/2)).
 * seq_info [num_seqs, 4] int32: first flat token, token count, position of the first token, state slot.  A sequence at
 * position 0 starts from zero; the slot (state + slot * slot_stride floats, [heads, dk, dv]) is written after the last
 * token.  q, k [T, heads, dk], v [T, heads, dv] views (strides in elements), z [T, heads * dk] fp32 rows z_token apart,
 * z_bias `dtype` or NULL, out [T, heads, dv] fp32 contiguous.  dk <= 256.
 * max_tokens_per_seq = the largest token count in seq_info (known to the host).  Up to TLB_DECAY_SCAN_SEGMENT tokens a
 * sequence is walked in one go.  Longer portions are cut at the multiples of the segment length in absolute positions and
 * run in three launches (every segment's local end state and decay product from a zero state; the segments' start
 * states by walking those in order; outputs per segment), which needs tlb_decay_scan_workspace(...) bytes. */
#define TLB_DECAY_SCAN_SEGMENT 64
size_t tlb_decay_scan_workspace(int num_seqs, int max_tokens_per_seq, int heads, int dk, int dv);
int tlb_decay_scan(const void *q, long long q_token, long long q_head, const void *k, long long k_token, long long k_head, const void *v,
                   long long v_token, long long v_head, const float *z, long long z_token, const void *z_bias, float tau, const float *head_decay,
                   const float *rope_cos, const float *rope_sin, int rope_dims, int rope_interleaved, float q_scale, int heads,
                   int dk, int dv, const int32_t *seq_info, int num_seqs, int max_tokens_per_seq, float *state, long long slot_stride,
                   int num_slots, float *out, void *workspace, size_t workspace_bytes, int decay_kind, const void *a_log, const void *bonus,
                   int qk_heads, const void *skip, int dtype, void *stream);
/* decay_kind 0: as above.  2: alpha = exp(-exp(z + z_bias)) per key channel.  3: one decay per head and token,
 * alpha = exp(-exp(a_log[h]) dt), dt = softplus(z[t, h] + z_bias[h]) (z [T, heads]), and the token's key is multiplied by dt
 * (a discretised state-space step; a_log [heads] in `dtype`).  qk_heads (0 = heads): q and k have that many heads, head h
 * reads h / (heads / qk_heads).  skip [heads] (`dtype`, or NULL): out += skip[h] v.  bonus [heads, dk] (`dtype`, or NULL): the
 * read-out comes before the update and weighs the token's own k v^T by it, out = (S + diag(bonus) k v^T)^T q, then S is
 * updated. */
/* out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * act(gate[t, h, :]) (w NULL = no weight; gate rows g_token apart, NULL = no
 * gate; act 0 = the gate as it is, 1 = silu, 2 = sigmoid); o fp32 [tokens, heads, dv], out `dtype` [tokens, heads * dv].
 * wide_weight: w is [heads * dv], each head its own part, instead of [dv]; gate_first: the gate multiplies o BEFORE the
 * norm, out = n / rms(n) * w with n = o * act(gate). */
int tlb_head_norm_gate(const float *o, const void *w, float eps, const void *gate, long long g_token, int act, void *out, int tokens, int heads,
                       int dv, int wide_weight, int gate_first, int dtype, void *stream);

/* Gated delta rule, state in fp32 slots.  Per sequence and head S [dk, dv], token by token:
 *   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  out = S^T q
 *   g = exp(-exp(a_log[head]) * softplus(a + dt_bias)), beta = sigmoid(b); q, k made unit vectors per head
 *   (x / sqrt(sum x^2 + unit_eps)), q times q_scale.  per_channel: a [T, heads * dk] and dt_bias [heads * dk] give one decay
 *   per key channel; else a [T, heads], dt_bias [heads] one per head.  a is fp32 (a_is_f32) or `dtype`, rows a_token apart.
 * q, k [T, key_heads, dk] (head h reads key head h / (heads / key_heads)), v [T, heads, dv], beta [T, heads] rows b_token apart:
 * views in `dtype`, strides in elements.  seq_info, state slots and out as for tlb_decay_scan.  dk <= 256.
 * max_tokens_per_seq = the largest token count in seq_info.  Up to TLB_DELTA_SCAN_SEGMENT tokens a sequence is walked in
 * one go.  Longer portions are cut at the multiples of the segment length in absolute positions and run in three launches
 * (every segment's end state from zero and its transition matrix [dk, dk], by the same walk started from the identity; the
 * segments' start states in order; outputs per segment), which needs tlb_delta_scan_workspace(...) bytes. */
#define TLB_DELTA_SCAN_SEGMENT 64
size_t tlb_delta_scan_workspace(int num_seqs, int max_tokens_per_seq, int heads, int dk, int dv);
int tlb_delta_scan(const void *q, long long q_token, long long q_head, const void *k, long long k_token, long long k_head, const void *v,
                   long long v_token, long long v_head, const void *beta, long long b_token, const void *a, int a_is_f32, long long a_token,
                   int per_channel, const void *a_log, const void *dt_bias, float q_scale, float unit_eps, int heads, int key_heads, int dk, int dv,
                   const int32_t *seq_info, int num_seqs, int max_tokens_per_seq, float *state, long long slot_stride, int num_slots, float *out,
                   void *workspace, size_t workspace_bytes, int dtype, void *stream);
/* Short causal convolution along every sequence, per channel: y[t, c] = act(bias[c] + sum_i taps[c, K-1-i] x[t-i, c]) (act 1 =
 * silu, 0 = none; bias NULL = none; add_input: x[t, c] is added before the activation), zeros before position 0.  x [T, channels] rows x_token apart, taps [channels, K] (K <= 16), y [T, channels]
 * contiguous.  The K-1 inputs before a step's first token live in the sequence's state slot (state + slot * slot_stride
 * floats, [channels, K-1], oldest first) and are replaced by the step's last ones. */
int tlb_short_conv(const void *x, long long x_token, const void *taps, const void *bias, int add_input, int channels, int num_taps, int act,
                   const int32_t *seq_info, int num_seqs, int max_tokens_per_seq, float *state, long long slot_stride, int num_slots, void *y, int dtype, void *stream);

/* out = act(x) elementwise over [rows, width]; act 0 = silu, 1 = gelu (tanh form), 2 = squared relu, 4 = tanh. */
int tlb_act_rows(const void *x, void *out, int rows, int width, int act, int dtype, void *stream);
/* x <- cap * tanh(x / cap), fp32 [rows, width] in place. */
int tlb_softcap_rows(float *x, int rows, int width, float cap, void *stream);
/* dst[r, 0:dim] = src[r, :] rounded to `dtype`; dst rows dst_stride elements apart. */
int tlb_cast_rows(const float *src, void *dst, long long dst_stride, int rows, int dim, int dtype, void *stream);

/* out[t, j] = act(gu[t, j]) * gu[t, width + j]; act 0 = silu, 1 = gelu (tanh form). */
int tlb_gated_act(const void *gu, void *out, int rows, int width, int act, float limit, float slope, int dtype, void *stream);
/* act 3: g = min(gate, limit), u = clamp(up, -limit, limit), out = g sigmoid(slope g) (u + 1). */

/* n residual streams xs [rows, n, dim] fp32 around a sublayer, n <= 8.  With write_w (mix [n, n] indexed [from, to], then
 * out [n]; fp32 on the device) and the sublayer's output y [rows, dim] fp32 (+ y_bias [dim] in `dtype`):
 *     x_t <- sum_s mix[s, t] x_s + out[t] (y + y_bias); the right-hand side reads the streams as they were before the call.
 * With read_w (in [n], then the norm's one weight g): h = rms_norm(sum_s in[s] x_s) * g, rounded to `dtype`.  x0 [rows, dim]
 * fp32: every stream starts as that row (the embedding) instead of being read.  Either half may be absent. */
int tlb_streams_step(float *xs, const float *x0, const float *y, const void *y_bias, const float *write_w, const float *read_w, float eps, void *h,
                     int rows, int streams, int dim, int dtype, void *stream);
/* Token shift: out[i, t, :] = h[t] + (h[t-1] - h[t]) * mu[i] for i < parts <= 8 (mu [parts, dim]); h[-1] is zero at position
 * 0 and the sequence's slot (state + slot * slot_stride, fp32 [dim]) otherwise; the slot then takes the step's last row.
 * h rows h_token apart; out [parts] blocks out_part elements apart, each [T, dim]. */
int tlb_shift_mix(const void *h, long long h_token, const void *mu, int parts, int dim, const int32_t *seq_info, int num_seqs, int max_tokens_per_seq,
                  float *state, long long slot_stride, int num_slots, void *out, long long out_part, int dtype, void *stream);

/* Router: logits = W h + b in fp32 (h, W, b stored in `dtype`; b may be NULL), the `top` largest per token (lower index
 * wins a tie).  scoring 0: weights = softmax over the chosen logits; 1: weights = sigmoid of each chosen logit, not
 * renormalised; 2: scores = softmax over ALL logits, the choice is made by score + choice_bias (`dtype` [experts] or NULL),
 * weights = the chosen scores / (their sum + 1e-20) * weight_scale.  idx [tokens, top] int32, gate [tokens, top] fp32. */
int tlb_moe_route(const void *h, const void *w, const void *b, int tokens, int dim, int experts, int top, int scoring, const void *choice_bias,
                  float weight_scale, int32_t *idx, float *gate, int dtype, void *stream);

/* Rows per expert tile of the grouped products: 32, or 64 for the tensor-core kernels (bf16, reduction length % 8 == 0)
 * when experts get many rows (half the weight traffic per row). */
#define TLB_MOE_TILE_ROWS 32
/* upper bound of sorted rows (pairs grouped by expert, every group padded to whole tiles) */
long long tlb_moe_max_rows(int tokens, int top, int experts, int tile_rows);
/* Group the (token, choice) pairs by expert: sorted_pair [max_rows] (pair id or -1), tile_expert [max_rows / tile_rows],
 * counters [2] = {tiles in use, rows in use}.  One launch, no host involvement. */
int tlb_moe_sort(const int32_t *idx, int tokens, int top, int experts, int tile_rows, int32_t *sorted_pair, int32_t *tile_expert,
                 int32_t *counters, void *stream);
/* inter[row, :] = act(Wg[e] h[token(row)]) * (Wu[e] h[token(row)]); Wg, Wu [experts, ff, dim]; inter [max_rows, ff]. */
int tlb_moe_gate_up(const void *h, const void *wg, const void *wu, const int32_t *sorted_pair, const int32_t *tile_expert,
                    const int32_t *counters, int tokens, int top, int experts, int tile_rows, int dim, int ff, int act, void *inter,
                    int dtype, void *stream);
/* Experts without a gate: inter[row, :] = act(Wu[e] a[src(row)]) with a = h (token rows, rows_are_pairs = 0) or one row per
 * (token, choice) pair (rows_are_pairs = 1).  act 0 = silu, 1 = gelu (tanh form), 2 = squared relu. */
int tlb_moe_up(const void *a, const void *wu, const int32_t *sorted_pair, const int32_t *tile_expert, const int32_t *counters, int tokens,
               int top, int experts, int tile_rows, int dim, int ff, int act, int rows_are_pairs, void *inter, int dtype, void *stream);
/* out[t * top + k, :] = gate[t, k] * h[t, :] rounded to `dtype`: inputs of experts whose weight multiplies the input. */
int tlb_moe_scale_rows(const void *h, const float *gate, void *out, int tokens, int top, int dim, int dtype, void *stream);
/* pair_out[pair, :] = Wd[e] inter[row, :] (fp32); Wd [experts, dim, ff]. */
int tlb_moe_down(const void *inter, const void *wd, const int32_t *sorted_pair, const int32_t *tile_expert, const int32_t *counters,
                 int tokens, int top, int experts, int tile_rows, int dim, int ff, float *pair_out, int dtype, void *stream);
/* y[t,:] = sum_k gate[t,k] * pair_out[t*top+k,:] (+ shared[t,:] if shared != NULL, stored in `dtype`), fp32, in choice order;
 * gate == NULL: every weight is 1.  idx != NULL: a choice with idx[t,k] >= experts is an identity expert (the router has
 * more outputs than there are experts): its output is the token's input h[t,:] (`dtype`), and the grouped products, given
 * `experts` as their count, skip it. */
int tlb_moe_combine(const float *pair_out, const float *gate, const void *shared, const int32_t *idx, int experts, const void *h, float *y,
                    int tokens, int top, int dim, int dtype, void *stream);

/* Row-wise arg-max of fp32 logits [rows, vocab] (lowest index wins a tie). */
int tlb_argmax_rows(const float *logits, int32_t *out, int rows, int vocab, void *stream);

#ifdef __cplusplus
}
#endif
#endif
