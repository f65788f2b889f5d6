/*
 * b2l_seq.h - C ABI of libb200seq.so: sequence-mixer kernels for B200 (sm_100a) beside the quantized-LLaMA
 * library (b2l.h).  One call = one mechanism over one portion of ONE sequence: T consecutive tokens that start at
 * position pos0 of the sequence held in state slot `slot`.
 *
 * Conventions (those of b2l.h unless stated):
 *  - every pointer is a device pointer owned by the caller; calls only enqueue on `stream` (graph capturable);
 *    0 = ok, <0 = B2L_E_*, >0 = cudaError_t; b2l_seq_last_error() gives the message; no CPU fallback.
 *  - `meta` is a device int32[2] = {slot, pos0}: kernels read it on the device, so a captured decode step replays
 *    for any slot and position.
 *  - "act" tensors (projection outputs, weights, caches) have the dtype `act_dtype` (B2L_BF16 or B2L_F32);
 *    everything named f32 is float.  What a recurrence or a softmax consumes is f32 in both modes: residual,
 *    norms, angles, scores, decays, gates of a recurrence, states.
 *  - row-major, leading dimensions in elements; a "heads x size" operand is `heads` consecutive blocks of `size`.
 */
#ifndef B2L_SEQ_H_
#define B2L_SEQ_H_

#include <stddef.h>
#include <stdint.h>

#include "b2l.h"

#ifdef __cplusplus
extern "C" {
#endif

int b2l_seq_version(void);
const char* b2l_seq_last_error(void);

/* x[t, :] = table[token[t], :] * scale (f32 residual stream).  Tokens outside the table read row 0. */
int b2l_seq_embed(const void* tokens, int tokens_i64, const void* table, int act_dtype, float scale, float* x,
                  int T, int D, int vocab, b2l_stream_t stream);

/* out[t, :] = x / sqrt(mean(x^2) + eps) * w, x f32 -> out act.  `rows` (device int32[n_rows], may be null) picks
 * the rows of x to normalise (out row r <- x row rows[r]); null = rows 0..n_rows-1. */
int b2l_seq_rmsnorm(const float* x, const void* w, float eps, void* out, const int* rows, int n_rows, int D,
                    int act_dtype, b2l_stream_t stream);

/* Post-norm residual step fused with the next pre-norm:
 *   x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w_post;   if w_next: h[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w_next */
int b2l_seq_norm_add_norm(const void* y, const void* w_post, float eps, float* x, const void* w_next, void* h, int T,
                          int D, int act_dtype, b2l_stream_t stream);

/* out[t, j] = act(gu[t, j]) * gu[t, F + j]  (gated feed-forward, both halves from one product).
 * B2L_SEQ_ACT_CLAMPED_SWISH is a gated unit with clamped halves: g = min(gu[t, j], limit),
 * u = clamp(gu[t, F + j], -limit, limit), out = g * sigmoid(1.702 g) * (u + 1).  `limit` is read by it alone. */
enum { B2L_SEQ_ACT_GELU_TANH = 0, B2L_SEQ_ACT_SILU = 1, B2L_SEQ_ACT_SIGMOID = 2, B2L_SEQ_ACT_CLAMPED_SWISH = 3, B2L_SEQ_ACT_XIELU = 4,
       B2L_SEQ_ACT_NONE = 5 };
int b2l_seq_gated_act(const void* gu, int ldgu, void* out, int T, int F, int act, float limit, int act_dtype, b2l_stream_t stream);

/* out[t, j] = act(in[t, j]) for an ungated feed-forward: gelu_tanh, silu, sigmoid, or B2L_SEQ_ACT_XIELU with its two
 * coefficients coef = {a, b} (f32, on the device; from the learned numbers p, q: a = softplus(p), b = 1/2 + softplus(q)):
 *   z > 0: a z^2 + z / 2;   z <= 0: b (exp(z) - 1 - z) + z / 2.
 * `coef` is read by xIELU alone.  out may be in (in place). */
int b2l_seq_unary_act(const void* in, int ldin, void* out, int ldout, int T, int F, int act, const float* coef, int act_dtype,
                      b2l_stream_t stream);

/* Short causal convolution over time per channel, then silu, with the last taps-1 inputs of the sequence carried
 * in `state` ([n_slots][taps-1][C] act, oldest first; a fresh slot holds zeros):
 *   out[t, c] = silu(bias[c] + sum_j w[c, taps-1-j] * in[t-j, c]),  in[<0] from the state.
 * The state is advanced by the T tokens.  w is [C, taps] act, bias act or null, out f32. */
int b2l_seq_conv_silu(const void* in, int ldin, const void* w, const void* bias, void* state, const int* meta,
                      float* out, int ldout, int T, int C, int taps, int act_dtype, b2l_stream_t stream);

/* Attention operands from one stacked projection with a short causal convolution over time on every channel and a
 * rotation by position afterwards.  proj (act [T, ld]) holds q at q_off (q_heads x K), and, unless k_off < 0 (a layer
 * that attends over another layer's keys and values), k at k_off (k_heads x K) and v at v_off (n_v channels); all three
 * lie inside the C convolved channels [c_off, c_off + C), every offset even.  Per channel c of those:
 *   y[t, c] = sum_j w[c, j] * u[t - (taps - 1) + j, c]       (w act [C, taps], no bias, no activation)
 * with the last taps-1 rows of u per sequence carried in `state` ([n_slots][taps-1][C] act, oldest first, zeros in a fresh
 * slot) and advanced by the T tokens.  Then in every head of q and k the first rot_dims entries turn by the angle
 * (pos0 + t) * freq[i], pairs (2i, 2i+1) when interleaved, else (i, i + rot_dims/2), cos and sin times rot_mult.
 * q_out f32 [T, q_heads*K]; k_out act [T, k_heads*K]; v_out act [T, n_v]. */
typedef struct {
  const void* proj; int ld;
  int c_off, C, taps;
  const void* w; void* state; const int* meta;
  int q_off, q_heads, k_off, k_heads, K, v_off, n_v;
  const float* freq; int rot_dims, interleaved; float rot_mult;
  float* q_out; void* k_out; void* v_out;
  int T, act_dtype;
} b2l_seq_conv_rope_args;
int b2l_seq_conv_rope(const b2l_seq_conv_rope_args* a, b2l_stream_t stream);

/* In place on f32: every block of `size` becomes x * mult / sqrt(sum(x^2) + eps). */
int b2l_seq_unit_norm(float* x, int ld, int T, int heads, int size, float eps, float mult, b2l_stream_t stream);

/* Decay factors of a recurrence from a projection `a` (act, [T, lda], heads x size):
 *   B2L_SEQ_DECAY_EXP_SOFTPLUS: dt = softplus(a + bias), out = exp(-exp(A_log[head]) * dt); dt_out (may be null)
 *                               receives dt
 *   B2L_SEQ_DECAY_SIGMOID_ROOT: out = sigmoid(a + bias)^(1/tau)
 * bias is act [heads*size] (may be null), A_log act [heads]. */
enum { B2L_SEQ_DECAY_EXP_SOFTPLUS = 0, B2L_SEQ_DECAY_SIGMOID_ROOT = 1 };
int b2l_seq_decay(const void* a, int lda, const void* bias, const void* A_log, int mode, float tau, float* out,
                  float* dt_out, int T, int heads, int size, int act_dtype, b2l_stream_t stream);

/* Linear recurrence with a matrix state per head, S [K x V], carried per slot in f32:
 *     S <- diag(d_t) S                           (d_t per key channel, or one number per head)
 *     delta == 0:  S <- S + k_t v'_t^T
 *     delta != 0:  u = sigmoid(beta_t) (v'_t - S^T k_t);  S <- S + k_t u^T
 *     o_t = S^T q_t (+ skip[head] * v_t)
 * with v'_t = v_t * vscale[t, head] when vscale is given.  q and k have `qk_heads` heads, value head h reads
 * q/k head h / (heads / qk_heads).  `state` is [n_slots][heads][V][K] f32 (key channel fastest). */
typedef struct {
  const float* q; int ldq;
  const float* k; int ldk;
  const float* v; int ldv;
  float q_mult;                             /* o_t = q_mult * S^T q_t */
  const float* decay; int ldd; int decay_per_channel;
  const void* beta; int ldb; int delta;     /* act [T, ldb], one per head; read only when delta != 0 */
  const float* vscale; int ldvs;            /* f32 [T, heads] or null */
  const void* skip;                         /* act [heads] or null */
  float* state; const int* meta;
  float* out; int ldo;
  int T, heads, qk_heads, K, V, act_dtype;
  /* Without the delta rule a long portion may be cut into n_chunks (> 1) chunks that run in parallel: every chunk's
   * local end state and total decay first, a short combine that gives every chunk its start state, then the outputs.
   * work_state: f32 [n_chunks][heads][V][K]; work_decay: f32 [n_chunks][heads][K] (per-channel decay) or
   * [n_chunks][heads].  b2l_seq_scan_chunks() says how many chunks a portion of T tokens wants (1 = sequential). */
  float* work_state; float* work_decay; int n_chunks;
} b2l_seq_scan_args;
int b2l_seq_scan_chunks(int T, int delta);
int b2l_seq_scan(const b2l_seq_scan_args* a, b2l_stream_t stream);

/* Read-out of a recurrence: groups of `group` consecutive channels of o (f32 [T, n]) are divided by their root
 * mean square, multiplied by w (act; `w_shared` != 0: w has `group` entries used by every group, else n) and by
 * act(gate) (act [T, ldg]) and by out_mult; gate_first != 0 applies the gate before the norm. */
int b2l_seq_group_norm_gate(const float* o, int ldo, const void* w, int w_shared, const void* gate, int ldg,
                            int gate_act, int gate_first, float eps, float out_mult, void* out, int ldout, int T,
                            int n, int group, int act_dtype, b2l_stream_t stream);

/* Per-head RMS norm (weight of `size`, shared by heads) then rotation of the first rot_dims entries of each head
 * (entry i with entry i + rot_dims/2) by the angle (pos0 + t) * freq[i], cos and sin multiplied by rot_mult.
 * x act [T, ldx] -> out act or f32 [T, heads*size] (out_f32).  w may be null (no norm), rot_dims may be 0. */
int b2l_seq_headnorm_rope(const void* x, int ldx, const void* w, float eps, const float* freq, int rot_dims,
                          float rot_mult, const int* meta, void* out, int out_f32, int T, int heads, int size,
                          int act_dtype, b2l_stream_t stream);

/* Local causal softmax attention.  window == 0 (block-local): the query at position p sees the keys j <= p with
 * j / block == p / block.  window > 0 (sliding window): it sees the keys p - window + 1 .. p, and `block` (>= window)
 * is only the size of the ring.  Score s = softcap * tanh(q.k * scale / softcap) (softcap <= 0: none); weights
 * exp(s_j) / (sink + sum exp(s_j)) with sink = 1 (has_sink) or 0 (ordinary softmax); when gate is given head h's
 * output is multiplied by sigmoid(gate[t, h]), or channel c of it by sigmoid(gate[t, h*V + c]) (gate_per_channel).
 * Keys of this portion come from k_new / v_new, older ones from the ring cache ([n_slots][block][kv_heads][K or V]
 * act, entry p % block).  After the call the ring holds the portion's tokens that share the last token's block
 * (block-local) or its last `block` tokens (sliding window). */
typedef struct {
  const float* q;                 /* f32 [T, heads*K], normalised and rotated */
  const void* k_new;              /* act [T, kv_heads*K], normalised and rotated */
  const void* v_new; int ldv;     /* act [T, ldv] */
  void* cache_k; void* cache_v;
  const int* meta;
  const void* gate; int ldg;      /* act [T, ldg] or null */
  void* out; int ldo;             /* act [T, ldo] */
  float scale, softcap, out_mult;  /* out_mult scales the output (a mixing weight of a parallel branch) */
  int has_sink, block, T, heads, kv_heads, K, V, act_dtype;
  int window;                     /* 0: block-local; > 0: sliding window of that many positions */
  int gate_per_channel;           /* gate is [T, heads*V] instead of [T, heads] */
  float* work; int work_floats;   /* optional f32 work space, see b2l_seq_block_attention_work_floats */
  /* Several attention maps over the same values (maps > 1; 0 and 1 mean one): `heads` counts the maps of all query
   * heads, laid out head by head as [map 0 | map 1 | ...] of K entries each; the keys likewise have kv_heads * maps
   * heads of K entries, the values kv_heads heads of V entries.  Query map (h, m) reads key map m of its key/value head
   * and that head's values; the maps' outputs lie side by side in `out` ([T, heads * V]) for the caller to combine. */
  int maps;
  int out_f32;                    /* out is f32 [T, ldo] instead of act */
  int no_append;                  /* leave the ring as it is: the portion's keys and values are another layer's, which
                                     appends them itself */
  /* Differential read-out of two maps (maps == 2, out_f32, no gate), when diff_out is given: per real head
   *   o = a_0 - diff_lambda a_1;   diff_out[t, h*V : (h+1)*V] = o / sqrt(mean(o^2) + diff_eps) * diff_mult   (act [T, ldd])
   * `out` (f32 [T, ldo]) is then only a scratch for the maps: the few-query form merges both maps of a head in one CTA
   * and never writes it, the other forms run the read-out as a second kernel of the call. */
  void* diff_out; int ldd;
  float diff_lambda, diff_eps, diff_mult;
} b2l_seq_attn_args;
int b2l_seq_block_attention(const b2l_seq_attn_args* a, b2l_stream_t stream);
/* With few queries (decoding) the keys of a query are cut into chunks that run in parallel and are merged afterwards;
 * that form needs a work space of this many floats (0: this call does not use one).  Without `work` the call runs a
 * slower form that needs none.  The count depends on T, the head counts, V and the window or block, not on positions. */
long long b2l_seq_block_attention_work_floats(const b2l_seq_attn_args* a);

/* Differential read-out of two attention maps per head: a f32 [T, lda] holds per head [map 0 (V) | map 1 (V)];
 *   o = a0 - lambda * a1;   out[t, h*V : (h+1)*V] = o / sqrt(mean(o^2) + eps) * mult      (act [T, ldo]) */
int b2l_seq_diff_combine(const float* a, int lda, float lambda, float eps, float mult, void* out, int ldo, int T, int heads, int V,
                         int act_dtype, b2l_stream_t stream);

/* Gated recurrence on every channel by itself (minGRU): from one stacked projection proj (act [T, ld]) with the gate logits
 * at z_off, the candidate inputs at x_off and the output gate at g_off (`width` channels each, biases already added):
 *   z = sigmoid(proj_z);  c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0), u = proj_x;  S_t = (1 - z) S_(t-1) + z c
 *   out[t] = S_t * silu(proj_g)                                  (act [T, ldo]; g_off < 0: S_t itself)
 * S lives per slot in `state` ([n_slots][width] f32, zeros in a fresh slot) and is advanced by the T tokens; everything
 * after the projections is f32.  A long portion runs as n_chunks (> 1) chunks in parallel: every chunk's decay product and
 * local end state, a short pass over the chunks, then the outputs; that form needs work: f32 [n_chunks][2][width].
 * b2l_seq_mingru_chunks() says how many chunks a portion of T tokens wants (1 = sequential). */
int b2l_seq_mingru_chunks(int T);
int b2l_seq_mingru(const void* proj, int ld, int z_off, int x_off, int g_off, float* state, const int* meta, void* out, int ldo,
                   float* work, int n_chunks, int T, int width, int act_dtype, b2l_stream_t stream);

/* out[t, j] = (float) in[t, j]: act columns of a product as f32 operands of a recurrence. */
int b2l_seq_cast_f32(const void* in, int ldin, float* out, int ldout, int T, int n, int act_dtype, b2l_stream_t stream);

/* Zero one slot of a state tensor laid out [n_slots][slot_bytes]. */
int b2l_seq_zero_slot(void* state, size_t slot_bytes, int slot, b2l_stream_t stream);

/* ---- two sublayers on the same input ----
 * x[r] += y1[r] + y2[r] (act, either may be null; the sum is f32), then up to two RMS norms of the new row with weights
 * stored around w_offset: h[r] = x[r] / sqrt(mean(x[r]^2) + eps) * (w_offset + w).  w2 / h2 may be null, and so may
 * w1 / h1 (then only the sum is done).  `rows` (device int32[n_rows], may be null, only when y1 is null) picks the
 * rows of x that are normalised (out row r <- x row rows[r]). */
int b2l_seq_add_norm2(const void* y1, const void* y2, float* x, const void* w1, void* h1, const void* w2, void* h2,
                      float w_offset, float eps, const int* rows, int n_rows, int D, int act_dtype, b2l_stream_t stream);

/* z <- cap * tanh(z / cap) in place on f32 (soft cap of logits). */
int b2l_seq_softcap(float* z, size_t n, float cap, b2l_stream_t stream);

/* Partial rotation by position, any layout.  Per head (`size` entries, heads every hsx elements of x and hso of out):
 * the entries [rot_off, rot_off + rot_dims) are rotated by the angle (pos0 + t) * freq[i]: pair (2i, 2i+1) when
 * interleaved, else (i, i + rot_dims/2); (u, v) -> (u cos - v sin, v cos + u sin), cos and sin multiplied by
 * rot_mult.  Every entry is multiplied by `mult` afterwards.  x is f32 (in_f32) or act, out f32 (out_f32) or act. */
int b2l_seq_rope(const void* x, int ldx, int in_f32, const float* freq, int rot_dims, int interleaved, int rot_off, float mult,
                 float rot_mult, const int* meta, void* out, int ldo, int out_f32, int T, int heads, int size, int hsx, int hso, int act_dtype,
                 b2l_stream_t stream);

/* ---- latent attention ----
 * Keys and values of all heads are linear images of one latent vector per position; beside it one rotated key part
 * is shared by all heads.  The cache holds [latent (rank) | rotated key (rot_dim)] per position:
 * [n_slots][max_pos][rank + rot_dim] act.
 *
 * b2l_seq_latent_prep, on the f32 product proj [T, ld] of the two down-projections:
 *   cq[t]  = rmsnorm(proj[t, q_off : q_off + q_rank]) * w_q                    (act [T, q_rank])
 *   cache[slot][pos0 + t] = [ rmsnorm(proj[t, kv_off : kv_off + rank]) * w_kv | rotate(proj[t, kv_off + rank : .. + rot_dim]) ]
 * with the rotation of b2l_seq_rope on the first rot_dims entries of the rotated part (cos and sin times rot_mult). */
int b2l_seq_latent_prep(const float* proj, int ld, int q_off, int q_rank, const void* w_q, void* cq, int kv_off, int rank,
                        const void* w_kv, int rot_dim, const float* freq, int rot_dims, int interleaved, float rot_mult, float eps,
                        const int* meta, void* cache, int max_pos, int T, int act_dtype, b2l_stream_t stream);

/* Causal softmax attention with a learned sink per head over keys 0 .. pos0 + t, or, with window > 0, over the keys
 * pos0 + t - window + 1 .. pos0 + t (the query's own position and the window - 1 before it):
 *   weights exp(score_j) / (exp(sink[h]) + sum_j exp(score_j)),  score = (q . key_j[score_off:]) * scale
 *   (sink null: ordinary softmax, no sink term)
 *   out[t, h*vdim : (h+1)*vdim] = sum_j weight_j key_j[0 : vdim]
 * A key row is [A (n_a entries) | B (n_b entries)]: A belongs to a key group (row j at key_a + slot*slot_stride_a +
 * group*hska + j*ldka), B is shared by all groups (key_b + slot*slot_stride_b + j*ldkb); heads_per_group consecutive
 * heads share a group.  The query of row (t, h) is [q_a (n_a - score_off entries) | q_b (n_b entries)], f32, at
 * q_x + t*ldqx_t + h*ldqx_h.
 *   latent form:   heads_per_group = heads, A = the cached latent (n_a = vdim = rank, score_off = 0), B = the cached
 *                  rotated key; q_a is the query already multiplied by the key up-projection; out is the weighted
 *                  latent, still to be mapped to the value space.
 *   expanded form: heads_per_group = 1, A = [value_h | unrotated key_h] of every position (score_off = vdim).
 * The cache must already hold the portion's own positions (b2l_seq_latent_prep).  `splits` > 1 cuts the keys into
 * that many ranges that run in parallel and are merged afterwards; it needs work: f32 [splits][T*heads][vdim + 2].
 * The grid does not depend on the position, so a captured single-token step replays anywhere. */
typedef struct {
  const float* q_a; long long ldqa_t; long long ldqa_h;
  const float* q_b; long long ldqb_t; long long ldqb_h;
  const void* key_a; long long ldka; long long hska; long long slot_stride_a;
  const void* key_b; long long ldkb; long long slot_stride_b;
  const float* sink;               /* f32 [heads], or null */
  const int* meta;
  void* out; int ldo;              /* act [T, ldo] */
  float* work;
  float scale;
  int T, heads, heads_per_group, n_a, n_b, vdim, score_off, splits, act_dtype;
  int window;                      /* 0: every earlier position; > 0: a sliding window of that many positions */
} b2l_seq_latent_attn_args;
int b2l_seq_latent_attention(const b2l_seq_latent_attn_args* a, b2l_stream_t stream);
int b2l_seq_latent_attention_warps(int T, int heads_per_group);    /* warps per CTA that own rows: 4 rows per warp */

/* ---- mixture of experts ----
 * Router, per token, from f32 logits [T, ld] over n experts: s = softmax(logits) over the experts, or sigmoid(logits)
 * of each (score_fn); choice = s + correction (f32 [n], may be null); the n experts form `groups` equal groups of
 * neighbours, a group's score is the sum of its `group_top` largest choice scores (1: its largest), only experts of the
 * `keep` best groups can be chosen (ties to the lower group);
 * idx[t, :] = the `top` largest choice scores among them (best first, ties to the lower index);
 * weights[t, k] = weight_scale * s[idx] / (sum of the chosen s + 1e-20) when `renormalize`, else weight_scale * s[idx]. */
enum { B2L_SEQ_SCORE_SOFTMAX = 0, B2L_SEQ_SCORE_SIGMOID = 1 };
int b2l_seq_moe_route(const float* logits, int ld, const float* correction, int n, int groups, int keep, int top, int score_fn,
                      int renormalize, int group_top, float weight_scale, int* idx, float* weights, int T, b2l_stream_t stream);

/* The same with the logits computed in the kernel, for a few tokens: logits[t] = w_router h[t] (w_router act [n][D],
 * f32 accumulation), one CTA per token, one launch for product and routing. */
int b2l_seq_moe_route_fused(const void* h, int ldh, const void* w_router, const float* correction, int D, int n, int groups, int keep,
                            int top, int score_fn, int renormalize, int group_top, float weight_scale, int* idx, float* weights, int T, int act_dtype, b2l_stream_t stream);

/* Experts of a few tokens, indices read on the device.  Expert e < n_real: W_down[e] (gated(W_gate[e] h, W_up[e] h))
 * with w_gate_up act [n_real][2*ff][D] (gate rows, then up rows), w_down act [n_real][D][ff] and the gated unit of
 * b2l_seq_gated_act (`act`, `limit`); e >= n_real: h itself.
 * y[t] = sum_k weights[t, k] * expert_idx[t,k](h[t]), or, with weight_input, sum_k expert_idx[t,k](weights[t, k] * h[t])
 * (the weighted input passes through the storage type).  mid: act [T*top, ff] scratch. */
int b2l_seq_moe_experts_small(const void* h, int ldh, const void* w_gate_up, const void* w_down, const int* idx,
                              const float* weights, void* mid, void* y, int ldy, int T, int D, int ff, int n_real, int top,
                              int act, float limit, int weight_input, int act_dtype, b2l_stream_t stream);

/* Long portions: the N = T*top assignments a = t*top + k sorted by expert.  offsets int32[n_real + 1]: expert e owns
 * the sorted places offsets[e] .. offsets[e+1]-1; perm[p] = assignment at place p; inv[a] = place of assignment a
 * (-1: an identity expert).  cursor: int32[n_real + 1] scratch. */
int b2l_seq_moe_sort(const int* idx, int N, int n_real, int* offsets, int* cursor, int* perm, int* inv, b2l_stream_t stream);
/* xg[p, :] = h[perm[p] / top, :] (times row_scale[perm[p]] when row_scale, f32 [N], is given: the router's weight on
 * an expert's input) for p < *n_rows (device int32: offsets[n_real]); launched over N rows. */
int b2l_seq_moe_gather(const void* h, int ldh, const int* perm, const int* n_rows, const float* row_scale, int top, void* xg, int N,
                       int D, int act_dtype, b2l_stream_t stream);
/* y[t] = sum_k weights[t, k] * (inv[a] >= 0 ? yg[inv[a]] : h[t]); weights null: every weight is 1. */
int b2l_seq_moe_combine(const void* yg, const int* inv, const float* weights, const void* h, int ldh, void* y, int ldy, int T,
                        int D, int top, int act_dtype, b2l_stream_t stream);

/* ---- several residual streams, token-pair embedding, attention operands ----
 * Token embedding plus a hashed token-pair embedding, written into `streams` equal residual streams x [T][streams][D]:
 *   x[t, s, :] = table[token[t]] * scale + pair_table[row(t)],
 *   row(t) = (previous token * mul_prev + token[t] * mul_cur) mod buckets; the sequence's first token (position 0)
 *   reads row `buckets`, the table's last.  pair_table null: the token embedding alone.
 * prev_state: int32 [n_slots], the last token of every sequence (read for the portion's first token when pos0 > 0,
 * then set to the portion's last token). */
int b2l_seq_embed_pair(const void* tokens, int tokens_i64, const void* table, const void* pair_table, float scale, int* prev_state,
                       const int* meta, long long mul_prev, long long mul_cur, int buckets, float* x, int T, int D, int vocab,
                       int streams, int act_dtype, b2l_stream_t stream);

/* One sublayer's step on S residual streams X [rows][S][D] (f32):
 *   y given (act [rows, D], with mix f32 [S][S] indexed [from][to] and out_w f32 [S]):
 *       X_t <- sum_s mix[s, t] X_s + out_w[t] y    for all t at once from the old streams;
 *   w_next given (act [D], with in_next f32 [S] and h act [n_rows, D]):
 *       h = u / sqrt(mean(u^2) + eps) * w_next,  u = sum_s in_next[s] X_s   (of the new streams).
 * `rows` (device int32 [n_rows], may be null, only without y) picks the rows that are read: h row r <- X row rows[r].
 * With S = 1, mix = out_w = in_next = 1 this is the ordinary residual step fused with the next pre-norm. */
int b2l_seq_hc_step(const void* y, float* X, const float* mix, const float* out_w, const float* in_next, const void* w_next, void* h,
                    float eps, const int* rows, int n_rows, int D, int streams, int act_dtype, b2l_stream_t stream);
/* out[t, :] = sum_s X[t, s, :]. */
int b2l_seq_hc_sum(const float* X, float* out, int T, int D, int streams, b2l_stream_t stream);

/* ---- norms with a bias, depth-weighted residual ----
 * out[r] = norm(x[rows[r]]) (rows null: row r), x f32 [*, D] -> out act [n_rows, D]:
 *   B2L_SEQ_NORM_RMS:   x / sqrt(mean(x^2) + eps) * w (+ b when given)
 *   B2L_SEQ_NORM_LAYER: (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b      (b may be null) */
enum { B2L_SEQ_NORM_RMS = 0, B2L_SEQ_NORM_LAYER = 1 };
int b2l_seq_norm(const float* x, const void* w, const void* b, int kind, float eps, void* out, const int* rows, int n_rows, int D,
                 int act_dtype, b2l_stream_t stream);

/* One layer's residual step when the next layer reads a learned average over everything earlier layers produced.
 * hist f32 [n_hist][T][D] holds the embedding output (entry 0) and the own results of the layers so far; this call
 *   writes the layer's own result      hist[n_hist - 1] = x_in + y1 + y2        (y1, y2 act [T, D]; y2 may be null)
 *   forms the next layer's input       x_out = sum_j avg[j] * hist[j], j < n_hist   (avg f32 [n_hist]; null: hist[n_hist - 1])
 *   and, with w_next, its norm         h = norm(x_out) as b2l_seq_norm (act [T, D])
 * x_in and x_out may be the same buffer.  With y1 null only the average and the norm are done (n_hist entries exist). */
int b2l_seq_depth_step(const void* y1, const void* y2, const float* x_in, float* hist, int n_hist, const float* avg, float* x_out,
                       const void* w_next, const void* b_next, int norm_kind, float eps, void* h, int T, int D, int act_dtype,
                       b2l_stream_t stream);

/* z <- z * mult in place on f32 (a constant scale of the logits). */
int b2l_seq_scale(float* z, size_t n, float mult, b2l_stream_t stream);

/* Attention operands from one stacked projection row proj[t] (act [T, ld]) with q at q_off (heads x K), k at k_off
 * (kv_heads x K) and v at v_off (kv_heads x V):
 *   q_out (f32 [T, heads*K]), k_out (act [T, kv_heads*K]): RMS norm with eps (whole_row: over all entries of the
 *   projection at once, weight of heads*K resp. kv_heads*K entries; else per head, weight of K entries shared by the
 *   heads; null weight: no norm), then rotation of the first rot_dims entries of each head (entry i with entry
 *   i + rot_dims/2) by the angle (pos0 + t) * freq[i], cos and sin multiplied by rot_mult;
 *   v_out (act [T, kv_heads*V]) = (1 - lambda) v + lambda v_first when v_first (act [T, ldvf]) is given; lambda is a
 *   device scalar (act).  Without v_first nothing is written to v_out. */
typedef struct {
  const void* proj; int ld; int q_off, k_off, v_off;
  const void* q_norm; const void* k_norm; int whole_row; float eps;
  const float* freq; int rot_dims; float rot_mult;
  const int* meta;
  float* q_out; void* k_out;
  const void* v_first; int ldvf; const void* lambda; void* v_out;
  int T, heads, kv_heads, K, V, act_dtype;
} b2l_seq_qkv_prep_args;
int b2l_seq_qkv_prep(const b2l_seq_qkv_prep_args* a, b2l_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B2L_SEQ_H_ */
