/* C ABI of libwf_seq.so: the serving engine for sequence models built as a stack of heterogeneous layers (an attention or a recurrent
 * mixer, then an optional routed feed-forward) — paged caches, fixed-size per-sequence state slots, ragged steps that mix prompt portions
 * with single decoded tokens.  Same conventions as wf_bitnet.h: plain pointers and sizes, int status (0 ok, -1 invalid argument,
 * -2 unsupported, -3 CUDA error), wf_last_error() has the text; nothing throws, nothing prints. */
#ifndef WF_SEQ_H
#define WF_SEQ_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define WF_SEQ_F32 0
#define WF_SEQ_BF16 1

#define WF_SEQ_LATENT_ATTENTION 0  /* sliding-window attention over a cached low-rank latent + one shared rotated key part */
#define WF_SEQ_DELTA 1             /* gated delta rule with short convolutions */
#define WF_SEQ_GQA_ATTENTION 2     /* grouped-query softmax attention over cached per-head keys and values */
#define WF_SEQ_SSD 3               /* state-space recurrence with one scalar decay per head (short convolution, gated grouped norm) */
#define WF_SEQ_MINGRU 4            /* element-wise gated recurrence: gate and candidate read only the current token */
#define WF_SEQ_MLSTM 5             /* matrix memory with exponential input gate, sigmoid forget gate and a running maximum of the log gates */

/* how a layer wraps its sublayers */
#define WF_SEQ_BLOCK_SANDWICH 0    /* x += norm_b(sub(conv(norm_a(x)))): grouped norms before and after, input convolution with carried tail */
#define WF_SEQ_BLOCK_POST 1        /* x += residual_mult * gain * rms(sub(x)): the sublayer reads the stream, ONE gain per norm */
#define WF_SEQ_BLOCK_PARALLEL 2    /* x += mixer(norm1(x)) + ff(norm2(x)): both branches read the same stream, each behind its own weighted norm */

/* feed-forward kinds (wf_seq_layer.has_ff) and gated activations (ff_act) */
#define WF_SEQ_FF_NONE 0
#define WF_SEQ_FF_ROUTED 1
#define WF_SEQ_FF_DENSE 2
#define WF_SEQ_ACT_SILU 0          /* silu(g) * u */
#define WF_SEQ_ACT_CLAMPED 1       /* g = min(g, limit), u = clamp(u, -limit, limit); g * sigmoid(1.702 g) * (u + 1) */
#define WF_SEQ_ACT_GELU_TANH 2     /* gelu(g) * u, gelu in its tanh form */
#define WF_SEQ_ACT_RELU2 3         /* relu(u)^2, no gate: the dense feed-forward has 'mlp.up' and 'mlp.down' only */

/* wf_seq_layer.qk_norm of grouped-query attention */
#define WF_SEQ_QKNORM_NONE 0
#define WF_SEQ_QKNORM_UNIT 1       /* each head divided by its root mean square */
#define WF_SEQ_QKNORM_HEAD 2       /* the same, times a weight vector of the head size shared by all heads (tensors mix.q.norm, mix.k.norm) */
#define WF_SEQ_QKNORM_FULL 3       /* RMS norm over the whole projection before the split into heads, weight of that size */

typedef struct wf_seq_layer {
    int type;
    int heads, dim, vdim;          /* both mixers: heads, query/key size per head (unrotated part for latent attention), value size */
    /* latent attention */
    int rot_dim, kv_rank, window, rope_dims;
    float scale, rope_base;
    /* delta */
    int kv_heads, conv;
    /* feed-forward: has_ff = WF_SEQ_FF_*; dense uses ff, ff_act, ff_limit only */
    int has_ff, experts, identity, top, groups, keep, ff;
    /* grouped-query attention: kv_heads key/value heads shared by heads / kv_heads query heads each.  qk_norm / v_norm: queries and keys /
     * values divided by their root mean square per head; proj_bias: q, k, v and the output projection have biases; head_gate: head h's
     * output times sigmoid(W_g x)_h; dist_exp > 0: score -= 2^(-dist_exp (h + 1) / heads) * (i - j); kv_from >= 0: no key / value
     * projections, the layer reads that earlier layer's cache.  window as above (keys i - window < j <= i). */
    int qk_norm, v_norm, proj_bias, head_gate, kv_from;
    float dist_exp;
    /* feed-forward details */
    int ff_act;                    /* WF_SEQ_ACT_* of the experts (and of a dense feed-forward) */
    float ff_limit;
    int router_act;                /* 0 softmax over the experts, 1 sigmoid of each */
    int group_top;                 /* a group's score = sum of its group_top largest choice scores (<= 1: the largest) */
    int router_norm;               /* 1: the chosen scores are divided by their sum (+ 1e-20) */
    float router_scale;            /* the weights are multiplied by this (0 is read as 1) */
    int shared_ff;                 /* > 0: a shared expert of this size runs for every token, times sigmoid(w_sg x) */
    float shared_limit;
    /* grouped-query attention, further: rope_dims > 0 rotates the first rope_dims entries of every query and key head (after the norm;
     * the cache holds rotated keys), pairs (2i, 2i + 1) when rope_interleaved else (i, i + rope_dims / 2), angle pos * rope_base^(-2i / rope_dims).
     * chunk > 0: key j is visible to query i only when floor(i / chunk) == floor(j / chunk) (besides j <= i and the window).
     * softcap > 0: score <- softcap * tanh(score / softcap) after the scale.  rel_rows > 0: a learned bias rel[bucket(i - j), h] (tensor
     * mix.rel [rel_rows, heads]) is added after the cap; bucket(n) = n below rel_rows / 2, then logarithmic steps that reach the last
     * row at distance rel_far.  sink: the softmax denominator carries an extra 1 (a key with score 0 and no value).
     * qk_norm: WF_SEQ_QKNORM_*.  proj_bias: 1 = q, k, v and output biases, 2 = q, k, v only.  head_gate: 1 = one sigmoid gate per head
     * (mix.g [heads, W]), 2 = one per output element (mix.g [heads * vdim, W]). */
    int rope_interleaved, chunk, rel_rows, sink;
    float softcap, rel_far;
    /* delta rule, further: decay_channels = 1: one decay per head AND key channel (the decay projection has heads * dim outputs, dt_bias
     * that many entries, A_log stays per head).  decay_rank / gate_rank > 0: that projection is a product of two matrices
     * (mix.a1 [rank, W], mix.a2 [outputs, rank]; mix.g1, mix.g2) instead of mix.a / mix.g.  gate_act: 0 silu, 1 sigmoid. */
    int decay_channels, decay_rank, gate_rank, gate_act;
    /* WF_SEQ_SSD: heads of vdim channels, state size `dim`, `kv_heads` groups of input / output maps (B, C) shared by heads / kv_heads
     * heads each, `conv` taps (with bias), the gated output normalised in out_norm_groups equal parts.  Tensors mix.in [2 inner + 2 groups
     * dim + heads, W] laid out [z | x | B | C | dt], mix.conv, mix.conv.b, mix.dt_bias, mix.A_log, mix.D, mix.norm, mix.o. */
    int out_norm_groups;
    /* a second mixer beside this one: `pair` > 0 is the index of its descriptor in the layer array (at or behind n_layers); both read the
     * same input and the mixer's output is mix_scale * this + pair_scale * that.  This mixer's tensors are then named 'l<i>.mix.left.*',
     * the other's 'l<i>.mix.right.*'. */
    int pair;
    float mix_scale, pair_scale;
    /* tied = 1: the layer has no tensors of its own and uses those of layer tied_to (another layer, untied, with the same descriptor;
     * it may come later); its cache rows and its state are its own. */
    int tied, tied_to;
    /* latent attention, further.  q_rank > 0: queries go through a latent of that size, q = W_uq (w * rms(W_dq x)) (tensors mix.dq,
     * mix.dq.norm, mix.uq instead of mix.q).  head_gate: 0 = no output gate, otherwise sigmoid(W_g x) per output element.  rope_interleaved
     * as for grouped-query attention.  sink = 2 (both attention kinds): the softmax denominator carries exp(s_h), s_h a learned number per
     * head (tensor mix.sink [heads]) that is neither scaled nor given a value.  window: as above; a causal layer passes a window no
     * sequence reaches. */
    int q_rank;
    /* rotation, both attention kinds.  rope_factor > 1: frequency interpolation.  With t(x) = rope_dims * ln(rope_orig / (2 pi x)) /
     * (2 ln rope_base), lo = max(floor(t(rope_fast)), 0), hi = min(ceil(t(rope_slow)), rope_dims - 1) and ramp_i = clamp((i - lo) /
     * max(hi - lo, 0.001), 0, 1), pair i turns with f_i / rope_factor * ramp_i + f_i * (1 - ramp_i), f_i = rope_base^(-2i / rope_dims),
     * and cosines and sines are multiplied by 0.1 ln(rope_factor) + 1.  (The engine tabulates the frequencies once, in double.) */
    float rope_factor, rope_orig, rope_fast, rope_slow;
    /* grouped-query attention: v_is_k = 1: there is no value projection; the values are the keys as cached (vdim == dim), and a page
     * holds the keys only. */
    int v_is_k;
    /* WF_SEQ_MINGRU: `vdim` channels (heads = dim = 1).  z = sigmoid(W_z x + b_z), u = W_x x + b_x, c = u + 1/2 (u >= 0) or sigmoid(u);
     * S <- (1 - z) S + z c per channel; output W_o (S * silu(W_g x)).  Tensors mix.z, mix.z.b, mix.x, mix.x.b, mix.g, mix.o.
     * WF_SEQ_MLSTM: heads of key size dim and value size vdim.  q = W_q x * dim^-1/2, k, v; per head log gates
     * i = cap tanh((W_i x + b_i) / cap), f = logsigmoid(cap tanh((W_f x + b_f) / cap)), cap = gate_cap (0: no cap); m <- max(f + m, i)
     * (m starts at 0); S <- e^(f + m' - m) S + e^(i - m) k v^T, n likewise with k; o = S^T q / (max(|n . q|, e^-m) + 1e-6); each head's o
     * divided by its root mean square, times mix.norm [heads * vdim], times sigmoid(W_g x), then W_o.  Tensors mix.q, mix.k, mix.v, mix.g,
     * mix.i, mix.i.b, mix.f, mix.f.b, mix.norm, mix.o. */
    float gate_cap;
} wf_seq_layer;

typedef struct wf_seq_config {
    int dtype;                     /* WF_SEQ_BF16: bf16 weights, caches and matrix-product operands; WF_SEQ_F32: everything in float */
    int vocab, width, n_layers;
    float eps;
    int norm_groups, canon_taps;
    int page_size, max_pages;      /* cache pool: max_pages pages of page_size tokens (all cached layers of a token share a page) */
    int slots;                     /* sequences alive at once (each owns one state slot and one block-table row) */
    int max_step_tokens;           /* most tokens in one step */
    int block_form;                /* WF_SEQ_BLOCK_* */
    float residual_mult;           /* WF_SEQ_BLOCK_POST */
    int pos_embed;                 /* 1: a sinusoidal position vector is added to the embedding (entry 2i sin, 2i + 1 cos of p * pos_base^(-2i / width)) */
    float pos_base;
    int n_extra;                   /* mixer descriptors behind the n_layers layer entries (the second mixers of paired layers) */
    float embed_scale;             /* the embedding row is multiplied by this (0 is read as 1) */
    int norm_weights;              /* WF_SEQ_BLOCK_POST: 1 = the norms have weight vectors of the width instead of a single gain */
    int tied_head;                 /* 1: logits are products with the embedding table itself; there is no 'head' tensor */
    float norm_offset;             /* added to every stored weight of the layer norms and the final norm (1: weights stored around zero) */
} wf_seq_config;

typedef struct wf_seq_engine wf_seq_engine;

int wf_seq_available(void);
int wf_seq_create(const wf_seq_config* cfg, const wf_seq_layer* layers, wf_seq_engine** out);
void wf_seq_destroy(wf_seq_engine* e);
size_t wf_seq_device_bytes(const wf_seq_engine* e);
/* Upload one checkpoint tensor by its checkpoint name ('embed', 'l3.mix.q', 'l0.mlp.e7.down', ...); data holds `count` elements of the
 * engine's dtype (host or device memory).  The engine lays the pieces out for its kernels (fused projections, stacked experts). */
int wf_seq_set_tensor(wf_seq_engine* e, const char* name, const void* data, size_t count, int is_host);
/* number of tensors the engine expects; name of the i-th and its element count (loader support, also lists what is still missing) */
int wf_seq_tensor_count(const wf_seq_engine* e);
const char* wf_seq_tensor_name(const wf_seq_engine* e, int i, size_t* count, int* loaded);
int wf_seq_finalize(wf_seq_engine* e);

/* Sequence life cycle.  admit: a free slot with zeroed state, length 0 (-1 in *slot when none is free: not an error).
 * release: its pages and its slot go back to the free lists. */
int wf_seq_admit(wf_seq_engine* e, int* slot);
int wf_seq_release(wf_seq_engine* e, int slot);
int wf_seq_length(const wf_seq_engine* e, int slot);
int wf_seq_free_pages(const wf_seq_engine* e);
int wf_seq_free_slots(const wf_seq_engine* e);

/* One step: sequence i (slot slots[i]) advances by counts[i] tokens taken in order from `tokens`; all of them run as one ragged batch.
 * want[j] are indices into the flat token list whose logits are computed (float [nwant, vocab], kept on the device until the next
 * step; copied to logits_host when that is not null).  Synchronous. */
int wf_seq_step(wf_seq_engine* e, int nseq, const int32_t* slots, const int32_t* counts, const int32_t* tokens, int nwant,
                const int32_t* want, float* logits_host);
/* Draw one token per wanted row of the last step: temperature <= 0 is greedy; else softmax(logits / temperature) limited to the top_k
 * most likely (0: all) and to the smallest set whose mass reaches top_p (>= 1: all); uniforms: one number in [0, 1) per row. */
int wf_seq_sample(wf_seq_engine* e, int nwant, float temperature, int top_k, float top_p, const float* uniforms_host, int32_t* next_host);
void* wf_seq_logits_device(wf_seq_engine* e);
int wf_seq_launches_last_step(const wf_seq_engine* e);

/* Parity taps.  layer_tap: when not null, the residual stream after every layer of the next steps is copied there
 * (float [n_layers, n, width], n = tokens of the step).  wf_seq_run_part runs ONE part of one layer on given float rows (host memory,
 * [n, width]) through the same kernels, caches and state as wf_seq_step, and returns that part's float output [n, width]:
 * 0 first norm, 1 input convolution of the mixer (carried state), 2 the mixer, 3 the feed-forward, 4 input convolution of the
 * feed-forward (1 and 4: WF_SEQ_BLOCK_SANDWICH only; part 0 of WF_SEQ_BLOCK_POST is residual_mult * gain * rms(rows)), 5 second norm
 * (WF_SEQ_BLOCK_PARALLEL only).
 * Sequence lengths advance as in a step. */
int wf_seq_set_layer_tap(wf_seq_engine* e, float* host);
int wf_seq_run_part(wf_seq_engine* e, int layer, int part, int nseq, const int32_t* slots, const int32_t* counts, const float* in_host,
                    float* out_host);
/* mean device time of one step shape (measurement): runs the step `iters` times on synthetic tokens and returns milliseconds per step.
 * Sequence lengths and pages are left as they were; the slots' convolution tails and recurrent state ARE advanced by the timed tokens,
 * so the slots are not to be used for real requests afterwards without a release / admit. */
int wf_seq_time_step(wf_seq_engine* e, int nseq, const int32_t* slots, const int32_t* counts, int iters, float* ms_out);
/* the same, with an event after every launch group: out receives JSON {"kind": [ms per step, launches per step], ...} */
int wf_seq_profile_step(wf_seq_engine* e, int nseq, const int32_t* slots, const int32_t* counts, int iters, char* out, size_t cap);
/* measurement: declare that a live slot holds `len` tokens (pages are allocated, their contents are whatever the pool holds) */
int wf_seq_set_length(wf_seq_engine* e, int slot, int len);

/* The engine's matrix product on its own: C[m, n] = sum_k A[m, k] * B[n, k] (device pointers; A is dtype or float, C float or dtype).
 * tile_group (optional): expert of every 128-row tile of A / C (< 0: skipped), experts' [N, K] matrices group_stride elements apart.
 * algo: 0 as the engine chooses, 1 plain FMA, 2 mma.sync, 3 tcgen05, 4 few-row streaming. */
int wf_seq_op_gemm(int dtype, const void* A, int a_f32, int lda, const void* B, int ldb, void* C, int c_f32, int ldc, int M, int N, int K,
                   const int32_t* tile_group, long long group_stride, int n_groups, int algo, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WF_SEQ_H */
