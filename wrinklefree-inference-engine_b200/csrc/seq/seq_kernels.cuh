// Launchers of the sequence-model kernels; the engine (seq_engine.cu) and the per-op C ABI (seq_capi.cu) both call these.
// dt: WF_BF16 or WF_F32 = the storage type T of weights, caches and matrix-product operands.
#pragma once
#include "seq_common.cuh"

#define WF_F32 0
#define WF_BF16 1

namespace wf {
namespace seq {

// x[i, :] = scale * table[tokens[i], :] as float; x_t: optional T copy
int launch_embed_f32(int dt, const void* table, const int32_t* tokens, int n, int W, float* x, cudaStream_t s, float scale = 1.f, void* x_t = nullptr);
// y = a * y + b * y2 over count floats
int launch_axpby(float* y, float a, const float* y2, float b, size_t count, cudaStream_t s);
// y = [res +] w * x / sqrt(mean_g(x^2) + eps) per row and per group of W / groups consecutive elements.  x, y, res float [n, W] with row
// strides ldx / ldy (res shares ldy; y may alias res); rows: optional gather of the input AND residual rows.  y_t: optional T copy of y.
// x2 (optional, same layout as x): the input is a * x + b * x2.  w_offset is added to every weight (1: weights stored around zero).
int launch_group_rmsnorm(int dt, const float* x, int ldx, const void* w, int groups, float eps, int n, int W, const float* res, float* y,
                         int ldy, void* y_t, int ldt, const int32_t* rows, cudaStream_t s, const float* x2 = nullptr, float a = 1.f, float b = 0.f,
                         float w_offset = 0.f);
// The stream update and the input norms of a layer whose two branches read the same stream, in one kernel:
// x += (a1 * y1 + a2 * y2) + y3 (each term optional; x, y* float [n, W] dense), then with r = x / sqrt(mean(x^2) + eps):
// h1 = r * (w_offset + w1), h2 = r * (w_offset + w2) as T [n, W] (each optional: null weights).  The row statistics are formed once.
int launch_add_dual_norm(int dt, float* x, const float* y1, float a1, const float* y2, float a2, const float* y3, const void* w1, const void* w2,
                         float w_offset, float eps, int n, int W, void* h1, void* h2, cudaStream_t s);
// x[i, :] = table[tokens[i], :] + sinusoidal position vector of tok_pos[i] (entry 2k sin, 2k + 1 cos of pos * base^(-2k / W)); x_t: optional T copy
int launch_embed_pos(int dt, const void* table, const int32_t* tokens, const int32_t* tok_pos, int n, int W, float base, float* x, void* x_t, cudaStream_t s);
// x_t T [n, W] = x float [n, W] rounded to the storage type (dense rows)
int launch_round_rows(int dt, const float* x, int n, int W, void* x_t, cudaStream_t s);
// RMS norm with a single gain (gain: one T element): out = [res +] mult * gain * (y + bias) / sqrt(mean((y + bias)^2) + eps).  bias T [W] or null;
// out float (may alias res) and / or out_t T; rows: optional gather of the input AND residual rows.
int launch_scalar_rmsnorm(int dt, const float* y, int ldy, const void* bias, const void* gain, float mult, float eps, int n, int W, const float* res, float* out,
                          int ldo, void* out_t, int ldt, const int32_t* rows, cudaStream_t s);
int launch_add_bias(int dt, float* y, int ld, const void* bias, int n, int W, cudaStream_t s);
// causal depthwise taps over time with carried state: out_t = [identity ? in_t : 0] + sum_j w[c, j] * in_(t - taps + 1 + j), optional silu.
// in float [n, C] (ld_in); state float [slot][taps - 1][C] (slot_stride floats between slots) = the last taps - 1 inputs of each sequence,
// read here and rolled forward by launch_taps_state AFTER this kernel.  out: T [n, C] (out_t) and / or float (out_f).  bias: optional T [C],
// added before the activation.
int launch_causal_taps(int dt, const Batch& b, const float* in, int ld_in, const void* w, int taps, int C, const float* state,
                       size_t slot_stride, int identity, int silu, void* out_t, int ld_t, float* out_f, int ld_f, cudaStream_t s,
                       const void* bias = nullptr);
int launch_taps_state(const Batch& b, const float* in, int ld_in, int taps, int C, float* state, size_t slot_stride, cudaStream_t s, int skip_single = 0);
// grouped RMS norm of x (float [n, W]) and the identity-plus-taps convolution over the normalised rows in one kernel: out_t T [n, W].
// hn (float [n, W]) receives the normalised rows of each portion's last taps - 1 tokens, for launch_taps_state(..., skip_single = 1)
// afterwards; sequences that bring one token have their state rolled here.
inline bool norm_taps_usable(int groups, int taps, int W) { return groups >= 1 && groups <= 32 && taps >= 1 && taps <= 8 && W % groups == 0; }
// the form for many tokens: row statistics first (inv: float [n, groups] scratch), then one thread per (token, channel); no state is
// rolled here (launch_taps_state without skip_single afterwards)
int launch_norm_taps_rows(int dt, const Batch& b, const float* x, int ldx, const void* nw, int groups, float eps, const void* cw, int taps, int W,
                          const float* state, size_t slot_stride, void* out_t, int ld_t, float* hn, float* inv, cudaStream_t s);
int launch_norm_taps(int dt, const Batch& b, const float* x, int ldx, const void* nw, int groups, float eps, const void* cw, int taps, int W, float* state,
                     size_t slot_stride, void* out_t, int ld_t, float* hn, cudaStream_t s);

// C[m, n] = sum_k A[m, k] * B[n, k]  (B stored [N, K] row-major, i.e. a Linear weight), float accumulation.
struct GemmArgs {
    const void* A = nullptr; int a_f32 = 0;  // A is T, or float when a_f32 (rounded to T on the tensor-core path)
    int lda = 0;
    const void* B = nullptr; int ldb = 0;
    void* C = nullptr; int c_f32 = 1;        // C is float, or T
    int ldc = 0;
    int M = 0, N = 0, K = 0;
    int batch = 1;                           // grid.z problems with element strides sA, sB, sC
    long long sA = 0, sB = 0, sC = 0;
    // grouped form (routed experts): rows [t * GEMM_BM, (t + 1) * GEMM_BM) use weight tile_group[t] (B + group * group_stride), or are skipped when < 0;
    // a_rows (optional) gathers A rows (-1 = a zero row).  M is then the padded row count bound; m_dev (optional) the real one on the device.
    const int32_t* tile_group = nullptr;
    long long group_stride = 0;
    const int32_t* a_rows = nullptr;
    int n_groups = 1;                        // weight matrices stacked behind B (grouped form)
    int algo = 0;                            // 0 = choose; 1 plain FMA, 2 mma.sync, 3 tcgen05, 4 few-row streaming (tests and measurements)
};
constexpr int GEMM_BM = 128;                 // row granule of the grouped form (the token tile of the tcgen05 kernel)
int launch_gemm(int dt, const GemmArgs& g, cudaStream_t s);
// tcgen05 form (seq_gemm_tc.cu): bf16 operands, dense A rows; launch_gemm picks it from WF_SEQ_TC_MIN (17) rows up
bool gemm_tc_usable(const GemmArgs& g);
int launch_gemm_tc(const GemmArgs& g, int n_groups, cudaStream_t s);
int gemm_tc_error(cudaStream_t s);           // 0 = no bounded wait of the tcgen05 kernel ever ran out on this device
// dst T [P, W] = src T [rows[i], :] (zero rows where rows[i] < 0)
int launch_gather_rows(int dt, const void* src, int ld, const int32_t* rows, int P, int W, void* dst, cudaStream_t s);
// routed experts while decoding: pair p (p < pairs) computes C[p, :] = B[pair_expert[p]] . A[p / pair_div, :]  (skipped when pair_expert[p]
// is not in [0, n_experts)); B + expert * g.group_stride is that expert's [N, K] matrix.  Needs 16-byte aligned rows (gemv_pairs_usable).
bool gemv_pairs_usable(int dt, const GemmArgs& g);
int launch_gemv_pairs(int dt, const GemmArgs& g, const int32_t* pair_expert, int n_experts, int pairs, int pair_div, cudaStream_t s);

// ---- latent attention ---------------------------------------------------------------------------------------------------
// interleaved: rotated pairs are (2i, 2i + 1) instead of (i, i + rope_dims / 2).  freq (device, double [rope_dims / 2]): the pairs'
// frequencies, tabulated by the caller (null: rope_base^(-2i / rope_dims) in float); the angle pos * freq, its cosine and sine are then
// formed in double and rounded once; mscale multiplies cosines and sines.  sink (device, float [H]): the softmax denominator carries
// exp(sink[h]) (null: nothing).
struct LatentDims { int H, d, r, dv, R; float scale, rope_base; int rope_dims, window;
                    int interleaved = 0; const double* freq = nullptr; float mscale = 1.f; const float* sink = nullptr; };
// q float [n, H * (d + r)] (ldq): unrotated parts -> qn T [n, H, d]; rotated parts -> rotary at tok_pos -> qr float [n, H, r]
int launch_latent_q_prep(int dt, const Batch& b, const LatentDims& L, const float* q, int ldq, void* qn, float* qr, cudaStream_t s);
// dkv float [n, R + r] (ld): first R RMS-normed with weight w (plain), last r rotated; written as T into the paged cache row of
// (sequence, position): cache + page * page_stride + layer_off + slot_in_page * (R + r)
struct PagedCache { void* pool; long long page_stride; long long layer_off; int page_size; const int32_t* block_table; int max_blocks; };
int launch_latent_kv_write(int dt, const Batch& b, const LatentDims& L, const float* dkv, int ld, const void* w, float eps, const PagedCache& pc,
                           cudaStream_t s);
// per (token, head): softmax over positions j in (pos - window, pos] of (qa . c_j + qr . kr_j) * scale; out T [n, H, R] = sum p_j c_j.
// qa float [n, H, R] (the query carried through the key up-projection), qr float [n, H, r].
int launch_latent_attn(int dt, const Batch& b, const LatentDims& L, const float* qa, const float* qr, const PagedCache& pc, void* out, cudaStream_t s);
// the same on tensor cores (bf16 storage only; seq_latent_mma.cu).  splits > 1 cuts every token's key range over that many CTAs and needs
// workspace for n * splits partial results (latent_attn_mma_workspace(n * splits, H, R) bytes).  The cache rows must start 16-byte aligned.
bool latent_attn_mma_usable(const LatentDims& L);
size_t latent_attn_mma_workspace(int token_splits, int H, int R);
int latent_attn_mma_ctas_per_sm(const LatentDims& L);
// the same with the keys as the M rows of the tiles and the heads as 8-wide N tiles (up to 32 heads, latent a multiple of 16 up to 512)
bool latent_attn_kt_usable(const LatentDims& L);
int latent_attn_kt_ctas_per_sm(const LatentDims& L);
int launch_latent_attn_kt(const Batch& b, const LatentDims& L, const float* qa, const float* qr, const PagedCache& pc, void* out, float* workspace,
                          int splits, cudaStream_t s);   // resident CTAs per SM (shared-memory bound)
int launch_latent_attn_mma(const Batch& b, const LatentDims& L, const float* qa, const float* qr, const PagedCache& pc, void* out, float* workspace,
                           int splits, cudaStream_t s);
// y T [n, C] = x float [n, C] (ldx) * act(g float [n, C] (ldg)); act 0 = sigmoid, 1 = silu, 2 = none (a plain conversion of x)
int launch_gate_mul(int dt, const float* x, int ldx, const float* g, int ldg, int act, int n, int C, void* y, int ldy, cudaStream_t s);
// out T [H][C][R] = in T [H][R][C]   (per-head transpose, done once at load)
int launch_transpose_heads(int dt, const void* in, int H, int R, int C, void* out, cudaStream_t s);

// ---- grouped-query attention (seq_attn.cu) ----------------------------------------------------------------------------------------
// qk_norm: 0 none, 1 each head divided by its root mean square, 2 the same times a weight vector of the head size (q_norm_w / k_norm_w,
// T [d]), 3 RMS norm over the whole projection with weights T [H * d] / [G * d].  rope_dims > 0: the first rope_dims entries of every query
// and key head are rotated after the norm (pairs (2i, 2i + 1) when rope_interleaved, else (i, i + rope_dims / 2)).  chunk > 0: a query sees
// only keys of its own chunk of that many positions.  softcap > 0: score <- softcap * tanh(score / softcap).  rel (float [rel_n, H], on the
// device): bias by distance, rel[min(i - j, rel_n - 1), h], added after the cap.  sink: the softmax denominator carries an extra 1.
// gate_elem: the gate has one entry per output element ([n, H * dv]) instead of one per head ([n, H]).
struct GqaDims {
    int H, G, d, dv; float scale, dist_exp; int window, qk_norm, v_norm;
    int rope_dims = 0, rope_interleaved = 0; float rope_base = 0.f;
    const void *q_norm_w = nullptr, *k_norm_w = nullptr;
    int chunk = 0, sink = 0, gate_elem = 0; float softcap = 0.f;
    const float* rel = nullptr; int rel_n = 0;
    int v_is_k = 0;               // the values are the cached keys (dv == d): a page holds keys only, nothing is projected or stored for values
};
// elements one layer's keys and values take in a cache page: keys [G][page_size][d], then values [G][page_size][dv]
long long gqa_cache_elems(const GqaDims& D, int page_size);
// proj float [n, ld]: queries at column 0 (H * d), keys at k_off (G * d), values at v_off (G * dv), gate logits at g_off (H); negative
// offsets: that part is absent (k_off and v_off together: the layer reads another layer's cache).  Adds the biases (T, or null), divides
// by the root mean square per head where D says so; queries -> qn T [n, H, d]; keys / values -> the token's cache row; gate float [n, H]
// = sigmoid of the gate logits (1 when g_off < 0; gate null: not written); [n, H * dv] with D.gate_elem.
int launch_gqa_prep(int dt, const Batch& b, const GqaDims& D, const float* proj, int ld, int k_off, int v_off, int g_off, const void* qb, const void* kb,
                    const void* vb, float eps, const PagedCache& pc, void* qn, float* gate, cudaStream_t s);
// out T [n, H * dv]: per (token, head) softmax over keys j in (pos - window, pos] of q . k_j * scale - slope_h * (pos - j), weighted value
// sum, times gate[n, H] (null: no gate).
int launch_gqa_attn(int dt, const Batch& b, const GqaDims& D, const void* qn, const float* gate, const PagedCache& pc, void* out, cudaStream_t s);

// the same on tensor cores (bf16 storage only; seq_attn_mma.cu): group sizes up to 16, per-head sizes multiples of 8 up to 128, cache rows
// 16-byte aligned.  When every sequence brings one token the key range can be cut over `splits` CTAs; that needs a workspace of
// gqa_attn_mma_workspace(n * H, splits, dv) bytes.
bool gqa_attn_mma_usable(const GqaDims& D, const PagedCache& pc);
bool gqa_attn_mma_takes(const GqaDims& D);      // the score and mask options of D that the tensor-core form implements
size_t gqa_attn_mma_workspace(int rows, int splits, int dv);
int launch_gqa_attn_mma(const Batch& b, const GqaDims& D, const void* qn, const float* gate, const PagedCache& pc, void* out, float* workspace, int splits,
                        cudaStream_t s);

// ---- gated delta rule ----------------------------------------------------------------------------------------------------
// vec_decay: the decay has one entry per head and key channel ([n, H, d]) instead of one per head.  q_off / k_off / v_off: columns of the
// first query head, key head and value head in a row (negative: the layout [q heads | k heads | v heads]).  no_delta: the write is
// u = beta v (a plain decayed outer-product accumulation: the state-space recurrence) instead of u = beta (v - S^T k).
// ones_col (no_delta form): the state has one more column whose value input is 1 for every token, so that column dv of the output is
// n . q with n the decayed sum of the written keys; state [H][d][dv + 1] and o [n, H, dv + 1] then.
struct DeltaDims { int H, Hk, d, dv; int vec_decay = 0, no_delta = 0, q_off = -1, k_off = -1, v_off = -1, ones_col = 0; };
// in place on qkv float [n, C = 2 * Hk * d + H * dv] (ld): q and k heads -> unit vectors (x / sqrt(sum x^2 + 1e-6)), q also times d^-1/2.
// beta[n, H] = sigmoid(b_raw), decay[n, H] = exp(-exp(A_log[h]) * softplus(a_raw + dt_bias[h]))   (a_raw, b_raw float with strides);
// with D.vec_decay a_raw and dt_bias have H * d entries and decay is [n, H, d]
int launch_delta_prep(int dt, const DeltaDims& D, int n, float* qkv, int ld, const float* a_raw, int lda, const float* b_raw, int ldb_,
                      const void* A_log, const void* dt_bias, float* beta, float* decay, cudaStream_t s);
// per (sequence, head): for each token in order  S = decay S;  u = beta (v - S^T k);  S += k u^T;  o = S^T q.   S float [slot][H][d][dv]
// scan (optional, no_delta form with one decay per head only): long portions are cut into chunks of SCAN_CHUNK tokens that run in parallel —
// every chunk's own contribution from a zero state, a short pass that chains the chunks' start states (S_start[c + 1] = prod_c S_start[c]
// + local_c, the recurrence being linear in the state), then every chunk again from its start state for the outputs.
constexpr int SCAN_CHUNK = 128;
struct ScanWorkspace { float* local = nullptr; float* start = nullptr; float* prod = nullptr; int chunks = 0; };   // chunks: entries of H * d * dv floats each
inline int scan_chunks_needed(int max_step_tokens, int slots) { return max_step_tokens / SCAN_CHUNK + slots + 1; }
int launch_delta_rule(const Batch& b, const DeltaDims& D, const float* qkv, int ld, const float* beta, const float* decay, float* state,
                      size_t slot_stride, float* o, cudaStream_t s, const ScanWorkspace* scan = nullptr);
// y T [n, H * dv] = o / sqrt(mean_dv(o^2) + eps) * w[dv] * act(g float [n, H * dv] (ldg)); act 0 silu, 1 sigmoid
int launch_delta_post(int dt, const DeltaDims& D, int n, const float* o, const void* w, float eps, const float* g, int ldg, void* y, cudaStream_t s, int act = 0);
// state-space recurrence around launch_delta_rule (no_delta form).  prep: step[n, H] = softplus(dt_raw + dt_bias[h]) (no clamp),
// decay[n, H] = exp(-exp(A_log[h]) * step).  post: y T [n, H * dv] = grouped RMS norm (groups equal parts of H * dv, weight w [H * dv]) of
// (o + D[h] * x) * silu(z); x float [n, H * dv] (ldx), z float (ldz).
int launch_ssd_prep(int dt, int n, int H, const float* dt_raw, int ld, const void* A_log, const void* dt_bias, float* step, float* decay, cudaStream_t s);
int launch_ssd_post(int dt, int n, int H, int dv, int groups, const float* o, const float* x, int ldx, const float* z, int ldz, const void* Dskip,
                    const void* w, float eps, void* y, cudaStream_t s);

// ---- gated recurrences (seq_gated.cu) ------------------------------------------------------------------------------------------
// element-wise gated recurrence over C channels: z = sigmoid(proj[z_off + c] + zb[c]), u = proj[x_off + c] + xb[c], cand = u + 1/2 where
// u >= 0 else sigmoid(u); S <- (1 - z) S + z cand (state float [slot][C], carried); out T [n, C] = S * silu(proj[g_off + c]).
// Long portions are cut into time slices that run in parallel inside a block (the recurrence is linear in S).
int launch_mingru(int dt, const Batch& b, int C, const float* proj, int ld, int z_off, int x_off, int g_off, const void* zb, const void* xb,
                  float* state, size_t slot_stride, void* out, cudaStream_t s);
// log gates of the matrix memory and their running maximum, per (sequence, head) in token order (a block's warps scan 32 tokens each):
// li = cap tanh((proj[i_off + h] + ib[h]) / cap), lf = logsigmoid(cap tanh((proj[f_off + h] + fb[h]) / cap)) (cap <= 0: no cap);
// m_t = max(lf + m_(t-1), li) with m carried in mstate[slot * slot_stride + h]; keep[n, H] = exp(lf + m_(t-1) - m_t),
// put[n, H] = exp(li - m_t), mrun[n, H] = m_t.
int launch_mlstm_gates(int dt, const Batch& b, int H, const float* proj, int ld, int i_off, int f_off, const void* ib, const void* fb, float cap,
                       float* mstate, size_t slot_stride, float* keep, float* put, float* mrun, cudaStream_t s);
// read-out of the matrix memory: o float [n, H, dv + 1] (column dv = n . q) -> per head o * qscale / (max(|n . q| * qscale, exp(-m)) + 1e-6),
// divided by its root mean square (eps), times w[H * dv], times sigmoid(g float [n, H * dv] (ldg)) -> y T [n, H * dv]
int launch_mlstm_post(int dt, int n, int H, int dv, const float* o, const float* mrun, float qscale, const void* w, float eps, const float* g, int ldg,
                      void* y, cudaStream_t s);

// ---- routed feed-forward ---------------------------------------------------------------------------------------------------
struct RouterDims {
    int E, I, top, groups, keep;   // E real experts, I identity experts (indices E .. E + I - 1)
    int act = 0;                   // scores: 0 softmax over all outputs, 1 sigmoid of each
    int group_top = 1;             // a group's score is the sum of this many of its largest choice scores
    int norm = 0;                  // 1: weights divided by the sum of the chosen scores (+ 1e-20)
    float scale = 1.f;             // weights multiplied by this
};
// z float [n, E + I] (ldz) -> ids [n, top], wts [n, top]; counts[E] += tokens per real expert (zero on entry; null: not counted)
int launch_moe_route(int dt, const RouterDims& R, int n, const float* z, int ldz, const void* correction, int32_t* ids, float* wts,
                     int32_t* counts, cudaStream_t s);
// the router product and the choice in one kernel: z[i, 0..NZ) = w[NZ, W] . x[i, :] with x FLOAT (ldx) and float products, then the choice
// as launch_moe_route makes it from the first E + I logits.  NZ >= E + I: extra rows (a shared expert's gate) are only multiplied.
bool router_fused_usable(const RouterDims& R, int NZ, int W);
int launch_router_fused(int dt, const RouterDims& R, int n, const float* x, int ldx, const void* w, int NZ, int W, float* z, int ldz, const void* correction,
                        int32_t* ids, float* wts, int32_t* counts, cudaStream_t s);
// from counts: expert segments padded to GEMM_BM rows.  sorted_rows[P] = token of the row or -1; pair_row[n * top] = row of the pair or -1
// (identity expert); tile_group[P / GEMM_BM] = expert of the row tile or -1.  P = row bound = round_up(n * top, BM) + E * BM.
// scratch: 2 * E + 1 ints.
int launch_moe_plan(const RouterDims& R, int n, const int32_t* ids, const int32_t* counts, int32_t* scratch, int32_t* sorted_rows,
                    int32_t* pair_row, int32_t* tile_group, int P, cudaStream_t s);
// hmid T [P, ff] = act(gu[:, :ff], gu[:, ff:])   (gu float [P, 2 ff]); rows of skipped tiles are left alone (tile_group null: every row).
// act 0: silu(g) * u;  act 1: g = min(g, limit), u = clamp(u, -limit, limit), g * sigmoid(1.702 g) * (u + 1);  act 2: gelu(g) * u (tanh form);
// act 3: relu(u)^2 with gu float [P, ff] (no gate half)
int launch_silu_mul(int dt, const float* gu, int P, int ff, const int32_t* tile_group, void* hmid, cudaStream_t s, int act = 0, float limit = 0.f);
// out float [n, W] = sum_k wts[t, k] * (ids[t, k] < E ? y[pair_row[t, k], :] : h[t, :])     (h T [n, W]; pair_row null: row t * top + k)
// shared_y (optional, float [n, W]): a shared expert's output, added times sigmoid(shared_gate[i * ld_gate]) (shared_gate null: times 1)
int launch_moe_combine(int dt, const RouterDims& R, int n, int W, const int32_t* ids, const float* wts, const int32_t* pair_row, const float* y,
                       const void* h, float* out, cudaStream_t s, const float* shared_y = nullptr, const float* shared_gate = nullptr, int ld_gate = 0);

// ---- sampling ----------------------------------------------------------------------------------------------------------------
// next[i] = argmax (temperature <= 0) or a draw from softmax(logits / temperature) restricted to the top_k largest (0 = all) and the
// smallest prefix whose mass reaches top_p; one uniform u[i] in [0, 1) per row.  logits float [m, V].
int launch_sample(const float* logits, int m, int V, float temperature, int top_k, float top_p, const float* u, int32_t* next, cudaStream_t s);

}  // namespace seq
}  // namespace wf
