// Grouped-query softmax attention over a paged cache of per-head keys and values.  Positions can enter through a rotation of queries and
// keys (partial, pairs interleaved or split in halves), through a linear distance penalty per head (score -= slope_h * (i - j),
// slope_h = 2^(-dist_exp (h + 1) / H)) or through a learned bias by distance; the visible keys are the causal ones inside a sliding window
// and / or inside the query's own chunk of positions; scores can be capped by a tanh and the softmax denominator can carry an extra one.
// Queries, keys and values can be normalised before use (per head, with or without weights, or over the whole projection; the cache holds
// keys and values in that form), and the output can be multiplied by a sigmoid gate computed from the layer input, per head or per element.
// A layer may read the cache rows that an earlier layer wrote instead of projecting its own.
// Norms, scores, softmax and the weighted sum are float; the cache and the query operand are the storage type.
//
// Cache layout of one layer inside a page: keys [G][page_size][d], then values [G][page_size][dv] (no value part when the values are the keys).
#include "seq_kernels.cuh"
#include <math.h>

namespace wf {
namespace seq {

namespace {

constexpr int GA_WARPS = 4;
constexpr int GA_MAXD = 16;    // per-head sizes up to 32 * 16

constexpr int GA_MAXROT = 256;  // rotated pairs per head

// One block per token; its warps walk the token's head vectors (H query heads, then G key heads, then G value heads): bias, norm
// (per head, or over the whole projection with two block-wide sums first), rotation, store.  The cosines and sines of the token's
// angles are formed once per block in double, so that the float values are the correctly rounded ones at any position.
template <typename T>
__global__ void __launch_bounds__(GA_WARPS * 32) gqa_prep_kernel(Batch b, GqaDims D, const float* __restrict__ proj, int ld, int k_off, int v_off, int g_off,
                                                                   const T* __restrict__ qb, const T* __restrict__ kb, const T* __restrict__ vb, float eps,
                                                                   PagedCache pc, T* __restrict__ qn, float* __restrict__ gate) {
    __shared__ float rot_c[GA_MAXROT], rot_s[GA_MAXROT];
    __shared__ float vec[GA_WARPS][32 * GA_MAXD];
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sq = b.tok_seq[i], pos = b.tok_pos[i];
    const float* row = proj + (size_t)i * ld;
    const int units = D.H + (k_off >= 0 ? (D.v_is_k ? D.G : 2 * D.G) : 0);      // the values are stored only when they are not the keys
    T* page = nullptr;
    if (k_off >= 0) {
        const int pg = pc.block_table[(size_t)b.seq_slot[sq] * pc.max_blocks + pos / pc.page_size];
        page = (T*)pc.pool + (size_t)pg * pc.page_stride + pc.layer_off;
    }
    const int slot = pos % pc.page_size;
    const int half = D.rope_dims / 2;
    if (half > 0) {
        const double lb = log2((double)D.rope_base);
        for (int p = threadIdx.x; p < half; p += blockDim.x) {
            const double a = (double)pos * exp2(-2.0 * (double)p / (double)D.rope_dims * lb);
            rot_c[p] = (float)cos(a); rot_s[p] = (float)sin(a);
        }
    }
    float inv_q = 1.f, inv_k = 1.f;
    if (D.qk_norm == 3) {           // root mean square of the whole query row and of the whole key row
        float sq_ = 0.f, sk_ = 0.f;
        for (int c = threadIdx.x; c < D.H * D.d; c += blockDim.x) { const float v = row[c] + (qb ? to_f(qb[c]) : 0.f); sq_ = fmaf(v, v, sq_); }
        sq_ = block_sum(sq_, scratch);
        inv_q = 1.f / sqrtf(sq_ / (float)(D.H * D.d) + eps);
        if (k_off >= 0) {
            for (int c = threadIdx.x; c < D.G * D.d; c += blockDim.x) { const float v = row[k_off + c] + (kb ? to_f(kb[c]) : 0.f); sk_ = fmaf(v, v, sk_); }
            sk_ = block_sum(sk_, scratch);
            inv_k = 1.f / sqrtf(sk_ / (float)(D.G * D.d) + eps);
        }
    }
    __syncthreads();
    const T* qw = (const T*)D.q_norm_w;
    const T* kw = (const T*)D.k_norm_w;
    for (int u = warp; u < units; u += GA_WARPS) {
        const float* src; const T* bias; T* dst; int dim; int norm; const T* nw = nullptr; float inv_all = 1.f; bool rot;
        if (u < D.H) {
            src = row + (size_t)u * D.d; bias = qb ? qb + (size_t)u * D.d : nullptr; dst = qn + ((size_t)i * D.H + u) * D.d; dim = D.d; norm = D.qk_norm; rot = half > 0;
            if (norm == 2) nw = qw; else if (norm == 3) { nw = qw + (size_t)u * D.d; inv_all = inv_q; }
        } else if (u < D.H + D.G) {
            const int g = u - D.H;
            src = row + k_off + (size_t)g * D.d; bias = kb ? kb + (size_t)g * D.d : nullptr; dim = D.d; norm = D.qk_norm; rot = half > 0;
            if (norm == 2) nw = kw; else if (norm == 3) { nw = kw + (size_t)g * D.d; inv_all = inv_k; }
            dst = page + ((size_t)g * pc.page_size + slot) * D.d;
        } else {
            const int g = u - D.H - D.G;
            src = row + v_off + (size_t)g * D.dv; bias = vb ? vb + (size_t)g * D.dv : nullptr; dim = D.dv; norm = D.v_norm ? 1 : 0; rot = false;
            dst = page + (size_t)D.G * pc.page_size * D.d + ((size_t)g * pc.page_size + slot) * D.dv;
        }
        float v[GA_MAXD];
        float ss = 0.f;
#pragma unroll
        for (int t = 0; t < GA_MAXD; ++t) {
            const int c = lane + 32 * t;
            v[t] = c < dim ? src[c] + (bias ? to_f(bias[c]) : 0.f) : 0.f;
            ss = fmaf(v[t], v[t], ss);
        }
        float inv = 1.f;
        if (norm == 1 || norm == 2) { ss = warp_sum(ss); inv = 1.f / sqrtf(ss / (float)dim + eps); }
        else if (norm == 3) inv = inv_all;
#pragma unroll
        for (int t = 0; t < GA_MAXD; ++t) { const int c = lane + 32 * t; if (c < dim) v[t] = v[t] * inv * (nw ? to_f(nw[c]) : 1.f); }
        if (rot) {
            float* sv = vec[warp];
            __syncwarp();
#pragma unroll
            for (int t = 0; t < GA_MAXD; ++t) { const int c = lane + 32 * t; if (c < dim) sv[c] = v[t]; }
            __syncwarp();
#pragma unroll
            for (int t = 0; t < GA_MAXD; ++t) {
                const int c = lane + 32 * t;
                if (c < D.rope_dims && c < dim) {
                    int p, other; bool first;
                    if (D.rope_interleaved) { p = c >> 1; other = c ^ 1; first = !(c & 1); }
                    else { first = c < half; p = first ? c : c - half; other = first ? c + half : c - half; }
                    const float o = sv[other];
                    v[t] = first ? v[t] * rot_c[p] - o * rot_s[p] : v[t] * rot_c[p] + o * rot_s[p];
                }
            }
        }
#pragma unroll
        for (int t = 0; t < GA_MAXD; ++t) { const int c = lane + 32 * t; if (c < dim) dst[c] = from_f<T>(v[t]); }
    }
    if (gate) {
        const int ng = D.gate_elem ? D.H * D.dv : D.H;
        for (int h = threadIdx.x; h < ng; h += blockDim.x) gate[(size_t)i * ng + h] = g_off >= 0 ? sigmoid_f(row[g_off + h]) : 1.f;
    }
}

// One block per (token, head).  Its warps take the visible keys round-robin, a warp one key at a time with its lanes over the dimensions;
// running max / sum / weighted value sum per warp, merged through shared memory.
template <typename T>
__global__ void __launch_bounds__(GA_WARPS * 32) gqa_attn_kernel(Batch b, GqaDims D, const T* __restrict__ qn, const float* __restrict__ gate, PagedCache pc,
                                                                   T* __restrict__ out) {
    extern __shared__ float sm[];   // [GA_WARPS][dv] partial sums, [GA_WARPS] m, [GA_WARPS] l
    const int i = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sq = b.tok_seq[i], pos = b.tok_pos[i];
    const int g = h / (D.H / D.G);
    int lo = pos - D.window + 1 > 0 ? pos - D.window + 1 : 0;
    if (D.chunk > 0) { const int c0 = pos / D.chunk * D.chunk; if (c0 > lo) lo = c0; }
    const int32_t* bt = pc.block_table + (size_t)b.seq_slot[sq] * pc.max_blocks;
    const float slope = D.dist_exp > 0.f ? exp2f(-D.dist_exp * (float)(h + 1) / (float)D.H) : 0.f;
    const T* qh = qn + ((size_t)i * D.H + h) * D.d;
    const size_t k_base = (size_t)g * pc.page_size * D.d, v_base = D.v_is_k ? k_base : (size_t)D.G * pc.page_size * D.d + (size_t)g * pc.page_size * D.dv;
    float qreg[GA_MAXD], acc[GA_MAXD];
#pragma unroll
    for (int t = 0; t < GA_MAXD; ++t) { const int c = lane + 32 * t; qreg[t] = c < D.d ? to_f(qh[c]) : 0.f; acc[t] = 0.f; }
    float m = -INFINITY, l = 0.f;
    for (int j = lo + warp; j <= pos; j += GA_WARPS) {
        const T* page = (const T*)pc.pool + (size_t)bt[j / pc.page_size] * pc.page_stride + pc.layer_off;
        const int slot = j % pc.page_size;
        const T* kr = page + k_base + (size_t)slot * D.d;
        const T* vr = page + v_base + (size_t)slot * D.dv;
        float part = 0.f;
#pragma unroll
        for (int t = 0; t < GA_MAXD; ++t) { const int c = lane + 32 * t; if (c < D.d) part = fmaf(qreg[t], to_f(kr[c]), part); }
        float sc = warp_sum(part) * D.scale;
        if (D.softcap > 0.f) sc = D.softcap * tanhf(sc / D.softcap);
        if (D.rel) { const int dist = pos - j; sc += D.rel[(size_t)(dist < D.rel_n ? dist : D.rel_n - 1) * D.H + h]; }
        sc -= slope * (float)(pos - j);
        const float mn = fmaxf(m, sc);
        const float corr = expf(m - mn);      // m = -inf on the first key: exp(-inf) = 0
        const float p = expf(sc - mn);
        l = l * corr + p;
#pragma unroll
        for (int t = 0; t < GA_MAXD; ++t) { const int c = lane + 32 * t; acc[t] = fmaf(p, c < D.dv ? to_f(vr[c]) : 0.f, acc[t] * corr); }
        m = mn;
    }
    float* part_sum = sm;
    float* part_m = sm + GA_WARPS * D.dv;
    float* part_l = part_m + GA_WARPS;
#pragma unroll
    for (int t = 0; t < GA_MAXD; ++t) { const int c = lane + 32 * t; if (c < D.dv) part_sum[warp * D.dv + c] = acc[t]; }
    if (lane == 0) { part_m[warp] = m; part_l[warp] = l; }
    __syncthreads();
    float mg = -INFINITY;
#pragma unroll
    for (int w = 0; w < GA_WARPS; ++w) mg = fmaxf(mg, part_m[w]);
    float lg = 0.f, sc_w[GA_WARPS];
#pragma unroll
    for (int w = 0; w < GA_WARPS; ++w) { sc_w[w] = part_m[w] == -INFINITY ? 0.f : expf(part_m[w] - mg); lg += part_l[w] * sc_w[w]; }
    if (D.sink) lg += expf(-mg);            // the extra key: score 0, no value
    const float inv_l = 1.f / lg;
    const float* grow = gate ? (D.gate_elem ? gate + ((size_t)i * D.H + h) * D.dv : gate + (size_t)i * D.H + h) : nullptr;
    for (int c = threadIdx.x; c < D.dv; c += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GA_WARPS; ++w) v += part_sum[w * D.dv + c] * sc_w[w];
        const float gm = grow ? (D.gate_elem ? grow[c] : grow[0]) : 1.f;
        out[((size_t)i * D.H + h) * D.dv + c] = from_f<T>(v * inv_l * gm);
    }
}

int check_dims(const GqaDims& D) {
    if (D.H <= 0 || D.G <= 0 || D.H % D.G || D.d <= 0 || D.dv <= 0 || D.window < 1) { set_error("attention: %d heads over %d key/value heads, sizes %d / %d, window %d", D.H, D.G, D.d, D.dv, D.window); return WF_ERR_INVALID; }
    if (D.d > 32 * GA_MAXD || D.dv > 32 * GA_MAXD) { set_error("attention: per-head sizes %d / %d above the supported %d", D.d, D.dv, 32 * GA_MAXD); return WF_ERR_UNSUPPORTED; }
    if (D.rope_dims < 0 || (D.rope_dims & 1) || D.rope_dims > D.d || D.rope_dims / 2 > GA_MAXROT) { set_error("attention: %d rotated entries of %d", D.rope_dims, D.d); return WF_ERR_INVALID; }
    if (D.qk_norm >= 2 && (!D.q_norm_w || !D.k_norm_w)) { set_error("attention: the query / key norm has no weights"); return WF_ERR_INVALID; }
    if (D.v_is_k && D.dv != D.d) { set_error("attention: values that are the keys have the keys' size (%d / %d)", D.d, D.dv); return WF_ERR_INVALID; }
    if (D.chunk < 0 || (D.rel && D.rel_n < 1)) { set_error("attention: chunk %d, %d bias rows", D.chunk, D.rel_n); return WF_ERR_INVALID; }
    return WF_OK;
}

}  // namespace

long long gqa_cache_elems(const GqaDims& D, int page_size) { return (long long)page_size * D.G * (D.d + (D.v_is_k ? 0 : D.dv)); }

int launch_gqa_prep(int dt, const Batch& b, const GqaDims& D, const float* proj, int ld, int k_off, int v_off, int g_off, const void* qb, const void* kb,
                    const void* vb, float eps, const PagedCache& pc, void* qn, float* gate, cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (int rc = check_dims(D)) return rc;
    if (!D.v_is_k && (k_off >= 0) != (v_off >= 0)) { set_error("attention: keys and values are projected together or not at all"); return WF_ERR_INVALID; }
    if (dt == WF_BF16) gqa_prep_kernel<<<b.n, GA_WARPS * 32, 0, s>>>(b, D, proj, ld, k_off, v_off, g_off, (const __nv_bfloat16*)qb, (const __nv_bfloat16*)kb, (const __nv_bfloat16*)vb, eps, pc, (__nv_bfloat16*)qn, gate);
    else gqa_prep_kernel<<<b.n, GA_WARPS * 32, 0, s>>>(b, D, proj, ld, k_off, v_off, g_off, (const float*)qb, (const float*)kb, (const float*)vb, eps, pc, (float*)qn, gate);
    return launch_check(cudaGetLastError(), "gqa_prep");
}

int launch_gqa_attn(int dt, const Batch& b, const GqaDims& D, const void* qn, const float* gate, const PagedCache& pc, void* out, cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (int rc = check_dims(D)) return rc;
    if (D.H > 65535) { set_error("attention: too many heads"); return WF_ERR_UNSUPPORTED; }
    dim3 grid(b.n, D.H);
    const size_t smem = ((size_t)GA_WARPS * D.dv + 2 * GA_WARPS) * sizeof(float);
    if (dt == WF_BF16) gqa_attn_kernel<<<grid, GA_WARPS * 32, smem, s>>>(b, D, (const __nv_bfloat16*)qn, gate, pc, (__nv_bfloat16*)out);
    else gqa_attn_kernel<<<grid, GA_WARPS * 32, smem, s>>>(b, D, (const float*)qn, gate, pc, (float*)out);
    return launch_check(cudaGetLastError(), "gqa_attn");
}

}  // namespace seq
}  // namespace wf
