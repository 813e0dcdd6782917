// Row-wise kernels of the sequence models: embedding gather, grouped RMS norm (+ residual add), causal depthwise taps with carried state.
#include "seq_kernels.cuh"

namespace wf {
namespace seq {

template <typename T>
__global__ void embed_f32_kernel(const T* __restrict__ table, const int32_t* __restrict__ tokens, int W, float* __restrict__ x, float scale, T* __restrict__ x_t) {
    const int i = blockIdx.x;
    const T* row = table + (size_t)tokens[i] * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = to_f(row[c]) * scale;
        x[(size_t)i * W + c] = v;
        if (x_t) x_t[(size_t)i * W + c] = from_f<T>(v);
    }
}

int launch_embed_f32(int dt, const void* table, const int32_t* tokens, int n, int W, float* x, cudaStream_t s, float scale, void* x_t) {
    if (n <= 0) return WF_OK;
    if (dt == WF_BF16) embed_f32_kernel<<<n, 256, 0, s>>>((const __nv_bfloat16*)table, tokens, W, x, scale, (__nv_bfloat16*)x_t);
    else embed_f32_kernel<<<n, 256, 0, s>>>((const float*)table, tokens, W, x, scale, (float*)x_t);
    return launch_check(cudaGetLastError(), "embed_f32");
}

__global__ void axpby_kernel(float* __restrict__ y, float a, const float* __restrict__ y2, float b, size_t count) {
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < count; k += (size_t)gridDim.x * blockDim.x) y[k] = a * y[k] + b * y2[k];
}

int launch_axpby(float* y, float a, const float* y2, float b, size_t count, cudaStream_t s) {
    if (count == 0) return WF_OK;
    const int blocks = (int)((count + 255) / 256 > 4096 ? 4096 : (count + 255) / 256);
    axpby_kernel<<<blocks, 256, 0, s>>>(y, a, y2, b, count);
    return launch_check(cudaGetLastError(), "axpby");
}

// x[i, :] = table[tokens[i], :] + position vector of tok_pos[i]: entry 2k = sin(a), entry 2k + 1 = cos(a), a = pos * base^(-2k / W).
// The frequency and the angle are formed in double so that the float result is the correctly rounded one also at large positions.
template <typename T>
__global__ void embed_pos_kernel(const T* __restrict__ table, const int32_t* __restrict__ tokens, const int32_t* __restrict__ tok_pos, int W, float base,
                                 float* __restrict__ x, T* __restrict__ x_t) {
    const int i = blockIdx.x;
    const T* row = table + (size_t)tokens[i] * W;
    const double pos = (double)tok_pos[i], lb = log2((double)base);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const double a = pos * exp2(-2.0 * (double)(c >> 1) / (double)W * lb);
        const float v = to_f(row[c]) + (float)((c & 1) ? cos(a) : sin(a));
        x[(size_t)i * W + c] = v;
        if (x_t) x_t[(size_t)i * W + c] = from_f<T>(v);
    }
}

int launch_embed_pos(int dt, const void* table, const int32_t* tokens, const int32_t* tok_pos, int n, int W, float base, float* x, void* x_t, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    if (dt == WF_BF16) embed_pos_kernel<<<n, 256, 0, s>>>((const __nv_bfloat16*)table, tokens, tok_pos, W, base, x, (__nv_bfloat16*)x_t);
    else embed_pos_kernel<<<n, 256, 0, s>>>((const float*)table, tokens, tok_pos, W, base, x, (float*)x_t);
    return launch_check(cudaGetLastError(), "embed_pos");
}

// x_t[i, :] = T(x[i, :])
template <typename T>
__global__ void round_rows_kernel(const float* __restrict__ x, size_t count, T* __restrict__ x_t) {
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < count; k += (size_t)gridDim.x * blockDim.x) x_t[k] = from_f<T>(x[k]);
}

int launch_round_rows(int dt, const float* x, int n, int W, void* x_t, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    const size_t count = (size_t)n * W;
    const int blocks = (int)((count + 255) / 256 > 4096 ? 4096 : (count + 255) / 256);
    if (dt == WF_BF16) round_rows_kernel<<<blocks, 256, 0, s>>>(x, count, (__nv_bfloat16*)x_t);
    else round_rows_kernel<<<blocks, 256, 0, s>>>(x, count, (float*)x_t);
    return launch_check(cudaGetLastError(), "round_rows");
}

// RMS norm with ONE gain: v = mult * gain * (y + bias) / sqrt(mean((y + bias)^2) + eps) [+ res].  One block per row; the row is kept in
// registers between the two passes (up to SN_PER values per thread, re-read beyond that).
constexpr int SN_THREADS = 256, SN_PER = 8;
template <typename T>
__global__ void __launch_bounds__(SN_THREADS) scalar_rmsnorm_kernel(const float* __restrict__ y, int ldy, const T* __restrict__ bias, const T* __restrict__ gain, float mult,
                                                                    float eps, int W, const float* res, float* out, int ldo, T* __restrict__ out_t, int ldt,
                                                                    const int32_t* __restrict__ rows) {
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;
    const float* yr = y + (size_t)src * ldy;
    float v[SN_PER];
    float ss = 0.f;
#pragma unroll
    for (int t = 0; t < SN_PER; ++t) {
        const int c = threadIdx.x + t * SN_THREADS;
        v[t] = c < W ? yr[c] + (bias ? to_f(bias[c]) : 0.f) : 0.f;
        ss = fmaf(v[t], v[t], ss);
    }
    for (int c = threadIdx.x + SN_PER * SN_THREADS; c < W; c += SN_THREADS) { const float u = yr[c] + (bias ? to_f(bias[c]) : 0.f); ss = fmaf(u, u, ss); }
    ss = block_sum(ss, scratch);
    const float k = mult * to_f(gain[0]) / sqrtf(ss / (float)W + eps);
#pragma unroll
    for (int t = 0; t < SN_PER; ++t) {
        const int c = threadIdx.x + t * SN_THREADS;
        if (c < W) {
            float u = v[t] * k;
            if (res) u += res[(size_t)src * ldo + c];
            if (out) out[(size_t)i * ldo + c] = u;
            if (out_t) out_t[(size_t)i * ldt + c] = from_f<T>(u);
        }
    }
    for (int c = threadIdx.x + SN_PER * SN_THREADS; c < W; c += SN_THREADS) {
        float u = (yr[c] + (bias ? to_f(bias[c]) : 0.f)) * k;
        if (res) u += res[(size_t)src * ldo + c];
        if (out) out[(size_t)i * ldo + c] = u;
        if (out_t) out_t[(size_t)i * ldt + c] = from_f<T>(u);
    }
}

int launch_scalar_rmsnorm(int dt, const float* y, int ldy, const void* bias, const void* gain, float mult, float eps, int n, int W, const float* res, float* out,
                          int ldo, void* out_t, int ldt, const int32_t* rows, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    if (res && rows && out == res) { set_error("scalar_rmsnorm: gathered rows cannot be added in place"); return WF_ERR_INVALID; }
    if (dt == WF_BF16) scalar_rmsnorm_kernel<<<n, SN_THREADS, 0, s>>>(y, ldy, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)gain, mult, eps, W, res, out, ldo, (__nv_bfloat16*)out_t, ldt, rows);
    else scalar_rmsnorm_kernel<<<n, SN_THREADS, 0, s>>>(y, ldy, (const float*)bias, (const float*)gain, mult, eps, W, res, out, ldo, (float*)out_t, ldt, rows);
    return launch_check(cudaGetLastError(), "scalar_rmsnorm");
}

// y[i, :] += bias
template <typename T>
__global__ void add_bias_kernel(float* __restrict__ y, int ld, const T* __restrict__ bias, int W) {
    for (int c = threadIdx.x; c < W; c += blockDim.x) y[(size_t)blockIdx.x * ld + c] += to_f(bias[c]);
}

int launch_add_bias(int dt, float* y, int ld, const void* bias, int n, int W, cudaStream_t s) {
    if (n <= 0 || !bias) return WF_OK;
    if (dt == WF_BF16) add_bias_kernel<<<n, 256, 0, s>>>(y, ld, (const __nv_bfloat16*)bias, W);
    else add_bias_kernel<<<n, 256, 0, s>>>(y, ld, (const float*)bias, W);
    return launch_check(cudaGetLastError(), "add_bias");
}

// one block per (row, group).  x2 (optional): the normalised quantity is a * x + b * x2 (two mixers' outputs combined on the way in)
template <typename T>
__global__ void group_rmsnorm_kernel(const float* __restrict__ x, int ldx, const T* __restrict__ w, int gw, float eps, const float* res,
                                     float* y, int ldy, T* __restrict__ y_t, int ldt, const int32_t* __restrict__ rows, const float* __restrict__ x2, float a,
                                     float b, float w_offset) {
    __shared__ float scratch[33];
    const int i = blockIdx.x, g = blockIdx.y;
    const int src = rows ? rows[i] : i;
    const float* xr = x + (size_t)src * ldx + (size_t)g * gw;
    const float* xr2 = x2 ? x2 + (size_t)src * ldx + (size_t)g * gw : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < gw; c += blockDim.x) { const float v = xr2 ? a * xr[c] + b * xr2[c] : xr[c]; ss += v * v; }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)gw + eps);
    for (int c = threadIdx.x; c < gw; c += blockDim.x) {
        float v = (xr2 ? a * xr[c] + b * xr2[c] : xr[c]) * inv * (w_offset + to_f(w[g * gw + c]));
        if (res) v += res[(size_t)src * ldy + g * gw + c];
        if (y) y[(size_t)i * ldy + g * gw + c] = v;
        if (y_t) y_t[(size_t)i * ldt + g * gw + c] = from_f<T>(v);
    }
}

int launch_group_rmsnorm(int dt, const float* x, int ldx, const void* w, int groups, float eps, int n, int W, const float* res, float* y,
                         int ldy, void* y_t, int ldt, const int32_t* rows, cudaStream_t s, const float* x2, float a, float b, float w_offset) {
    if (n <= 0) return WF_OK;
    if (groups <= 0 || W % groups) { set_error("group_rmsnorm: width %d not divisible into %d groups", W, groups); return WF_ERR_INVALID; }
    if (res && rows && y == res) { set_error("group_rmsnorm: gathered rows cannot be added in place"); return WF_ERR_INVALID; }
    const int gw = W / groups;
    const int threads = gw >= 2048 ? 512 : (gw >= 1024 ? 256 : (gw >= 256 ? 128 : 64));
    dim3 grid(n, groups);
    if (dt == WF_BF16) group_rmsnorm_kernel<<<grid, threads, 0, s>>>(x, ldx, (const __nv_bfloat16*)w, gw, eps, res, y, ldy, (__nv_bfloat16*)y_t, ldt, rows, x2, a, b, w_offset);
    else group_rmsnorm_kernel<<<grid, threads, 0, s>>>(x, ldx, (const float*)w, gw, eps, res, y, ldy, (float*)y_t, ldt, rows, x2, a, b, w_offset);
    return launch_check(cudaGetLastError(), "group_rmsnorm");
}

// One block per row; the updated row stays in registers between the sum of squares and the two scaled copies (up to AD_PER elements per
// thread; wider rows are re-read from x, which the same thread has just written).
constexpr int AD_THREADS = 256, AD_PER = 8;
template <typename T>
__global__ void __launch_bounds__(AD_THREADS) add_dual_norm_kernel(float* __restrict__ x, const float* __restrict__ y1, float a1, const float* __restrict__ y2, float a2,
                                                                     const float* __restrict__ y3, const T* __restrict__ w1, const T* __restrict__ w2, float w_offset,
                                                                     float eps, int W, T* __restrict__ h1, T* __restrict__ h2) {
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * W;
    const bool adds = y1 || y2 || y3;
    float keep[AD_PER];
    float ss = 0.f;
    int k = 0;
    for (int c = threadIdx.x; c < W; c += AD_THREADS, ++k) {
        float v = x[base + c];
        if (adds) {
            float t = 0.f;
            if (y1) t = a1 * y1[base + c];
            if (y2) t = fmaf(a2, y2[base + c], t);
            if (y3) t += y3[base + c];
            v += t;
            x[base + c] = v;
        }
        if (k < AD_PER) keep[k] = v;
        ss = fmaf(v, v, ss);
    }
    if (!w1 && !w2) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)W + eps);
    k = 0;
    for (int c = threadIdx.x; c < W; c += AD_THREADS, ++k) {
        const float r = (k < AD_PER ? keep[k] : x[base + c]) * inv;
        if (w1) h1[base + c] = from_f<T>(r * (w_offset + to_f(w1[c])));
        if (w2) h2[base + c] = from_f<T>(r * (w_offset + to_f(w2[c])));
    }
}

int launch_add_dual_norm(int dt, float* x, const float* y1, float a1, const float* y2, float a2, const float* y3, const void* w1, const void* w2,
                         float w_offset, float eps, int n, int W, void* h1, void* h2, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    if (dt == WF_BF16) add_dual_norm_kernel<<<n, AD_THREADS, 0, s>>>(x, y1, a1, y2, a2, y3, (const __nv_bfloat16*)w1, (const __nv_bfloat16*)w2, w_offset, eps, W, (__nv_bfloat16*)h1, (__nv_bfloat16*)h2);
    else add_dual_norm_kernel<<<n, AD_THREADS, 0, s>>>(x, y1, a1, y2, a2, y3, (const float*)w1, (const float*)w2, w_offset, eps, W, (float*)h1, (float*)h2);
    return launch_check(cudaGetLastError(), "add_dual_norm");
}

// thread per (token, channel)
template <typename T>
__global__ void causal_taps_kernel(Batch b, const float* __restrict__ in, int ld_in, const T* __restrict__ w, int taps, int C,
                                   const float* __restrict__ state, size_t slot_stride, int identity, int silu, T* __restrict__ out_t, int ld_t,
                                   float* __restrict__ out_f, int ld_f, const T* __restrict__ bias) {
    const int i = blockIdx.x;
    const int sq = b.tok_seq[i];
    const int li = i - b.seq_start[sq];                    // index inside this step's portion
    const float* st = state + (size_t)b.seq_slot[sq] * slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float acc = identity ? in[(size_t)i * ld_in + c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = li - (taps - 1) + j;           // portion-relative index of the tap's input
            const float v = src >= 0 ? in[(size_t)(i - li + src) * ld_in + c] : st[(size_t)(src + taps - 1) * C + c];
            acc = fmaf(to_f(w[(size_t)c * taps + j]), v, acc);
        }
        if (bias) acc += to_f(bias[c]);
        if (silu) acc = silu_f(acc);
        if (out_t) out_t[(size_t)i * ld_t + c] = from_f<T>(acc);
        if (out_f) out_f[(size_t)i * ld_f + c] = acc;
    }
}

int launch_causal_taps(int dt, const Batch& b, const float* in, int ld_in, const void* w, int taps, int C, const float* state,
                       size_t slot_stride, int identity, int silu, void* out_t, int ld_t, float* out_f, int ld_f, cudaStream_t s, const void* bias) {
    if (b.n <= 0) return WF_OK;
    if (taps < 1) { set_error("causal_taps: taps %d", taps); return WF_ERR_INVALID; }
    dim3 grid(b.n, (C + 255) / 256 > 8 ? 8 : (C + 255) / 256);
    if (dt == WF_BF16) causal_taps_kernel<<<grid, 256, 0, s>>>(b, in, ld_in, (const __nv_bfloat16*)w, taps, C, state, slot_stride, identity, silu, (__nv_bfloat16*)out_t, ld_t, out_f, ld_f, (const __nv_bfloat16*)bias);
    else causal_taps_kernel<<<grid, 256, 0, s>>>(b, in, ld_in, (const float*)w, taps, C, state, slot_stride, identity, silu, (float*)out_t, ld_t, out_f, ld_f, (const float*)bias);
    return launch_check(cudaGetLastError(), "causal_taps");
}

// thread per (sequence, channel): state[k] <- input at portion index len - (taps - 1) + k, taken from the old state when that is negative.
// Ascending k is safe in place: entry k reads old entry len + k > k.
__global__ void taps_state_kernel(Batch b, const float* __restrict__ in, int ld_in, int taps, int C, float* __restrict__ state, size_t slot_stride,
                                  int skip_single) {
    const int sq = blockIdx.x;
    const int len = b.seq_len[sq], start = b.seq_start[sq];
    if (skip_single && len == 1) return;                 // rolled by the fused norm + taps kernel
    float* st = state + (size_t)b.seq_slot[sq] * slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        for (int k = 0; k < taps - 1; ++k) {
            const int src = len - (taps - 1) + k;
            st[(size_t)k * C + c] = src >= 0 ? in[(size_t)(start + src) * ld_in + c] : st[(size_t)(src + taps - 1) * C + c];
        }
    }
}

int launch_taps_state(const Batch& b, const float* in, int ld_in, int taps, int C, float* state, size_t slot_stride, cudaStream_t s, int skip_single) {
    if (b.nseq <= 0 || taps <= 1) return WF_OK;
    dim3 grid(b.nseq, (C + 255) / 256 > 8 ? 8 : (C + 255) / 256);
    taps_state_kernel<<<grid, 256, 0, s>>>(b, in, ld_in, taps, C, state, slot_stride, skip_single);
    return launch_check(cudaGetLastError(), "taps_state");
}

// ---- grouped RMS norm fused with the input convolution that follows it ---------------------------------------------------------
// One block per token: it normalises the token's own row and the taps - 1 rows before it (those inside this step's portion; earlier ones
// come normalised from the carried state), applies the taps, and writes the operand of the sublayer's matrix products.  Rows that the
// next step will need are also written as float (hn) for the state roll; a sequence that brings a single token rolls its state here.
constexpr int NTAPS_MAX = 8;

template <typename T>
__global__ void norm_taps_kernel(Batch b, const float* __restrict__ x, int ldx, const T* __restrict__ nw, int groups, float eps, const T* __restrict__ cw,
                                 int taps, int W, float* __restrict__ state, size_t slot_stride, T* __restrict__ out_t, int ld_t, float* __restrict__ hn) {
    __shared__ float red[NTAPS_MAX][33];
    __shared__ float inv[NTAPS_MAX * 32];            // [tap][group]
    const int i = blockIdx.x;
    const int sq = b.tok_seq[i];
    const int li = i - b.seq_start[sq], len = b.seq_len[sq];
    const int gw = W / groups;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw_ = blockDim.x >> 5;
    float* st = state + (size_t)b.seq_slot[sq] * slot_stride;
    for (int g = 0; g < groups; ++g) {
        float ss[NTAPS_MAX];
#pragma unroll
        for (int j = 0; j < NTAPS_MAX; ++j) ss[j] = 0.f;
        for (int c = threadIdx.x; c < gw; c += blockDim.x) {
#pragma unroll
            for (int j = 0; j < NTAPS_MAX; ++j) {
                const int src = li - (taps - 1) + j;
                if (j < taps && src >= 0) { const float v = x[(size_t)(i - li + src) * ldx + g * gw + c]; ss[j] += v * v; }
            }
        }
#pragma unroll
        for (int j = 0; j < NTAPS_MAX; ++j) {
            if (j < taps) { const float v = warp_sum(ss[j]); if (lane == 0) red[j][warp] = v; }
        }
        __syncthreads();
        if (threadIdx.x < taps) {
            float t = 0.f;
            for (int w = 0; w < nw_; ++w) t += red[threadIdx.x][w];
            inv[threadIdx.x * 32 + g] = 1.f / sqrtf(t / (float)gw + eps);
        }
        __syncthreads();
    }
    const bool keep = li >= len - (taps - 1);        // one of the last taps - 1 rows of the portion: the next step's state
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const int g = c / gw;
        const float wn = to_f(nw[c]);
        float acc = 0.f, cur = 0.f, old[NTAPS_MAX];
#pragma unroll
        for (int j = 0; j < NTAPS_MAX; ++j) {
            if (j < taps) {
                const int src = li - (taps - 1) + j;
                float v;
                if (src >= 0) v = x[(size_t)(i - li + src) * ldx + c] * inv[j * 32 + g] * wn;
                else v = st[(size_t)(src + taps - 1) * W + c];
                old[j] = v;
                acc = fmaf(to_f(cw[(size_t)c * taps + j]), v, acc);
                if (j == taps - 1) cur = v;
            }
        }
        out_t[(size_t)i * ld_t + c] = from_f<T>(cur + acc);
        if (keep && hn) hn[(size_t)i * W + c] = cur;
        if (len == 1) {                               // old[j] is the input at distance taps - 1 - j: the new tail is old[1 .. taps - 1]
#pragma unroll
            for (int j = 1; j < NTAPS_MAX; ++j) if (j < taps) st[(size_t)(j - 1) * W + c] = old[j];
        }
    }
}

int launch_norm_taps(int dt, const Batch& b, const float* x, int ldx, const void* nw, int groups, float eps, const void* cw, int taps, int W, float* state,
                     size_t slot_stride, void* out_t, int ld_t, float* hn, cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (!norm_taps_usable(groups, taps, W)) { set_error("norm_taps: %d groups / %d taps are beyond the fused kernel", groups, taps); return WF_ERR_UNSUPPORTED; }
    const int threads = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
    if (dt == WF_BF16) norm_taps_kernel<<<b.n, threads, 0, s>>>(b, x, ldx, (const __nv_bfloat16*)nw, groups, eps, (const __nv_bfloat16*)cw, taps, W, state, slot_stride, (__nv_bfloat16*)out_t, ld_t, hn);
    else norm_taps_kernel<<<b.n, threads, 0, s>>>(b, x, ldx, (const float*)nw, groups, eps, (const float*)cw, taps, W, state, slot_stride, (float*)out_t, ld_t, hn);
    return launch_check(cudaGetLastError(), "norm_taps");
}

// ---- the same for many tokens: statistics once per row, then a fully parallel apply ------------------------------------------------
// inv[row][group] = 1 / sqrt(mean_group(x^2) + eps): one warp per (row, group)
__global__ void row_group_inv_rms_kernel(const float* __restrict__ x, int ldx, int n, int groups, int gw, float eps, float* __restrict__ inv) {
    const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (wid >= n * groups) return;
    const int row = wid / groups, g = wid - row * groups;
    const float* p = x + (size_t)row * ldx + (size_t)g * gw;
    float ss = 0.f;
    for (int c = lane; c < gw; c += 32) { const float v = p[c]; ss += v * v; }
    ss = warp_sum(ss);
    if (lane == 0) inv[wid] = 1.f / sqrtf(ss / (float)gw + eps);
}

// thread per (token, 4 channels): the taps over rows normalised with the precomputed statistics (or taken from the carried state).
// VEC = 4 needs W, the group width and the row strides to be multiples of 4 (one group per thread, 16-byte loads); VEC = 1 takes anything.
template <typename T, int VEC>
__global__ void norm_taps_apply_kernel(Batch b, const float* __restrict__ x, int ldx, const float* __restrict__ inv, const T* __restrict__ nw, int groups,
                                       const T* __restrict__ cw, int taps, int W, const float* __restrict__ state, size_t slot_stride, T* __restrict__ out_t,
                                       int ld_t, float* __restrict__ hn) {
    const int i = blockIdx.x;
    const int sq = b.tok_seq[i];
    const int li = i - b.seq_start[sq], len = b.seq_len[sq];
    const int gw = W / groups;
    const float* st = state + (size_t)b.seq_slot[sq] * slot_stride;
    const bool keep = li >= len - (taps - 1);
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC; c < W; c += gridDim.y * blockDim.x * VEC) {
        const int g = c / gw;
        float wn[VEC], acc[VEC], cur[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) { wn[v] = to_f(nw[c + v]); acc[v] = 0.f; cur[v] = 0.f; }
        for (int j = 0; j < taps; ++j) {
            const int src = li - (taps - 1) + j;
            float val[VEC];
            if (src >= 0) {
                const float* xr = x + (size_t)(i - li + src) * ldx + c;
                const float iv = inv[(size_t)(i - li + src) * groups + g];
                if (VEC == 4) { const float4 q = *reinterpret_cast<const float4*>(xr); val[0] = q.x; val[1 % VEC] = q.y; val[2 % VEC] = q.z; val[3 % VEC] = q.w; }
                else val[0] = xr[0];
#pragma unroll
                for (int v = 0; v < VEC; ++v) val[v] *= iv * wn[v];
            } else {
                const float* sr = st + (size_t)(src + taps - 1) * W + c;
#pragma unroll
                for (int v = 0; v < VEC; ++v) val[v] = sr[v];
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v) { acc[v] = fmaf(to_f(cw[(size_t)(c + v) * taps + j]), val[v], acc[v]); cur[v] = val[v]; }
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            out_t[(size_t)i * ld_t + c + v] = from_f<T>(cur[v] + acc[v]);
            if (keep && hn) hn[(size_t)i * W + c + v] = cur[v];
        }
    }
}

int launch_norm_taps_rows(int dt, const Batch& b, const float* x, int ldx, const void* nw, int groups, float eps, const void* cw, int taps, int W,
                          const float* state, size_t slot_stride, void* out_t, int ld_t, float* hn, float* inv, cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (groups < 1 || W % groups || taps < 1) { set_error("norm_taps_rows: %d groups / %d taps", groups, taps); return WF_ERR_INVALID; }
    const int warps = b.n * groups;
    row_group_inv_rms_kernel<<<(warps + 7) / 8, 256, 0, s>>>(x, ldx, b.n, groups, W / groups, eps, inv);
    if (int rc = launch_check(cudaGetLastError(), "row_group_inv_rms")) return rc;
    const bool vec = W % 4 == 0 && (W / groups) % 4 == 0 && ldx % 4 == 0 && (((uintptr_t)x) & 15) == 0;
    dim3 grid(b.n, vec ? (W + 1023) / 1024 : (W + 255) / 256);
    if (dt == WF_BF16) {
        if (vec) norm_taps_apply_kernel<__nv_bfloat16, 4><<<grid, 256, 0, s>>>(b, x, ldx, inv, (const __nv_bfloat16*)nw, groups, (const __nv_bfloat16*)cw, taps, W, state, slot_stride, (__nv_bfloat16*)out_t, ld_t, hn);
        else norm_taps_apply_kernel<__nv_bfloat16, 1><<<grid, 256, 0, s>>>(b, x, ldx, inv, (const __nv_bfloat16*)nw, groups, (const __nv_bfloat16*)cw, taps, W, state, slot_stride, (__nv_bfloat16*)out_t, ld_t, hn);
    } else {
        if (vec) norm_taps_apply_kernel<float, 4><<<grid, 256, 0, s>>>(b, x, ldx, inv, (const float*)nw, groups, (const float*)cw, taps, W, state, slot_stride, (float*)out_t, ld_t, hn);
        else norm_taps_apply_kernel<float, 1><<<grid, 256, 0, s>>>(b, x, ldx, inv, (const float*)nw, groups, (const float*)cw, taps, W, state, slot_stride, (float*)out_t, ld_t, hn);
    }
    return launch_check(cudaGetLastError(), "norm_taps_apply");
}

template <typename T>
__global__ void gate_mul_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ g, int ldg, int act, int C, T* __restrict__ y, int ldy) {
    const int i = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const float z = g[(size_t)i * ldg + c];
        y[(size_t)i * ldy + c] = from_f<T>(x[(size_t)i * ldx + c] * (act == 2 ? 1.f : (act ? silu_f(z) : sigmoid_f(z))));
    }
}

int launch_gate_mul(int dt, const float* x, int ldx, const float* g, int ldg, int act, int n, int C, void* y, int ldy, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    const dim3 grid(n, n < 64 ? (C + 255) / 256 : 1);
    if (dt == WF_BF16) gate_mul_kernel<<<grid, 256, 0, s>>>(x, ldx, g, ldg, act, C, (__nv_bfloat16*)y, ldy);
    else gate_mul_kernel<<<grid, 256, 0, s>>>(x, ldx, g, ldg, act, C, (float*)y, ldy);
    return launch_check(cudaGetLastError(), "gate_mul");
}

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, int ld, const int32_t* __restrict__ rows, int W, T* __restrict__ dst) {
    const int i = blockIdx.x, r = rows[i];
    for (int c = threadIdx.x; c < W; c += blockDim.x) dst[(size_t)i * W + c] = r >= 0 ? src[(size_t)r * ld + c] : from_f<T>(0.f);
}

int launch_gather_rows(int dt, const void* src, int ld, const int32_t* rows, int P, int W, void* dst, cudaStream_t s) {
    if (P <= 0) return WF_OK;
    if (dt == WF_BF16) gather_rows_kernel<<<P, 256, 0, s>>>((const __nv_bfloat16*)src, ld, rows, W, (__nv_bfloat16*)dst);
    else gather_rows_kernel<<<P, 256, 0, s>>>((const float*)src, ld, rows, W, (float*)dst);
    return launch_check(cudaGetLastError(), "gather_rows");
}

template <typename T>
__global__ void transpose_heads_kernel(const T* __restrict__ in, int R, int C, T* __restrict__ out) {
    const size_t h = blockIdx.y;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < R * C; idx += gridDim.x * blockDim.x) {
        const int r = idx / C, c = idx % C;
        out[h * R * C + (size_t)c * R + r] = in[h * R * C + idx];
    }
}

int launch_transpose_heads(int dt, const void* in, int H, int R, int C, void* out, cudaStream_t s) {
    dim3 grid((R * C + 255) / 256 > 1024 ? 1024 : (R * C + 255) / 256, H);
    if (dt == WF_BF16) transpose_heads_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)in, R, C, (__nv_bfloat16*)out);
    else transpose_heads_kernel<<<grid, 256, 0, s>>>((const float*)in, R, C, (float*)out);
    return launch_check(cudaGetLastError(), "transpose_heads");
}

}  // namespace seq
}  // namespace wf
