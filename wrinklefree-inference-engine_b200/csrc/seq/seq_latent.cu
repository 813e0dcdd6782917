// Latent attention over a paged cache of (latent c_j, shared rotated key part kr_j) rows, with a sliding window.
// Per head the key is k_j = [W_uk c_j, kr_j] and the value W_uv c_j; neither is ever materialised: the query's unrotated part is carried
// through the key up-projection once (qa = W_uk^T q, a per-head batched product done by the caller), scores are qa . c_j + qr . kr_j, the
// weighted sum runs over the latents and the value up-projection is applied to that sum (again a batched product).  Scores, softmax and
// the weighted sum are float.  The rotated parts turn in pairs (i, i + dims / 2) or (2i, 2i + 1); with a frequency table (interpolated
// frequencies, tabulated once by the engine) the angle, cosine and sine of a pair are formed in double, once per token, and rounded once.
// A learned per-head sink adds exp(sink_h) to the softmax denominator.
#include "seq_kernels.cuh"
#include <math.h>

namespace wf {
namespace seq {

namespace {

constexpr int LA_MAXPAIRS = 128;   // rotated pairs of a head

// cosines and sines of one token's pairs into shared memory (the caller synchronises): from the frequency table in double, or from the
// base in float
__device__ __forceinline__ void rope_table(const LatentDims& L, int pos, float* cs, float* sn) {
    const int half = L.rope_dims / 2;
    for (int p = threadIdx.x; p < half; p += blockDim.x) {
        if (L.freq) {
            const double a = (double)pos * L.freq[p];
            cs[p] = (float)cos(a) * L.mscale; sn[p] = (float)sin(a) * L.mscale;
        } else {
            const float a = (float)pos * powf(L.rope_base, -2.0f * (float)p / (float)L.rope_dims);
            float s_, c_;
            sincosf(a, &s_, &c_);
            cs[p] = c_ * L.mscale; sn[p] = s_ * L.mscale;
        }
    }
}
// entry e of a rotated part `src` (r entries, the first rope_dims of them in pairs) after the rotation
__device__ __forceinline__ float rope_entry(const LatentDims& L, const float* __restrict__ src, int e, const float* cs, const float* sn) {
    if (e >= L.rope_dims) return src[e];
    const int half = L.rope_dims / 2;
    int p, other; bool first;
    if (L.interleaved) { p = e >> 1; other = e ^ 1; first = !(e & 1); }
    else { first = e < half; p = first ? e : e - half; other = first ? e + half : e - half; }
    return first ? src[e] * cs[p] - src[other] * sn[p] : src[e] * cs[p] + src[other] * sn[p];
}

template <typename T>
__global__ void latent_q_prep_kernel(Batch b, LatentDims L, const float* __restrict__ q, int ldq, T* __restrict__ qn, float* __restrict__ qr) {
    __shared__ float cs[LA_MAXPAIRS], sn[LA_MAXPAIRS];
    const int i = blockIdx.x;
    const int pos = b.tok_pos[i];
    const int per = L.d + L.r;
    rope_table(L, pos, cs, sn);
    __syncthreads();
    for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < L.H * per; idx += gridDim.y * blockDim.x) {
        const int h = idx / per, c = idx % per;
        const float* src = q + (size_t)i * ldq + (size_t)h * per;
        if (c < L.d) { qn[((size_t)i * L.H + h) * L.d + c] = from_f<T>(src[c]); continue; }
        qr[((size_t)i * L.H + h) * L.r + c - L.d] = rope_entry(L, src + L.d, c - L.d, cs, sn);
    }
}

// one block per token: latent RMS norm + rotary of the shared key part, stored as T in the token's cache row
template <typename T>
__global__ void latent_kv_write_kernel(Batch b, LatentDims L, const float* __restrict__ dkv, int ld, const T* __restrict__ w, float eps, PagedCache pc) {
    __shared__ float scratch[33];
    __shared__ float cs[LA_MAXPAIRS], sn[LA_MAXPAIRS];
    const int i = blockIdx.x;
    const int sq = b.tok_seq[i], pos = b.tok_pos[i];
    rope_table(L, pos, cs, sn);
    const int page = pc.block_table[(size_t)b.seq_slot[sq] * pc.max_blocks + pos / pc.page_size];
    T* row = (T*)pc.pool + (size_t)page * pc.page_stride + pc.layer_off + (size_t)(pos % pc.page_size) * (L.R + L.r);
    const float* src = dkv + (size_t)i * ld;
    float ss = 0.f;
    for (int c = threadIdx.x; c < L.R; c += blockDim.x) ss += src[c] * src[c];
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)L.R + eps);
    for (int c = threadIdx.x; c < L.R; c += blockDim.x) row[c] = from_f<T>(src[c] * inv * to_f(w[c]));
    // (block_sum has synchronised the block since the table was written)
    for (int e = threadIdx.x; e < L.r; e += blockDim.x) row[L.R + e] = from_f<T>(rope_entry(L, src + L.R, e, cs, sn));
}

constexpr int LA_WARPS = 4;
constexpr int LA_MAXR = 16;    // latent size up to 32 * 16
constexpr int LA_MAXr = 8;     // rotated size up to 32 * 8

// One block per (token, head).  Its warps take the visible positions round-robin; a warp handles one position at a time with its lanes
// over the dimensions (coalesced reads of the cache row), keeps a running max / sum / weighted latent sum, and the warps' partial results
// are merged through shared memory at the end.
template <typename T>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attn_kernel(Batch b, LatentDims L, const float* __restrict__ qa, const float* __restrict__ qr,
                                                                      PagedCache pc, T* __restrict__ out) {
    extern __shared__ float sm[];   // [LA_WARPS][R] partial sums, then [LA_WARPS] m, [LA_WARPS] l
    const int i = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sq = b.tok_seq[i], pos = b.tok_pos[i];
    const int lo = pos - L.window + 1 > 0 ? pos - L.window + 1 : 0;
    const int32_t* bt = pc.block_table + (size_t)b.seq_slot[sq] * pc.max_blocks;
    const int width = L.R + L.r;
    const float* qa_h = qa + ((size_t)i * L.H + h) * L.R;
    const float* qr_h = qr + ((size_t)i * L.H + h) * L.r;
    float qreg[LA_MAXR], rreg[LA_MAXr], acc[LA_MAXR];
#pragma unroll
    for (int t = 0; t < LA_MAXR; ++t) { const int c = lane + 32 * t; qreg[t] = c < L.R ? qa_h[c] : 0.f; acc[t] = 0.f; }
#pragma unroll
    for (int t = 0; t < LA_MAXr; ++t) { const int c = lane + 32 * t; rreg[t] = c < L.r ? qr_h[c] : 0.f; }
    float m = -INFINITY, l = 0.f;
    for (int j = lo + warp; j <= pos; j += LA_WARPS) {
        const int page = bt[j / pc.page_size];
        const T* row = (const T*)pc.pool + (size_t)page * pc.page_stride + pc.layer_off + (size_t)(j % pc.page_size) * width;
        float cv[LA_MAXR];
        float part = 0.f;
#pragma unroll
        for (int t = 0; t < LA_MAXR; ++t) {
            const int c = lane + 32 * t;
            cv[t] = c < L.R ? to_f(row[c]) : 0.f;
            part = fmaf(qreg[t], cv[t], part);
        }
#pragma unroll
        for (int t = 0; t < LA_MAXr; ++t) {
            const int c = lane + 32 * t;
            if (c < L.r) part = fmaf(rreg[t], to_f(row[L.R + c]), part);
        }
        const float sc = warp_sum(part) * L.scale;
        const float mn = fmaxf(m, sc);
        const float corr = expf(m - mn);      // m = -inf on the first position: exp(-inf) = 0
        const float p = expf(sc - mn);
        l = l * corr + p;
#pragma unroll
        for (int t = 0; t < LA_MAXR; ++t) acc[t] = fmaf(p, cv[t], acc[t] * corr);
        m = mn;
    }
    float* part_sum = sm;
    float* part_m = sm + LA_WARPS * L.R;
    float* part_l = part_m + LA_WARPS;
#pragma unroll
    for (int t = 0; t < LA_MAXR; ++t) { const int c = lane + 32 * t; if (c < L.R) part_sum[warp * L.R + c] = acc[t]; }
    if (lane == 0) { part_m[warp] = m; part_l[warp] = l; }
    __syncthreads();
    float mg = -INFINITY;
#pragma unroll
    for (int w = 0; w < LA_WARPS; ++w) mg = fmaxf(mg, part_m[w]);
    float lg = 0.f, sc_w[LA_WARPS];
#pragma unroll
    for (int w = 0; w < LA_WARPS; ++w) { sc_w[w] = part_m[w] == -INFINITY ? 0.f : expf(part_m[w] - mg); lg += part_l[w] * sc_w[w]; }
    if (L.sink) lg += expf(L.sink[h] - mg);      // the sink: a weight without a value
    const float inv = 1.f / lg;
    for (int c = threadIdx.x; c < L.R; c += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < LA_WARPS; ++w) v += part_sum[w * L.R + c] * sc_w[w];
        out[((size_t)i * L.H + h) * L.R + c] = from_f<T>(v * inv);
    }
}

int check_dims(const LatentDims& L) {
    if (L.R > 32 * LA_MAXR || L.r > 32 * LA_MAXr) { set_error("latent attention: kv_rank %d / rot_dim %d above the supported %d / %d", L.R, L.r, 32 * LA_MAXR, 32 * LA_MAXr); return WF_ERR_UNSUPPORTED; }
    if (L.rope_dims / 2 > LA_MAXPAIRS) { set_error("latent attention: %d rotated pairs above the supported %d", L.rope_dims / 2, LA_MAXPAIRS); return WF_ERR_UNSUPPORTED; }
    if (L.rope_dims > L.r || (L.rope_dims & 1) || L.window < 1) { set_error("latent attention: rotary dims %d of %d, window %d", L.rope_dims, L.r, L.window); return WF_ERR_INVALID; }
    return WF_OK;
}

}  // namespace

int launch_latent_q_prep(int dt, const Batch& b, const LatentDims& L, const float* q, int ldq, void* qn, float* qr, cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (int rc = check_dims(L)) return rc;
    const dim3 grid(b.n, b.n < 64 ? (L.H * (L.d + L.r) + 255) / 256 : 1);
    if (dt == WF_BF16) latent_q_prep_kernel<<<grid, 256, 0, s>>>(b, L, q, ldq, (__nv_bfloat16*)qn, qr);
    else latent_q_prep_kernel<<<grid, 256, 0, s>>>(b, L, q, ldq, (float*)qn, qr);
    return launch_check(cudaGetLastError(), "latent_q_prep");
}

int launch_latent_kv_write(int dt, const Batch& b, const LatentDims& L, const float* dkv, int ld, const void* w, float eps, const PagedCache& pc,
                           cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (int rc = check_dims(L)) return rc;
    if (dt == WF_BF16) latent_kv_write_kernel<<<b.n, 128, 0, s>>>(b, L, dkv, ld, (const __nv_bfloat16*)w, eps, pc);
    else latent_kv_write_kernel<<<b.n, 128, 0, s>>>(b, L, dkv, ld, (const float*)w, eps, pc);
    return launch_check(cudaGetLastError(), "latent_kv_write");
}

int launch_latent_attn(int dt, const Batch& b, const LatentDims& L, const float* qa, const float* qr, const PagedCache& pc, void* out, cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (int rc = check_dims(L)) return rc;
    if (L.H > 65535) { set_error("latent attention: too many heads"); return WF_ERR_UNSUPPORTED; }
    dim3 grid(b.n, L.H);
    const size_t smem = ((size_t)LA_WARPS * L.R + 2 * LA_WARPS) * sizeof(float);
    if (dt == WF_BF16) latent_attn_kernel<<<grid, LA_WARPS * 32, smem, s>>>(b, L, qa, qr, pc, (__nv_bfloat16*)out);
    else latent_attn_kernel<<<grid, LA_WARPS * 32, smem, s>>>(b, L, qa, qr, pc, (float*)out);
    return launch_check(cudaGetLastError(), "latent_attn");
}

}  // namespace seq
}  // namespace wf
