// Gated recurrences whose gates read only the current token, so that everything but a short linear chain runs in parallel over time.
//
//  * element-wise recurrence (minGRU form): S_t = (1 - z_t) S_(t-1) + z_t c_t per channel.  A block owns 32 (or 8) channels of one sequence
//    and cuts the portion into time slices, up to 64 of them: every slice first reduces itself to the pair (A, B) with S_end = A S_start + B,
//    the pairs are chained through shared memory, and every slice runs again from its start state for the outputs.
//  * matrix memory with exponential gating (mLSTM form): the log gates and their running maximum m_t = max(f_t + m_(t-1), i_t) are a
//    max-plus linear recurrence, scanned by a block per (sequence, head) whose warps take 32 tokens each; the matrix recurrence itself then is the
//    plain decayed outer-product accumulation of seq_delta.cu with keep = exp(f + m' - m) and put = exp(i - m), its normaliser n riding
//    along as one more value column.  The read-out (division, per-head unit RMS, weight, sigmoid gate) is one more row kernel.
// Gates, decays, exponentials, maxima and state are float in both storage modes.
#include "seq_kernels.cuh"
#include <math.h>

namespace wf {
namespace seq {

namespace {

constexpr int MG_MAXW = 16;     // most time slices (warps) of a block

constexpr int MG_UN = 8;        // tokens whose inputs are loaded before any of them is used: the loads do not wait for the chain

// ch: channels of a block (a power of two up to 32); a warp holds 32 / ch time slices of them.  Few channels per block make more blocks
// and more slices when one long portion has to fill the machine; 8 floats are still a whole 32-byte sector of a row.
template <typename T>
__global__ void __launch_bounds__(32 * MG_MAXW) mingru_kernel(Batch b, int C, int ch, const float* __restrict__ proj, int ld, int z_off, int x_off, int g_off,
                                                                const T* __restrict__ zb, const T* __restrict__ xb, float* __restrict__ state,
                                                                size_t slot_stride, T* __restrict__ out) {
    __shared__ float sA[32 * MG_MAXW], sB[32 * MG_MAXW];       // [slice][ch]
    const int sq = blockIdx.x, cl = threadIdx.x % ch, w = threadIdx.x / ch, nw = blockDim.x / ch;      // w: this thread's time slice of nw
    const int c = blockIdx.y * ch + cl;
    const bool ok = c < C;
    const int start = b.seq_start[sq], len = b.seq_len[sq];
    const int per = (len + nw - 1) / nw;
    const int t0 = w * per < len ? w * per : len, t1 = t0 + per < len ? t0 + per : len;
    float* Sp = state + (size_t)b.seq_slot[sq] * slot_stride + c;
    const float bz = ok ? to_f(zb[c]) : 0.f, bx = ok ? to_f(xb[c]) : 0.f;
    const float* base = proj + (size_t)start * ld + c;
    float S = 0.f;
    if (nw > 1) {
        // this slice as one affine map
        float A = 1.f, B = 0.f;
        if (ok)
            for (int t = t0; t < t1; t += MG_UN) {
                float zr[MG_UN], xr[MG_UN];
#pragma unroll
                for (int k = 0; k < MG_UN; ++k) { const bool in = t + k < t1; zr[k] = in ? base[(size_t)(t + k) * ld + z_off] : 0.f; xr[k] = in ? base[(size_t)(t + k) * ld + x_off] : 0.f; }
#pragma unroll
                for (int k = 0; k < MG_UN; ++k) {
                    if (t + k >= t1) break;
                    const float z = sigmoid_f(zr[k] + bz), u = xr[k] + bx;
                    const float keep = 1.f - z, put = z * (u >= 0.f ? u + 0.5f : sigmoid_f(u));
                    A *= keep;
                    B = fmaf(keep, B, put);
                }
            }
        sA[w * ch + cl] = A; sB[w * ch + cl] = B;
        __syncthreads();
        if (ok) {
            S = *Sp;
            for (int v = 0; v < w; ++v) S = fmaf(sA[v * ch + cl], S, sB[v * ch + cl]);
        }
    } else if (ok) S = *Sp;
    if (!ok) return;
    for (int t = t0; t < t1; t += MG_UN) {
        float zr[MG_UN], xr[MG_UN], gr[MG_UN];
#pragma unroll
        for (int k = 0; k < MG_UN; ++k) {
            const bool in = t + k < t1;
            const float* row = base + (size_t)(t + k) * ld;
            zr[k] = in ? row[z_off] : 0.f; xr[k] = in ? row[x_off] : 0.f; gr[k] = in ? row[g_off] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < MG_UN; ++k) {
            if (t + k >= t1) break;
            const float z = sigmoid_f(zr[k] + bz), u = xr[k] + bx;
            S = fmaf(1.f - z, S, z * (u >= 0.f ? u + 0.5f : sigmoid_f(u)));
            out[(size_t)(start + t + k) * C + c] = from_f<T>(S * silu_f(gr[k]));
        }
    }
    if (t1 == len && (t0 < t1 || w == 0)) *Sp = S;     // the slice that ends the portion leaves the state (empty slices behind it hold nothing)
}

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

constexpr int ML_MAXW = 32;

// One block per (sequence, head); its warps take 32 tokens each, side by side.  A token is the map m -> max(F + m, I) (F = log forget gate,
// I = log input gate); maps compose as (F1, I1) then (F2, I2) = (F1 + F2, max(F2 + I1, I2)).  Each warp scans its 32 maps with shuffles,
// the warps' totals are chained through shared memory, and the block walks the portion in passes of 32 tokens per warp.
template <typename T>
__global__ void __launch_bounds__(32 * ML_MAXW) mlstm_gates_kernel(Batch b, int H, const float* __restrict__ proj, int ld, int i_off, int f_off,
                                                                     const T* __restrict__ ib, const T* __restrict__ fb, float cap, float* __restrict__ mstate,
                                                                     size_t slot_stride, float* __restrict__ keep, float* __restrict__ put, float* __restrict__ mrun) {
    __shared__ float totF[ML_MAXW], totI[ML_MAXW];
    const int sq = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int start = b.seq_start[sq], len = b.seq_len[sq];
    float* mp = mstate + (size_t)b.seq_slot[sq] * slot_stride + h;
    float m = *mp;                          // every thread carries the block's running maximum
    const float bi = to_f(ib[h]), bf = to_f(fb[h]);
    for (int r0 = 0; r0 < len; r0 += 32 * nw) {
        const int t = r0 + w * 32 + lane;
        const bool ok = t < len;
        // tokens beyond the portion are the identity (F = 0, I = -inf)
        float li = -INFINITY, lf = 0.f;
        if (ok) {
            const float* row = proj + (size_t)(start + t) * ld;
            float zi = row[i_off + h] + bi, zf = row[f_off + h] + bf;
            if (cap > 0.f) { zi = cap * tanhf(zi / cap); zf = cap * tanhf(zf / cap); }
            li = zi; lf = log_sigmoid_f(zf);
        }
        float F = lf, I = li;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float Fp = __shfl_up_sync(0xffffffffu, F, o), Ip = __shfl_up_sync(0xffffffffu, I, o);
            if (lane >= o) { I = fmaxf(F + Ip, I); F = F + Fp; }
        }
        if (nw > 1) {
            if (lane == 31) { totF[w] = F; totI[w] = I; }
            __syncthreads();
        }
        float m_in = m;                     // the maximum before this warp's first token
        for (int v = 0; v < w; ++v) m_in = fmaxf(totF[v] + m_in, totI[v]);
        const float mt = fmaxf(F + m_in, I);
        float mprev = __shfl_up_sync(0xffffffffu, mt, 1);
        if (lane == 0) mprev = m_in;
        if (ok) {
            const size_t at = (size_t)(start + t) * H + h;
            keep[at] = expf(lf + mprev - mt);
            put[at] = expf(li - mt);
            mrun[at] = mt;
        }
        if (nw > 1) {
            for (int v = 0; v < nw; ++v) m = fmaxf(totF[v] + m, totI[v]);
            __syncthreads();                // the totals are overwritten in the next pass
        } else m = __shfl_sync(0xffffffffu, mt, 31);
    }
    if (threadIdx.x == 0) *mp = m;
}

// one warp per (token, head)
template <typename T>
__global__ void mlstm_post_kernel(int n, int H, int dv, const float* __restrict__ o, const float* __restrict__ mrun, float qscale, const T* __restrict__ w,
                                  float eps, const float* __restrict__ g, int ldg, T* __restrict__ y) {
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)n * H) return;
    const int i = (int)(unit / H), h = (int)(unit % H);
    const float* row = o + (size_t)unit * (dv + 1);
    const float den = fmaxf(fabsf(row[dv] * qscale), expf(-mrun[unit])) + 1e-6f;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) { const float v = row[c] * qscale / den; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
        const float v = row[c] * qscale / den;
        y[(size_t)unit * dv + c] = from_f<T>(v * inv * to_f(w[(size_t)h * dv + c]) * sigmoid_f(g[(size_t)i * ldg + (size_t)h * dv + c]));
    }
}

}  // namespace

int launch_mingru(int dt, const Batch& b, int C, const float* proj, int ld, int z_off, int x_off, int g_off, const void* zb, const void* xb,
                  float* state, size_t slot_stride, void* out, cudaStream_t s) {
    if (b.nseq <= 0) return WF_OK;
    if (C <= 0) { set_error("mingru: %d channels", C); return WF_ERR_INVALID; }
    // slices of at least 8 tokens; a block of single decoded tokens is one warp of 32 channels.  When long portions of few sequences
    // would leave most of the machine idle, a block takes 8 channels only: four times the blocks and, per warp, four times the slices.
    int ch = 32;
    if (b.max_len >= 256 && (long long)b.nseq * ((C + 31) / 32) < 2 * sm_count()) ch = 8;
    int nw = b.max_len / (8 * (32 / ch));
    nw = nw < 1 ? 1 : (nw > MG_MAXW ? MG_MAXW : nw);
    const dim3 grid(b.nseq, (C + ch - 1) / ch);
    if (dt == WF_BF16) mingru_kernel<<<grid, 32 * nw, 0, s>>>(b, C, ch, proj, ld, z_off, x_off, g_off, (const __nv_bfloat16*)zb, (const __nv_bfloat16*)xb, state, slot_stride, (__nv_bfloat16*)out);
    else mingru_kernel<<<grid, 32 * nw, 0, s>>>(b, C, ch, proj, ld, z_off, x_off, g_off, (const float*)zb, (const float*)xb, state, slot_stride, (float*)out);
    return launch_check(cudaGetLastError(), "mingru");
}

int launch_mlstm_gates(int dt, const Batch& b, int H, const float* proj, int ld, int i_off, int f_off, const void* ib, const void* fb, float cap,
                       float* mstate, size_t slot_stride, float* keep, float* put, float* mrun, cudaStream_t s) {
    if (b.nseq <= 0) return WF_OK;
    int nw = (b.max_len + 31) / 32;
    nw = nw < 1 ? 1 : (nw > ML_MAXW ? ML_MAXW : nw);
    const dim3 grid(b.nseq, H);
    if (dt == WF_BF16) mlstm_gates_kernel<<<grid, 32 * nw, 0, s>>>(b, H, proj, ld, i_off, f_off, (const __nv_bfloat16*)ib, (const __nv_bfloat16*)fb, cap, mstate, slot_stride, keep, put, mrun);
    else mlstm_gates_kernel<<<grid, 32 * nw, 0, s>>>(b, H, proj, ld, i_off, f_off, (const float*)ib, (const float*)fb, cap, mstate, slot_stride, keep, put, mrun);
    return launch_check(cudaGetLastError(), "mlstm_gates");
}

int launch_mlstm_post(int dt, int n, int H, int dv, const float* o, const float* mrun, float qscale, const void* w, float eps, const float* g, int ldg,
                      void* y, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    const long long units = (long long)n * H;
    const int blocks = (int)((units + 3) / 4);
    if (dt == WF_BF16) mlstm_post_kernel<<<blocks, 128, 0, s>>>(n, H, dv, o, mrun, qscale, (const __nv_bfloat16*)w, eps, g, ldg, (__nv_bfloat16*)y);
    else mlstm_post_kernel<<<blocks, 128, 0, s>>>(n, H, dv, o, mrun, qscale, (const float*)w, eps, g, ldg, (float*)y);
    return launch_check(cudaGetLastError(), "mlstm_post");
}

}  // namespace seq
}  // namespace wf
