// Gated delta rule: a per-head matrix state S [d, dv] in float that every token first decays (one factor per head, or one per head and key
// row), then corrects along its key (u = beta (v - S^T k), S += k u^T) and finally reads with its query (o = S^T q).  The same kernel
// without the correction (u = beta v) is the state-space recurrence S = a S + dt B x^T, y = S^T C with k = B, q = C, v = x, beta = dt.
// The state is carried per sequence slot across steps.
#include "seq_kernels.cuh"

namespace wf {
namespace seq {

namespace {

// one block per token: unit-normalise the q and k heads in place, compute the write strength and the decay of every head
template <typename T>
__global__ void delta_prep_kernel(DeltaDims D, float* __restrict__ qkv, int ld, const float* __restrict__ a_raw, int lda, const float* __restrict__ b_raw,
                                  int ldb, const T* __restrict__ A_log, const T* __restrict__ dt_bias, float* __restrict__ beta, float* __restrict__ decay) {
    const int i = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float* row = qkv + (size_t)i * ld;
    const float qscale = 1.f / sqrtf((float)D.d);
    for (int v = warp; v < 2 * D.Hk; v += nw) {          // vectors 0 .. Hk-1 are q heads, Hk .. 2Hk-1 are k heads
        float* x = row + (size_t)v * D.d;
        float ss = 0.f;
        for (int c = lane; c < D.d; c += 32) ss += x[c] * x[c];
        ss = warp_sum(ss);
        const float inv = (v < D.Hk ? qscale : 1.f) / sqrtf(ss + 1e-6f);
        for (int c = lane; c < D.d; c += 32) x[c] *= inv;
    }
    for (int h = threadIdx.x; h < D.H; h += blockDim.x) beta[(size_t)i * D.H + h] = sigmoid_f(b_raw[(size_t)i * ldb + h]);
    const int nd = D.vec_decay ? D.H * D.d : D.H;         // one decay per head, or per head and key channel
    for (int k = threadIdx.x; k < nd; k += blockDim.x) {
        const int h = D.vec_decay ? k / D.d : k;
        const float sp = softplus_f(a_raw[(size_t)i * lda + k] + to_f(dt_bias[k]));
        decay[(size_t)i * nd + k] = expf(-expf(to_f(A_log[h])) * sp);
    }
}

// state-space recurrence: the step size and the decay of every head
template <typename T>
__global__ void ssd_prep_kernel(int n, int H, const float* __restrict__ dt_raw, int ld, const T* __restrict__ A_log, const T* __restrict__ dt_bias,
                                float* __restrict__ step, float* __restrict__ decay) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= n * H) return;
    const int i = k / H, h = k - i * H;
    const float z = dt_raw[(size_t)i * ld + h] + to_f(dt_bias[h]);
    const float sp = z > 20.f ? z : log1pf(expf(z));     // softplus without a clamp
    step[k] = sp;
    decay[k] = expf(-expf(to_f(A_log[h])) * sp);
}

// one block per (token, norm group): v = (o + D_h x) * silu(z), divided by the root mean square of the group, times the weight
template <typename T>
__global__ void ssd_post_kernel(int H, int dv, int groups, const float* __restrict__ o, const float* __restrict__ x, int ldx, const float* __restrict__ z, int ldz,
                                const T* __restrict__ Dskip, const T* __restrict__ w, float eps, T* __restrict__ y) {
    __shared__ float scratch[33];
    const int i = blockIdx.x, g = blockIdx.y;
    const int inner = H * dv, gw = inner / groups;
    float ss = 0.f;
    for (int c = g * gw + threadIdx.x; c < (g + 1) * gw; c += blockDim.x) {
        const float xv = x[(size_t)i * ldx + c];
        const float v = (o[(size_t)i * inner + c] + to_f(Dskip[c / dv]) * xv) * silu_f(z[(size_t)i * ldz + c]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)gw + eps);
    for (int c = g * gw + threadIdx.x; c < (g + 1) * gw; c += blockDim.x) {
        const float xv = x[(size_t)i * ldx + c];
        const float v = (o[(size_t)i * inner + c] + to_f(Dskip[c / dv]) * xv) * silu_f(z[(size_t)i * ldz + c]);
        y[(size_t)i * inner + c] = from_f<T>(v * inv * to_f(w[c]));
    }
}

constexpr int DR_THREADS = 128, DR_TT = 16;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

// chunked run of a linear recurrence: pass 0 = whole portions in order (no chunks); pass 1 = a block takes one chunk from a ZERO state and
// leaves its end state (and the product of its decays) in the workspace; pass 3 = a block takes one chunk from the start state that
// scan_prefix_kernel chained and writes the outputs.  Workspace entry of (sequence, chunk): seq_start / chunk + sequence + chunk, which
// never collides between sequences and stays below tokens / chunk + sequences.
struct ScanArgs { int pass = 0, chunk = 0, nchunks = 1; float* local = nullptr; float* start = nullptr; float* prod = nullptr;
                  int v4 = 0; };   // v4: every staged row starts 16-byte aligned and has a multiple of 4 entries (16-byte copies)

__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

// block = (sequence, head, 16 value columns); thread = (column, eighth of the key rows: DPT consecutive ones), its part of the column in registers.
// Tokens are taken 16 at a time: the next group's k / q / v / gates are copied into the other half of shared memory (cp.async)
// while the current group runs, so the per-token chain is only register math, 16-byte shared-memory reads and two quad reductions.
// DR_PARTS = 8 (16 columns per block): short per-token chains and twice the blocks, for portions of many tokens;
// DR_PARTS = 4 (32 columns): wider, better coalesced state rows, for single decoded tokens where the state traffic is the cost.
// VEC: the decay is a vector over the key rows (staged per token like k and q) instead of one number per token.
// DELTA: the write is corrected by what the state already holds along the key (the delta rule); without it u = beta v.
template <int DPT, int DR_PARTS, bool VEC, bool DELTA>
__global__ void __launch_bounds__(DR_THREADS) delta_rule_kernel(Batch b, DeltaDims D, const float* __restrict__ qkv, int ld,
                                                                         const float* __restrict__ beta, const float* __restrict__ decay,
                                                                         float* __restrict__ state, size_t slot_stride, float* __restrict__ o, ScanArgs sa) {
    constexpr int DR_COLS = DR_THREADS / DR_PARTS;
    extern __shared__ __align__(16) float sm[];
    // A thread owns DPT consecutive key rows; a token's k / q / decay rows lie in shared memory with 4 floats of padding after every DPT, so
    // that the eight (or four) threads of a column read their parts as 16-byte vectors from distinct banks.
    constexpr int PS = DPT + 4, RS = DR_PARTS * PS;           // floats per part and per token row
    constexpr int tile_floats = (VEC ? 3 : 2) * DR_TT * RS + DR_TT * DR_COLS + 2 * DR_TT;   // k [TT][RS], q [TT][RS], v [TT][cols], beta [TT], decay [TT], vector decay [TT][RS]
    const int sq = sa.pass ? blockIdx.x / sa.nchunks : blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DR_COLS;
    const int tid = threadIdx.x, p = tid % DR_PARTS, jl = tid / DR_PARTS, col = col0 + jl;
    const int dvs = D.dv + D.ones_col;                      // state and output columns: the values, and the all-ones column behind them
    const bool col_ok = col < dvs;
    const int kh = h / (D.H / D.Hk);
    int start = b.seq_start[sq], len = b.seq_len[sq];
    float* S = state + (size_t)b.seq_slot[sq] * slot_stride + (size_t)h * D.d * dvs;       // where the state is read ...
    float* S_out = S;                                                                        // ... and where it is left
    if (sa.pass) {
        const int c = blockIdx.x - sq * sa.nchunks;
        if (c * sa.chunk >= len) return;                                                     // the whole block: this sequence has fewer chunks
        const size_t entry = ((size_t)(start / sa.chunk + sq + c) * D.H + h) * D.d * dvs;
        S = sa.pass == 1 ? nullptr : sa.start + entry;
        S_out = sa.pass == 1 ? sa.local + entry : nullptr;
        if (sa.pass == 1 && tid == 0 && blockIdx.z == 0) {                                   // the chunk's decay product (one decay per head)
            float pr = 1.f;
            const int t1 = len - c * sa.chunk < sa.chunk ? len - c * sa.chunk : sa.chunk;
            for (int t = 0; t < t1; ++t) pr *= decay[(size_t)(start + c * sa.chunk + t) * D.H + h];
            sa.prod[(size_t)(start / sa.chunk + sq + c) * D.H + h] = pr;
        }
        start += c * sa.chunk;
        len = len - c * sa.chunk < sa.chunk ? len - c * sa.chunk : sa.chunk;
    }
    float s[DPT];
#pragma unroll
    for (int m = 0; m < DPT; ++m) {
        const int i = p * DPT + m;
        s[m] = (S && col_ok && i < D.d) ? S[(size_t)i * dvs + col] : 0.f;
    }
    const int q_off = (D.q_off >= 0 ? D.q_off : 0) + kh * D.d, k_off = (D.k_off >= 0 ? D.k_off : D.Hk * D.d) + kh * D.d,
              v_off = (D.v_off >= 0 ? D.v_off : 2 * D.Hk * D.d) + h * D.dv;
    auto stage = [&](int buf, int t0) {
        float* ks = sm + (size_t)buf * tile_floats;
        float* qs = ks + DR_TT * RS;
        float* vs = qs + DR_TT * RS;
        float* bs = vs + DR_TT * DR_COLS;
        float* gs = bs + DR_TT;
        float* gv = gs + DR_TT;
        const int tt = len - t0 < DR_TT ? len - t0 : DR_TT;
        if (sa.v4) {
            const int d4 = D.d >> 2;
            for (int idx = tid; idx < tt * d4; idx += blockDim.x) {
                const int t = idx / d4, c = (idx - t * d4) << 2;
                const int at = t * RS + c + (c / DPT) * 4;    // the padded place of rows c .. c + 3 (DPT is a multiple of 4: one part holds them)
                const float* row = qkv + (size_t)(start + t0 + t) * ld;
                cp_async16(ks + at, row + k_off + c);
                cp_async16(qs + at, row + q_off + c);
                if (VEC) cp_async16(gv + at, decay + ((size_t)(start + t0 + t) * D.H + h) * D.d + c);
            }
            for (int idx = tid; idx < tt * (DR_COLS / 4); idx += blockDim.x) {
                const int t = idx / (DR_COLS / 4), c = (idx % (DR_COLS / 4)) << 2;
                if (col0 + c < D.dv) cp_async16(vs + t * DR_COLS + c, qkv + (size_t)(start + t0 + t) * ld + v_off + col0 + c);
                else {
#pragma unroll
                    for (int k = 0; k < 4; ++k) vs[t * DR_COLS + c + k] = (D.ones_col && col0 + c + k == D.dv) ? 1.f : 0.f;
                }
            }
        } else {
            for (int idx = tid; idx < tt * D.d; idx += blockDim.x) {
                const int t = idx / D.d, c = idx - t * D.d;
                const int at = t * RS + c + (c / DPT) * 4;    // the padded place of row c
                const float* row = qkv + (size_t)(start + t0 + t) * ld;
                cp_async4(ks + at, row + k_off + c);
                cp_async4(qs + at, row + q_off + c);
                if (VEC) cp_async4(gv + at, decay + ((size_t)(start + t0 + t) * D.H + h) * D.d + c);
            }
            for (int idx = tid; idx < tt * DR_COLS; idx += blockDim.x) {
                const int t = idx / DR_COLS, c = idx % DR_COLS;
                if (col0 + c < D.dv) cp_async4(vs + idx, qkv + (size_t)(start + t0 + t) * ld + v_off + col0 + c);
                else vs[idx] = (D.ones_col && col0 + c == D.dv) ? 1.f : 0.f;
            }
        }
        if (tid < tt) {
            cp_async4(bs + tid, beta + (size_t)(start + t0 + tid) * D.H + h);
            if (!VEC) cp_async4(gs + tid, decay + (size_t)(start + t0 + tid) * D.H + h);
        }
        cp_async_commit();
    };
    if (len > 0) stage(0, 0);
    int buf = 0;
    for (int t0 = 0; t0 < len; t0 += DR_TT, buf ^= 1) {
        const int tt = len - t0 < DR_TT ? len - t0 : DR_TT;
        cp_async_wait<0>();
        __syncthreads();                                      // group t0 landed; everyone is done with the other half
        if (t0 + DR_TT < len) stage(buf ^ 1, t0 + DR_TT);
        const float* ks = sm + (size_t)buf * tile_floats;
        const float* qs = ks + DR_TT * RS;
        const float* vs = qs + DR_TT * RS;
        const float* bs = vs + DR_TT * DR_COLS;
        const float* gs = bs + DR_TT;
        const float* gv = gs + DR_TT;
        const int i0 = p * DPT;                               // this thread's first key row
        for (int t = 0; t < tt; ++t) {
            const float4* kt = reinterpret_cast<const float4*>(ks + t * RS + p * PS);
            const float4* qt = reinterpret_cast<const float4*>(qs + t * RS + p * PS);
            const float4* gt = reinterpret_cast<const float4*>(gv + t * RS + p * PS);
            const float g = VEC ? 1.f : gs[t];
            // rows at and beyond D.d hold a zero state and stay zero: what the padding or an unstaged row holds never reaches them
            if (VEC) {                                        // the rows decay first, each by its own factor
#pragma unroll
                for (int m4 = 0; m4 < DPT / 4; ++m4) {
                    const float4 gg = gt[m4];
                    const int i = i0 + 4 * m4;
                    if (i < D.d) s[4 * m4] *= gg.x;
                    if (i + 1 < D.d) s[4 * m4 + 1] *= gg.y;
                    if (i + 2 < D.d) s[4 * m4 + 2] *= gg.z;
                    if (i + 3 < D.d) s[4 * m4 + 3] *= gg.w;
                }
            }
            float rs = 0.f;
            if (DELTA) {
                float r[4] = {0.f, 0.f, 0.f, 0.f};            // four chains: the sum over this thread's rows is not one dependent sequence
#pragma unroll
                for (int m4 = 0; m4 < DPT / 4; ++m4) {
                    const float4 kk = kt[m4];
                    const int i = i0 + 4 * m4;
                    if (i < D.d) r[0] = fmaf(s[4 * m4], kk.x, r[0]);
                    if (i + 1 < D.d) r[1] = fmaf(s[4 * m4 + 1], kk.y, r[1]);
                    if (i + 2 < D.d) r[2] = fmaf(s[4 * m4 + 2], kk.z, r[2]);
                    if (i + 3 < D.d) r[3] = fmaf(s[4 * m4 + 3], kk.w, r[3]);
                }
                rs = (r[0] + r[1]) + (r[2] + r[3]);
                rs += __shfl_xor_sync(0xffffffffu, rs, 1);
                rs += __shfl_xor_sync(0xffffffffu, rs, 2);
                if (DR_PARTS == 8) rs += __shfl_xor_sync(0xffffffffu, rs, 4);
            }
            const float u = bs[t] * (vs[t * DR_COLS + jl] - g * rs);
            if (sa.pass == 1) {                               // only the end state is wanted: no read-out
#pragma unroll
                for (int m4 = 0; m4 < DPT / 4; ++m4) {
                    const float4 kk = kt[m4];
                    const int i = i0 + 4 * m4;
                    if (i < D.d) s[4 * m4] = fmaf(kk.x, u, g * s[4 * m4]);
                    if (i + 1 < D.d) s[4 * m4 + 1] = fmaf(kk.y, u, g * s[4 * m4 + 1]);
                    if (i + 2 < D.d) s[4 * m4 + 2] = fmaf(kk.z, u, g * s[4 * m4 + 2]);
                    if (i + 3 < D.d) s[4 * m4 + 3] = fmaf(kk.w, u, g * s[4 * m4 + 3]);
                }
                continue;
            }
            float out[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int m4 = 0; m4 < DPT / 4; ++m4) {
                const float4 kk = kt[m4], qq = qt[m4];
                const int i = i0 + 4 * m4;
                if (i < D.d) { s[4 * m4] = fmaf(kk.x, u, g * s[4 * m4]); out[0] = fmaf(s[4 * m4], qq.x, out[0]); }
                if (i + 1 < D.d) { s[4 * m4 + 1] = fmaf(kk.y, u, g * s[4 * m4 + 1]); out[1] = fmaf(s[4 * m4 + 1], qq.y, out[1]); }
                if (i + 2 < D.d) { s[4 * m4 + 2] = fmaf(kk.z, u, g * s[4 * m4 + 2]); out[2] = fmaf(s[4 * m4 + 2], qq.z, out[2]); }
                if (i + 3 < D.d) { s[4 * m4 + 3] = fmaf(kk.w, u, g * s[4 * m4 + 3]); out[3] = fmaf(s[4 * m4 + 3], qq.w, out[3]); }
            }
            float os = (out[0] + out[1]) + (out[2] + out[3]);
            os += __shfl_xor_sync(0xffffffffu, os, 1);
            os += __shfl_xor_sync(0xffffffffu, os, 2);
            if (DR_PARTS == 8) os += __shfl_xor_sync(0xffffffffu, os, 4);
            if (p == 0 && col_ok) o[((size_t)(start + t0 + t) * D.H + h) * dvs + col] = os;
        }
    }
    if (!S_out) return;
#pragma unroll
    for (int m = 0; m < DPT; ++m) {
        const int i = p * DPT + m;
        if (col_ok && i < D.d) S_out[(size_t)i * dvs + col] = s[m];
    }
}

// thread per (sequence, head, state element): chains the chunks' start states from the slot's state and leaves the end state in the slot
__global__ void scan_prefix_kernel(Batch b, int H, int dd, int chunk, float* __restrict__ state, size_t slot_stride, const float* __restrict__ local,
                                   float* __restrict__ startws, const float* __restrict__ prod) {
    const int sq = blockIdx.x, h = blockIdx.y, e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= dd) return;
    const int len = b.seq_len[sq], nc = (len + chunk - 1) / chunk, base = b.seq_start[sq] / chunk + sq;
    float* Sp = state + (size_t)b.seq_slot[sq] * slot_stride + (size_t)h * dd + e;
    float S = *Sp;
    for (int c = 0; c < nc; ++c) {
        const size_t entry = (size_t)(base + c) * H + h;
        startws[entry * dd + e] = S;
        S = fmaf(prod[entry], S, local[entry * dd + e]);
    }
    *Sp = S;
}

template <typename T>
__global__ void delta_post_kernel(DeltaDims D, const float* __restrict__ o, const T* __restrict__ w, float eps, const float* __restrict__ g, int ldg,
                                  T* __restrict__ y, int act) {
    const int i = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int h = blockIdx.y * nw + warp; h < D.H; h += gridDim.y * nw) {
        const float* x = o + ((size_t)i * D.H + h) * D.dv;
        float ss = 0.f;
        for (int c = lane; c < D.dv; c += 32) ss += x[c] * x[c];
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)D.dv + eps);
        for (int c = lane; c < D.dv; c += 32) {
            const float z = g[(size_t)i * ldg + (size_t)h * D.dv + c];
            y[((size_t)i * D.H + h) * D.dv + c] = from_f<T>(x[c] * inv * to_f(w[c]) * (act ? sigmoid_f(z) : silu_f(z)));
        }
    }
}

}  // namespace

int launch_delta_prep(int dt, const DeltaDims& D, int n, float* qkv, int ld, const float* a_raw, int lda, const float* b_raw, int ldb_,
                      const void* A_log, const void* dt_bias, float* beta, float* decay, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    if (D.Hk <= 0 || D.H % D.Hk) { set_error("delta: %d heads over %d key heads", D.H, D.Hk); return WF_ERR_INVALID; }
    if (dt == WF_BF16) delta_prep_kernel<<<n, 128, 0, s>>>(D, qkv, ld, a_raw, lda, b_raw, ldb_, (const __nv_bfloat16*)A_log, (const __nv_bfloat16*)dt_bias, beta, decay);
    else delta_prep_kernel<<<n, 128, 0, s>>>(D, qkv, ld, a_raw, lda, b_raw, ldb_, (const float*)A_log, (const float*)dt_bias, beta, decay);
    return launch_check(cudaGetLastError(), "delta_prep");
}

namespace {
template <bool VEC, bool DELTA>
int delta_rule_launch(const Batch& b, const DeltaDims& D, const float* qkv, int ld, const float* beta, const float* decay, float* state,
                      size_t slot_stride, float* o, cudaStream_t s, ScanArgs sa = ScanArgs()) {
    const bool decode = b.n == b.nseq;                     // every sequence brings one token
    const int parts = decode ? 4 : 8, cols = DR_THREADS / parts;
    dim3 grid(sa.pass ? b.nseq * sa.nchunks : b.nseq, D.H, (D.dv + D.ones_col + cols - 1) / cols);
    const int dpt_raw = (D.d + parts - 1) / parts, dpt_t = dpt_raw <= 8 ? 8 : (dpt_raw <= 16 ? 16 : (dpt_raw <= 32 ? 32 : 64));
    const size_t smem = 2 * ((size_t)(VEC ? 3 : 2) * DR_TT * parts * (dpt_t + 4) + DR_TT * cols + 2 * DR_TT) * sizeof(float);   // two token groups, padded rows
    static DevOnce once;
    if (once.need()) {
#define DR_ATTR(dp, pa) cudaFuncSetAttribute(delta_rule_kernel<dp, pa, VEC, DELTA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)
        DR_ATTR(8, 8); DR_ATTR(16, 8); DR_ATTR(32, 8); DR_ATTR(64, 8); DR_ATTR(8, 4); DR_ATTR(16, 4); DR_ATTR(32, 4); DR_ATTR(64, 4);
#undef DR_ATTR
    }
    const int dpt = (D.d + parts - 1) / parts;
    {   // 16-byte staging copies when every row the kernel stages starts aligned and has a multiple of 4 entries
        const int qo = D.q_off >= 0 ? D.q_off : 0, ko = D.k_off >= 0 ? D.k_off : D.Hk * D.d, vo = D.v_off >= 0 ? D.v_off : 2 * D.Hk * D.d;
        sa.v4 = D.d % 4 == 0 && D.dv % 4 == 0 && ld % 4 == 0 && qo % 4 == 0 && ko % 4 == 0 && vo % 4 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)decay & 15) == 0;
    }
#define DR_LAUNCH(dp, pa) delta_rule_kernel<dp, pa, VEC, DELTA><<<grid, DR_THREADS, smem, s>>>(b, D, qkv, ld, beta, decay, state, slot_stride, o, sa)
    if (D.d > 256 || smem > 160 * 1024) { set_error("delta: key dimension %d above the supported 256", D.d); return WF_ERR_UNSUPPORTED; }
    if (decode) { if (dpt <= 8) DR_LAUNCH(8, 4); else if (dpt <= 16) DR_LAUNCH(16, 4); else if (dpt <= 32) DR_LAUNCH(32, 4); else DR_LAUNCH(64, 4); }
    else { if (dpt <= 8) DR_LAUNCH(8, 8); else if (dpt <= 16) DR_LAUNCH(16, 8); else if (dpt <= 32) DR_LAUNCH(32, 8); else DR_LAUNCH(64, 8); }
#undef DR_LAUNCH
    return launch_check(cudaGetLastError(), "delta_rule");
}
}  // namespace

int launch_delta_rule(const Batch& b, const DeltaDims& D, const float* qkv, int ld, const float* beta, const float* decay, float* state,
                      size_t slot_stride, float* o, cudaStream_t s, const ScanWorkspace* scan) {
    if (b.nseq <= 0) return WF_OK;
    if (D.Hk <= 0 || D.H % D.Hk) { set_error("delta: %d heads over %d key heads", D.H, D.Hk); return WF_ERR_INVALID; }
    if (D.ones_col && !D.no_delta) { set_error("delta: the all-ones column belongs to the plain recurrence"); return WF_ERR_UNSUPPORTED; }
    if (D.no_delta) {
        if (D.vec_decay) { set_error("delta: the plain recurrence takes one decay per head"); return WF_ERR_UNSUPPORTED; }
        // long portions: chunks in parallel (two short sequential passes instead of one long one)
        if (scan && scan->local && b.n != b.nseq && b.max_len >= 2 * SCAN_CHUNK && b.n / SCAN_CHUNK + b.nseq + 1 <= scan->chunks) {
            ScanArgs sa;
            sa.chunk = SCAN_CHUNK; sa.nchunks = (b.max_len + SCAN_CHUNK - 1) / SCAN_CHUNK;
            sa.local = scan->local; sa.start = scan->start; sa.prod = scan->prod;
            sa.pass = 1;
            if (int rc = delta_rule_launch<false, false>(b, D, qkv, ld, beta, decay, state, slot_stride, o, s, sa)) return rc;
            const int dd = D.d * (D.dv + D.ones_col);
            scan_prefix_kernel<<<dim3(b.nseq, D.H, (dd + 255) / 256), 256, 0, s>>>(b, D.H, dd, SCAN_CHUNK, state, slot_stride, scan->local, scan->start, scan->prod);
            if (int rc = launch_check(cudaGetLastError(), "scan_prefix")) return rc;
            sa.pass = 3;
            return delta_rule_launch<false, false>(b, D, qkv, ld, beta, decay, state, slot_stride, o, s, sa);
        }
        return delta_rule_launch<false, false>(b, D, qkv, ld, beta, decay, state, slot_stride, o, s);
    }
    return D.vec_decay ? delta_rule_launch<true, true>(b, D, qkv, ld, beta, decay, state, slot_stride, o, s)
                       : delta_rule_launch<false, true>(b, D, qkv, ld, beta, decay, state, slot_stride, o, s);
}

int launch_delta_post(int dt, const DeltaDims& D, int n, const float* o, const void* w, float eps, const float* g, int ldg, void* y, cudaStream_t s, int act) {
    if (n <= 0) return WF_OK;
    const dim3 grid(n, n < 64 ? (D.H + 3) / 4 : 1);
    if (dt == WF_BF16) delta_post_kernel<<<grid, 128, 0, s>>>(D, o, (const __nv_bfloat16*)w, eps, g, ldg, (__nv_bfloat16*)y, act);
    else delta_post_kernel<<<grid, 128, 0, s>>>(D, o, (const float*)w, eps, g, ldg, (float*)y, act);
    return launch_check(cudaGetLastError(), "delta_post");
}

int launch_ssd_prep(int dt, int n, int H, const float* dt_raw, int ld, const void* A_log, const void* dt_bias, float* step, float* decay, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    const int blocks = (n * H + 127) / 128;
    if (dt == WF_BF16) ssd_prep_kernel<<<blocks, 128, 0, s>>>(n, H, dt_raw, ld, (const __nv_bfloat16*)A_log, (const __nv_bfloat16*)dt_bias, step, decay);
    else ssd_prep_kernel<<<blocks, 128, 0, s>>>(n, H, dt_raw, ld, (const float*)A_log, (const float*)dt_bias, step, decay);
    return launch_check(cudaGetLastError(), "ssd_prep");
}

int launch_ssd_post(int dt, int n, int H, int dv, int groups, const float* o, const float* x, int ldx, const float* z, int ldz, const void* Dskip,
                    const void* w, float eps, void* y, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    if (groups <= 0 || (H * dv) % groups) { set_error("ssd: %d channels not divisible into %d norm groups", H * dv, groups); return WF_ERR_INVALID; }
    const int gw = H * dv / groups;
    const int threads = gw >= 1024 ? 256 : (gw >= 256 ? 128 : 64);
    const dim3 grid(n, groups);
    if (dt == WF_BF16) ssd_post_kernel<<<grid, threads, 0, s>>>(H, dv, groups, o, x, ldx, z, ldz, (const __nv_bfloat16*)Dskip, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)y);
    else ssd_post_kernel<<<grid, threads, 0, s>>>(H, dv, groups, o, x, ldx, z, ldz, (const float*)Dskip, (const float*)w, eps, (float*)y);
    return launch_check(cudaGetLastError(), "ssd_post");
}

}  // namespace seq
}  // namespace wf
