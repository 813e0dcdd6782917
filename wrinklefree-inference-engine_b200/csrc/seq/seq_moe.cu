// Routed feed-forward: softmax or sigmoid router with an additive choice correction, group-limited top-k choice (groups ranked by their
// largest choice score or by the sum of their few largest), identity experts, an optional gated shared expert in the combine, and the
// bookkeeping that turns the chosen (token, expert) pairs into expert-contiguous, tile-padded row ranges for the grouped matrix products.
#include "seq_kernels.cuh"
#include <math.h>

namespace wf {
namespace seq {

namespace {

__device__ __forceinline__ void warp_argmax(float& v, int& idx) {   // largest value, lowest index among equals; all lanes get it
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
}

// The choice of one token by one warp.  zr: the token's logits (global or shared); sm: 2 N + groups floats of shared memory
// (s[N] scores, ch[N] choice scores, gs[G] group scores).
template <typename T>
__device__ void route_token(const RouterDims& R, const float* zr, const T* __restrict__ correction, int32_t* __restrict__ ids, float* __restrict__ wts,
                            int32_t* __restrict__ counts, float* sm, int i, int lane) {
    const int N = R.E + R.I, gsz = N / R.groups;
    float* sc = sm;
    float* ch = sc + N;
    float* gs = ch + N;
    if (R.act == 1) {
        for (int e = lane; e < N; e += 32) { sc[e] = sigmoid_f(zr[e]); ch[e] = sc[e] + to_f(correction[e]); }
    } else {
        float mx = -INFINITY;
        for (int e = lane; e < N; e += 32) mx = fmaxf(mx, zr[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < N; e += 32) { const float p = expf(zr[e] - mx); sc[e] = p; sum += p; }
        sum = warp_sum(sum);
        const float inv = 1.f / sum;
        for (int e = lane; e < N; e += 32) { sc[e] *= inv; ch[e] = sc[e] + to_f(correction[e]); }
    }
    __syncwarp();
    // group score = sum of the group's group_top largest choice scores (the largest alone when group_top <= 1); keep the best `keep` groups
    for (int g = lane; g < R.groups; g += 32) {
        float acc = 0.f;
        int prev_e = -1;
        float prev_v = INFINITY;
        const int take = R.group_top < 1 ? 1 : (R.group_top < gsz ? R.group_top : gsz);
        for (int r = 0; r < take; ++r) {       // r-th largest: the largest entry that comes after (prev_v, prev_e) in (value desc, index asc) order
            float m = -INFINITY; int me = -1;
            for (int e = g * gsz; e < (g + 1) * gsz; ++e) {
                const float x = ch[e];
                const bool after = x < prev_v || (x == prev_v && e > prev_e);
                if (after && (me < 0 || x > m)) { m = x; me = e; }
            }
            acc += m; prev_v = m; prev_e = me;
        }
        gs[g] = acc;
    }
    __syncwarp();
    if (R.keep < R.groups) {
        // the groups that are NOT among the best `keep` lose their experts: mark the winners with NaN-free sentinel +inf, then mask
        for (int r = 0; r < R.keep; ++r) {
            float v = -INFINITY; int gi = 0x7fffffff;
            for (int g = lane; g < R.groups; g += 32) { const float x = gs[g]; if (x != INFINITY && (x > v || (x == v && g < gi))) { v = x; gi = g; } }
            warp_argmax(v, gi);
            if (lane == 0 && gi != 0x7fffffff) gs[gi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < N; e += 32) if (gs[e / gsz] != INFINITY) ch[e] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < R.top; ++k) {
        float v = -INFINITY; int ei = 0x7fffffff;
        for (int e = lane; e < N; e += 32) { const float x = ch[e]; if (!isnan(x) && (x > v || (x == v && e < ei))) { v = x; ei = e; } }
        warp_argmax(v, ei);
        if (ei == 0x7fffffff) ei = 0;
        if (lane == 0) {
            ids[(size_t)i * R.top + k] = ei;
            wts[(size_t)i * R.top + k] = sc[ei];
            ch[ei] = NAN;                                   // taken
            if (counts && ei < R.E) atomicAdd(&counts[ei], 1);
        }
        __syncwarp();
    }
    if (R.norm || R.scale != 1.f) {
        float* w = wts + (size_t)i * R.top;
        float tot = 0.f;
        if (R.norm) for (int k = 0; k < R.top; ++k) tot += w[k];       // every lane, same order: identical sums
        const float mul = R.norm ? R.scale / (tot + 1e-20f) : R.scale;
        __syncwarp();
        for (int k = lane; k < R.top; k += 32) w[k] *= mul;
    }
}

// one warp per token
template <typename T>
__global__ void moe_route_kernel(RouterDims R, const float* __restrict__ z, int ldz, const T* __restrict__ correction, int32_t* __restrict__ ids,
                                 float* __restrict__ wts, int32_t* __restrict__ counts) {
    extern __shared__ float sm[];
    route_token(R, z + (size_t)blockIdx.x * ldz, correction, ids, wts, counts, sm, blockIdx.x, threadIdx.x);
}

// Router product and choice in one kernel, one block per `tb` tokens: the tokens' FLOAT rows are staged in shared memory, every warp forms
// the logits of a few outputs for all of them against the storage-type weight rows with float products (a weight row is loaded once per
// block; NZ rows: the router's outputs, then optional extra rows such as a shared expert's gate), the logits go to z (float [n, ldz])
// and warp t makes the choice of token t from the shared copy.
// RF_TB bounds tb.  Measured at 2048 tokens x 31 rows x 2560: 8 tokens per block 70 us, 1 token per block 75 us (the weight rows come from
// L2 either way; fewer, longer blocks fill the machine worse), while single decoded tokens pay for the unused accumulators: so 1.
constexpr int RF_THREADS = 256, RF_TB = 1;
template <typename T, bool VEC>
__global__ void __launch_bounds__(RF_THREADS) router_fused_kernel(RouterDims R, int n, int tb, const float* __restrict__ x, int ldx, const T* __restrict__ w, int NZ, int W,
                                                                  float* __restrict__ z, int ldz, const T* __restrict__ correction, int32_t* __restrict__ ids,
                                                                  float* __restrict__ wts, int32_t* __restrict__ counts) {
    extern __shared__ __align__(16) float sm[];
    const int Wp = (W + 3) / 4 * 4, N = R.E + R.I, per = 2 * N + R.groups;
    float* xs = sm;                                  // [tb][Wp]
    float* zl = xs + (size_t)tb * Wp;                // [tb][NZ]
    float* scratch = zl + (size_t)tb * NZ;           // [tb][per]: route_token's
    const int i0 = blockIdx.x * tb, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nt = n - i0 < tb ? n - i0 : tb;
    if (RF_TB == 1) { for (int c = threadIdx.x; c < W; c += RF_THREADS) xs[c] = x[(size_t)i0 * ldx + c]; }
    else for (int idx = threadIdx.x; idx < nt * W; idx += RF_THREADS) { const int t = idx / W, c = idx - t * W; xs[(size_t)t * Wp + c] = x[(size_t)(i0 + t) * ldx + c]; }
    __syncthreads();
    constexpr int VN = 16 / sizeof(T);               // elements per 16-byte load
    for (int e = warp; e < NZ; e += RF_THREADS / 32) {
        const T* wr = w + (size_t)e * W;
        float acc[RF_TB];
#pragma unroll
        for (int t = 0; t < RF_TB; ++t) acc[t] = 0.f;
        if (VEC) {
            for (int c = lane * VN; c < W; c += 32 * VN) {
                const uint4 q = *reinterpret_cast<const uint4*>(wr + c);
                const T* v = reinterpret_cast<const T*>(&q);
                float wv[VN];
#pragma unroll
                for (int k = 0; k < VN; ++k) wv[k] = to_f(v[k]);
#pragma unroll
                for (int t = 0; t < RF_TB; ++t) {
                    if (t < nt) {
#pragma unroll
                        for (int k = 0; k < VN; k += 4) {      // 16-byte reads of the staged rows too
                            const float4 a = *reinterpret_cast<const float4*>(xs + (size_t)t * Wp + c + k);
                            acc[t] = fmaf(a.x, wv[k], acc[t]); acc[t] = fmaf(a.y, wv[k + 1], acc[t]); acc[t] = fmaf(a.z, wv[k + 2], acc[t]); acc[t] = fmaf(a.w, wv[k + 3], acc[t]);
                        }
                    }
                }
            }
        } else {
            for (int c = lane; c < W; c += 32) {
                const float wv = to_f(wr[c]);
#pragma unroll
                for (int t = 0; t < RF_TB; ++t) if (t < nt) acc[t] = fmaf(xs[(size_t)t * Wp + c], wv, acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < RF_TB; ++t) {
            if (t < nt) {
                const float v = warp_sum(acc[t]);
                if (lane == 0) { zl[(size_t)t * NZ + e] = v; z[(size_t)(i0 + t) * ldz + e] = v; }
            }
        }
    }
    __syncthreads();
    if (warp < nt) route_token(R, zl + (size_t)warp * NZ, correction, ids, wts, counts, scratch + (size_t)warp * per, i0 + warp, lane);
}

// single block.  scratch: off[E + 1], cursor[E]
__global__ void moe_plan_kernel(RouterDims R, int n, const int32_t* __restrict__ ids, const int32_t* __restrict__ counts, int32_t* __restrict__ scratch,
                                int32_t* __restrict__ sorted_rows, int32_t* __restrict__ pair_row, int32_t* __restrict__ tile_group, int P) {
    int32_t* off = scratch;
    int32_t* cursor = scratch + R.E + 1;
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < R.E; ++e) { off[e] = acc; acc += (counts[e] + GEMM_BM - 1) / GEMM_BM * GEMM_BM; cursor[e] = 0; }
        off[R.E] = acc;
    }
    for (int r = threadIdx.x; r < P; r += blockDim.x) sorted_rows[r] = -1;
    for (int t = threadIdx.x; t < P / GEMM_BM; t += blockDim.x) tile_group[t] = -1;
    __syncthreads();
    for (int e = 0; e < R.E; ++e)
        for (int t = off[e] / GEMM_BM + threadIdx.x; t < off[e + 1] / GEMM_BM; t += blockDim.x) tile_group[t] = e;
    for (int pi = threadIdx.x; pi < n * R.top; pi += blockDim.x) {
        const int e = ids[pi];
        if (e >= R.E) { pair_row[pi] = -1; continue; }
        const int pos = off[e] + atomicAdd(&cursor[e], 1);
        sorted_rows[pos] = pi / R.top;
        pair_row[pi] = pos;
    }
}

// VEC = 4: ff a multiple of 4 (16-byte loads of the gate and up halves)
template <typename T, int VEC>
__global__ void silu_mul_kernel(const float* __restrict__ gu, int ff, const int32_t* __restrict__ tile_group, T* __restrict__ hmid, int act, float limit) {
    const int r = blockIdx.x;
    if (tile_group && tile_group[r / GEMM_BM] < 0) return;
    const float* row = gu + (size_t)r * (act == 3 ? 1 : 2) * ff;
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC; c < ff; c += gridDim.y * blockDim.x * VEC) {
        float g[VEC], u[VEC];
        if (act == 3) {                   // no gate half: relu(u)^2
#pragma unroll
            for (int v = 0; v < VEC; ++v) { const float z = fmaxf(row[c + v], 0.f); hmid[(size_t)r * ff + c + v] = from_f<T>(z * z); }
            continue;
        }
        if (VEC == 4) {
            const float4 a = *reinterpret_cast<const float4*>(row + c), b = *reinterpret_cast<const float4*>(row + ff + c);
            g[0] = a.x; g[1 % VEC] = a.y; g[2 % VEC] = a.z; g[3 % VEC] = a.w;
            u[0] = b.x; u[1 % VEC] = b.y; u[2 % VEC] = b.z; u[3 % VEC] = b.w;
        } else { g[0] = row[c]; u[0] = row[ff + c]; }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            float a;
            if (act == 1) {
                const float gg = fminf(g[v], limit), uu = fminf(fmaxf(u[v], -limit), limit);
                a = gg * sigmoid_f(1.702f * gg) * (uu + 1.f);
            } else if (act == 2) {
                const float z = g[v];
                a = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))) * u[v];
            } else a = silu_f(g[v]) * u[v];
            hmid[(size_t)r * ff + c + v] = from_f<T>(a);
        }
    }
}

// VEC = 4: W a multiple of 4
template <typename T, int VEC>
__global__ void moe_combine_kernel(RouterDims R, int W, const int32_t* __restrict__ ids, const float* __restrict__ wts, const int32_t* __restrict__ pair_row,
                                   const float* __restrict__ y, const T* __restrict__ h, float* __restrict__ out, const float* __restrict__ shared_y,
                                   const float* __restrict__ shared_gate, int ld_gate) {
    const int i = blockIdx.x;
    const float sg = shared_y ? (shared_gate ? sigmoid_f(shared_gate[(size_t)i * ld_gate]) : 1.f) : 0.f;
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC; c < W; c += gridDim.y * blockDim.x * VEC) {
        float acc[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
        for (int k = 0; k < R.top; ++k) {
            const size_t pi = (size_t)i * R.top + k;
            const int e = ids[pi];
            const float w = wts[pi];
            float val[VEC];
            if (e < R.E) {
                const float* yr = y + (size_t)(pair_row ? pair_row[pi] : (int)pi) * W + c;
                if (VEC == 4) { const float4 q = *reinterpret_cast<const float4*>(yr); val[0] = q.x; val[1 % VEC] = q.y; val[2 % VEC] = q.z; val[3 % VEC] = q.w; }
                else val[0] = yr[0];
            } else {
#pragma unroll
                for (int v = 0; v < VEC; ++v) val[v] = to_f(h[(size_t)i * W + c + v]);
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] = fmaf(w, val[v], acc[v]);
        }
        if (shared_y) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) acc[v] = fmaf(sg, shared_y[(size_t)i * W + c + v], acc[v]);
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) out[(size_t)i * W + c + v] = acc[v];
    }
}

}  // namespace

int launch_moe_route(int dt, const RouterDims& R, int n, const float* z, int ldz, const void* correction, int32_t* ids, float* wts,
                     int32_t* counts, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    const int N = R.E + R.I;
    if (R.groups < 1 || N % R.groups || R.keep < 1 || R.keep > R.groups || R.top < 1 || R.top > N) {
        set_error("router: %d outputs, %d groups (keep %d), top %d", N, R.groups, R.keep, R.top);
        return WF_ERR_INVALID;
    }
    const size_t smem = (size_t)(2 * N + R.groups) * sizeof(float);
    if (smem > 48 * 1024) { set_error("router: %d outputs do not fit in shared memory", N); return WF_ERR_UNSUPPORTED; }
    if (dt == WF_BF16) moe_route_kernel<<<n, 32, smem, s>>>(R, z, ldz, (const __nv_bfloat16*)correction, ids, wts, counts);
    else moe_route_kernel<<<n, 32, smem, s>>>(R, z, ldz, (const float*)correction, ids, wts, counts);
    return launch_check(cudaGetLastError(), "moe_route");
}

namespace {
size_t router_fused_smem(const RouterDims& R, int NZ, int W, int tb) { return (size_t)tb * ((size_t)(W + 3) / 4 * 4 + NZ + 2 * (R.E + R.I) + R.groups) * sizeof(float); }
}
bool router_fused_usable(const RouterDims& R, int NZ, int W) { return router_fused_smem(R, NZ, W, 1) <= 48 * 1024; }

int launch_router_fused(int dt, const RouterDims& R, int n, const float* x, int ldx, const void* w, int NZ, int W, float* z, int ldz, const void* correction,
                        int32_t* ids, float* wts, int32_t* counts, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    const int N = R.E + R.I;
    if (R.groups < 1 || N % R.groups || R.keep < 1 || R.keep > R.groups || R.top < 1 || R.top > N || NZ < N) {
        set_error("router: %d outputs (%d rows), %d groups (keep %d), top %d", N, NZ, R.groups, R.keep, R.top);
        return WF_ERR_INVALID;
    }
    if (!router_fused_usable(R, NZ, W)) { set_error("router: width %d with %d outputs does not fit in shared memory", W, N); return WF_ERR_UNSUPPORTED; }
    // tokens per block: as many as fit in 48 KB of shared memory (a weight row is then loaded once for all of them), but no more than
    // leaves a block for every SM
    int tb = RF_TB;
    while (tb > 1 && (router_fused_smem(R, NZ, W, tb) > 48 * 1024 || (n + tb - 1) / tb < sm_count())) tb >>= 1;
    const size_t smem = router_fused_smem(R, NZ, W, tb);
    const size_t esz = dt == WF_BF16 ? 2 : 4;
    const bool vec = (W * esz) % 16 == 0 && (((uintptr_t)w) & 15) == 0;
    const int blocks = (n + tb - 1) / tb;
    if (dt == WF_BF16) {
        if (vec) router_fused_kernel<__nv_bfloat16, true><<<blocks, RF_THREADS, smem, s>>>(R, n, tb, x, ldx, (const __nv_bfloat16*)w, NZ, W, z, ldz, (const __nv_bfloat16*)correction, ids, wts, counts);
        else router_fused_kernel<__nv_bfloat16, false><<<blocks, RF_THREADS, smem, s>>>(R, n, tb, x, ldx, (const __nv_bfloat16*)w, NZ, W, z, ldz, (const __nv_bfloat16*)correction, ids, wts, counts);
    } else {
        if (vec) router_fused_kernel<float, true><<<blocks, RF_THREADS, smem, s>>>(R, n, tb, x, ldx, (const float*)w, NZ, W, z, ldz, (const float*)correction, ids, wts, counts);
        else router_fused_kernel<float, false><<<blocks, RF_THREADS, smem, s>>>(R, n, tb, x, ldx, (const float*)w, NZ, W, z, ldz, (const float*)correction, ids, wts, counts);
    }
    return launch_check(cudaGetLastError(), "router_fused");
}

int launch_moe_plan(const RouterDims& R, int n, const int32_t* ids, const int32_t* counts, int32_t* scratch, int32_t* sorted_rows,
                    int32_t* pair_row, int32_t* tile_group, int P, cudaStream_t s) {
    if (n <= 0) return WF_OK;
    if (P % GEMM_BM) { set_error("moe_plan: row bound %d is not a multiple of the row tile", P); return WF_ERR_INVALID; }
    moe_plan_kernel<<<1, 512, 0, s>>>(R, n, ids, counts, scratch, sorted_rows, pair_row, tile_group, P);
    return launch_check(cudaGetLastError(), "moe_plan");
}

int launch_silu_mul(int dt, const float* gu, int P, int ff, const int32_t* tile_group, void* hmid, cudaStream_t s, int act, float limit) {
    if (P <= 0) return WF_OK;
    const bool vec = ff % 4 == 0 && (((uintptr_t)gu) & 15) == 0;
    const int per = 128 * (vec ? 4 : 1);
    const dim3 grid(P, P < 256 ? (ff + per - 1) / per : 1);
    if (dt == WF_BF16) { if (vec) silu_mul_kernel<__nv_bfloat16, 4><<<grid, 128, 0, s>>>(gu, ff, tile_group, (__nv_bfloat16*)hmid, act, limit); else silu_mul_kernel<__nv_bfloat16, 1><<<grid, 128, 0, s>>>(gu, ff, tile_group, (__nv_bfloat16*)hmid, act, limit); }
    else { if (vec) silu_mul_kernel<float, 4><<<grid, 128, 0, s>>>(gu, ff, tile_group, (float*)hmid, act, limit); else silu_mul_kernel<float, 1><<<grid, 128, 0, s>>>(gu, ff, tile_group, (float*)hmid, act, limit); }
    return launch_check(cudaGetLastError(), "silu_mul");
}

int launch_moe_combine(int dt, const RouterDims& R, int n, int W, const int32_t* ids, const float* wts, const int32_t* pair_row, const float* y,
                       const void* h, float* out, cudaStream_t s, const float* shared_y, const float* shared_gate, int ld_gate) {
    if (n <= 0) return WF_OK;
    const bool vec = W % 4 == 0 && (((uintptr_t)y) & 15) == 0 && (((uintptr_t)out) & 15) == 0;
    const int per = 256 * (vec ? 4 : 1);
    const dim3 grid(n, n < 64 ? (W + per - 1) / per : 1);       // few tokens: spread a row over several blocks
    if (dt == WF_BF16) { if (vec) moe_combine_kernel<__nv_bfloat16, 4><<<grid, 256, 0, s>>>(R, W, ids, wts, pair_row, y, (const __nv_bfloat16*)h, out, shared_y, shared_gate, ld_gate); else moe_combine_kernel<__nv_bfloat16, 1><<<grid, 256, 0, s>>>(R, W, ids, wts, pair_row, y, (const __nv_bfloat16*)h, out, shared_y, shared_gate, ld_gate); }
    else { if (vec) moe_combine_kernel<float, 4><<<grid, 256, 0, s>>>(R, W, ids, wts, pair_row, y, (const float*)h, out, shared_y, shared_gate, ld_gate); else moe_combine_kernel<float, 1><<<grid, 256, 0, s>>>(R, W, ids, wts, pair_row, y, (const float*)h, out, shared_y, shared_gate, ld_gate); }
    return launch_check(cudaGetLastError(), "moe_combine");
}

// ---- sampling --------------------------------------------------------------------------------------------------------------
namespace {

constexpr int SM_THREADS = 256;

__device__ float block_reduce_sum(float v, float* scratch) { return block_sum(v, scratch); }

// One block per row.  Greedy: argmax, lowest index among equals.  Otherwise p = softmax(logits / temperature); the kept set is
// {p >= tau} with tau found by bisection so that it holds at most top_k entries and is the smallest such set whose mass reaches top_p;
// the draw walks the kept entries in index order.
__global__ void __launch_bounds__(SM_THREADS) sample_kernel(const float* __restrict__ logits, int V, float temperature, int top_k, float top_p,
                                                             const float* __restrict__ u, int32_t* __restrict__ next) {
    __shared__ float scratch[33];
    __shared__ float sv[SM_THREADS / 32];
    __shared__ int si[SM_THREADS / 32];
    __shared__ float part[SM_THREADS];
    const float* row = logits + (size_t)blockIdx.x * V;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int c = tid; c < V; c += SM_THREADS) { const float x = row[c]; if (x > bv) { bv = x; bi = c; } }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    bv = sv[0]; bi = si[0];
    for (int w = 1; w < SM_THREADS / 32; ++w) if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    if (temperature <= 0.f) { if (tid == 0) next[blockIdx.x] = bi; return; }
    const float it = 1.f / temperature;
    float z = 0.f;
    for (int c = tid; c < V; c += SM_THREADS) z += expf((row[c] - bv) * it);
    z = block_reduce_sum(z, scratch);
    // thresholds on the unnormalised weight w_c = exp((x_c - max) / T) in (0, 1], each found by bisection:
    // tau_k = the smallest threshold that keeps at most top_k entries, tau_p = the largest one whose kept mass still reaches top_p
    const bool k_active = top_k > 0 && top_k < V, p_active = top_p > 0.f && top_p < 1.f;
    float tau = 0.f;
    if (k_active) {
        float lo = 0.f, hi = 1.f;                    // {w >= hi} always fits (the maximum alone, w = 1)
        for (int r = 0; r < 30; ++r) {
            const float mid = 0.5f * (lo + hi);
            float cnt = 0.f;
            for (int c = tid; c < V; c += SM_THREADS) cnt += expf((row[c] - bv) * it) >= mid ? 1.f : 0.f;
            cnt = block_reduce_sum(cnt, scratch);
            if (cnt <= (float)top_k) hi = mid; else lo = mid;
        }
        tau = hi;
    }
    if (p_active) {
        float lo = 0.f, hi = 1.f;                    // {w >= lo} always reaches the mass (everything)
        for (int r = 0; r < 30; ++r) {
            const float mid = 0.5f * (lo + hi);
            float mass = 0.f;
            for (int c = tid; c < V; c += SM_THREADS) { const float w = expf((row[c] - bv) * it); if (w >= mid) mass += w; }
            mass = block_reduce_sum(mass, scratch);
            if (mass >= top_p * z) lo = mid; else hi = mid;
        }
        tau = fmaxf(tau, lo);
    }
    // kept mass per thread over a contiguous chunk, then the draw
    const int chunk = (V + SM_THREADS - 1) / SM_THREADS;
    const int c0 = tid * chunk, c1 = c0 + chunk < V ? c0 + chunk : V;
    float mine = 0.f;
    for (int c = c0; c < c1; ++c) { const float w = expf((row[c] - bv) * it); if (w >= tau) mine += w; }
    part[tid] = mine;
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int t = 0; t < SM_THREADS; ++t) total += part[t];
        float target = u[blockIdx.x] * total, run = 0.f;
        int pick = bi, t = 0;
        for (; t < SM_THREADS; ++t) { if (run + part[t] > target) break; run += part[t]; }
        if (t < SM_THREADS) {
            const int a0 = t * chunk, a1 = a0 + chunk < V ? a0 + chunk : V;
            for (int c = a0; c < a1; ++c) {
                const float w = expf((row[c] - bv) * it);
                if (w >= tau) { run += w; if (run > target) { pick = c; break; } }
            }
        }
        next[blockIdx.x] = pick;
    }
}

}  // namespace

int launch_sample(const float* logits, int m, int V, float temperature, int top_k, float top_p, const float* u, int32_t* next, cudaStream_t s) {
    if (m <= 0) return WF_OK;
    if (temperature > 0.f && !u) { set_error("sample: uniforms required when temperature > 0"); return WF_ERR_INVALID; }
    sample_kernel<<<m, SM_THREADS, 0, s>>>(logits, V, temperature, top_k, top_p, u, next);
    return launch_check(cudaGetLastError(), "sample");
}

}  // namespace seq
}  // namespace wf
