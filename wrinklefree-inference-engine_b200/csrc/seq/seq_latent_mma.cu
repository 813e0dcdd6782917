// Latent attention on tensor cores (bf16 mma.sync, fp32 softmax): one CTA per (query token, key split) with ALL heads as the rows of
// m16 tiles, because every head reads the same cached rows [latent c_j | rotated key part kr_j]:
//   S[h, j] = (qa_h . c_j + qr_h . kr_j) * scale          Q = [qa | qr] rounded to bf16, K tile = 32 cached rows staged once for all heads
//   O[h, :] = sum_j softmax_j(S[h, :]) c_j                 the same staged rows, read transposed, as the value operand
// Four warps serve 16 heads: each computes the scores of 8 of the tile's 32 keys, the row maxima meet in shared memory, the
// probabilities go to shared memory as bf16, and each warp accumulates a quarter of the latent dimensions.  Long windows with few
// query tokens are split along the keys over several CTAs whose partial (max, sum, O) are merged by a second kernel.
#include "seq_kernels.cuh"
#include <math.h>

namespace wf {
namespace seq {

namespace {

constexpr int KT = 32;                    // keys per tile

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct MmaParams {
    int splits;          // key splits per token (grid.y)
    float* part;         // splits > 1: [n][splits][H][R + 2] partial (O unnormalised, max, sum)
    int dkp;             // R + r rounded up to 16
    int stride;          // shared-memory row stride of Q / K rows in elements (dkp + 8: conflict-free ldmatrix)
};

// NT = R / 32: n-tiles (8 latent dimensions each) per warp in the value product
template <int NT>
__global__ void latent_attn_mma_kernel(Batch b, LatentDims L, const float* __restrict__ qa, const float* __restrict__ qr, PagedCache pc,
                                       __nv_bfloat16* __restrict__ out, MmaParams mp) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int HT = (L.H + 15) / 16, rows = HT * 16;
    const int stride = mp.stride, width = L.R + L.r;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);                 // [rows][stride]
    __nv_bfloat16* Ks = Qs + (size_t)rows * stride;                              // [2][KT][stride]
    __nv_bfloat16* Ps = Ks + (size_t)2 * KT * stride;                            // [rows][KT + 8]
    float* smax = reinterpret_cast<float*>(Ps + (size_t)rows * (KT + 8));        // [HT][4][16]
    float* ssum = smax + HT * 64;                                                // [HT][4][16]
    const int i = blockIdx.x, split = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ht = warp >> 2, w4 = warp & 3;                                     // head tile, warp inside it
    const int sq = b.tok_seq[i], pos = b.tok_pos[i];
    const int lo_all = pos - L.window + 1 > 0 ? pos - L.window + 1 : 0;
    const int cnt = pos + 1 - lo_all;
    int chunk = (cnt + mp.splits - 1) / mp.splits;
    chunk = (chunk + KT - 1) / KT * KT;
    const int lo = lo_all + split * chunk;
    const int hi = lo + chunk < pos + 1 ? lo + chunk : pos + 1;                  // keys [lo, hi)
    const int32_t* bt = pc.block_table + (size_t)b.seq_slot[sq] * pc.max_blocks;

    // ---- Q = [qa | qr] of every head as bf16 (rows beyond H and columns beyond R + r are zero): a warp per head, lanes over columns
    const int nwarps = blockDim.x >> 5;
    for (int h = warp; h < rows; h += nwarps) {
        __nv_bfloat16* qd = Qs + (size_t)h * stride;
        const float* a_src = qa + ((size_t)i * L.H + h) * L.R;
        const float* r_src = qr + ((size_t)i * L.H + h) * L.r;
        for (int c = lane; c < mp.dkp; c += 32) {
            float v = 0.f;
            if (h < L.H) {
                if (c < L.R) v = a_src[c];
                else if (c < width) v = r_src[c - L.R];
            }
            qd[c] = __float2bfloat16_rn(v);
        }
    }
    // ---- staging of one key tile: 16-byte chunks of the cached rows; rows past `hi` and the padding columns are zero.
    // A thread always serves the same row of the tile (one page lookup per tile) and every tpr-th chunk of it.
    const int chunks_per_row = mp.dkp / 8;
    const int tpr = blockDim.x / KT;                                              // threads per key row (4 warps per 16 heads: >= 4)
    const int st_row = tid / tpr, st_sub = tid - st_row * tpr;
    auto stage = [&](int buf, int j0) {
        __nv_bfloat16* d = Ks + ((size_t)buf * KT + st_row) * stride;
        const int j = j0 + st_row;
        if (j < hi) {
            const int page = bt[j / pc.page_size];
            const __nv_bfloat16* src = (const __nv_bfloat16*)pc.pool + (size_t)page * pc.page_stride + pc.layer_off + (size_t)(j % pc.page_size) * width;
            for (int c = st_sub; c < chunks_per_row; c += tpr) {
                if (c * 8 + 8 <= width) cp_async16(d + c * 8, src + c * 8);
                else *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
        } else {
            for (int c = st_sub; c < chunks_per_row; c += tpr) *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
        cp_async_commit();
    };
    float o[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) { o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};              // rows lane / 4 and lane / 4 + 8 of this head tile
    const int r0 = lane >> 2, cq = (lane & 3) * 2;
    const int ntiles = hi > lo ? (hi - lo + KT - 1) / KT : 0;
    if (ntiles > 0) stage(0, lo);
    for (int t = 0; t < ntiles; ++t) {
        const int buf = t & 1;
        cp_async_wait<0>();
        __syncthreads();                                                          // tile t (and, first time, Q) visible; every warp is done with tile t - 1
        if (t + 1 < ntiles) stage(buf ^ 1, lo + (t + 1) * KT);                    // overwrites the buffer tile t - 1 was read from
        const __nv_bfloat16* Kt = Ks + (size_t)buf * KT * stride;
        // ---- scores of this warp's 8 keys for the 16 heads of its tile
        // (four independent accumulation chains over the feature dimension, summed at the end: one chain would be latency-bound)
        float s[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f}, s3[4] = {0.f, 0.f, 0.f, 0.f};
        const __nv_bfloat16* qrow = Qs + (size_t)(ht * 16 + (lane & 15)) * stride + (lane >> 4) * 8;
        const __nv_bfloat16* krow = Kt + (size_t)(w4 * 8 + (lane & 7)) * stride + ((lane >> 3) & 1) * 8;
        int k0 = 0;
        for (; k0 + 64 <= mp.dkp; k0 += 64) {
            uint32_t a0[4], a1[4], a2[4], a3[4], b0[2], b1[2], b2[2], b3[2];
            ldsm_x4(a0, qrow + k0); ldsm_x2(b0, krow + k0);
            ldsm_x4(a1, qrow + k0 + 16); ldsm_x2(b1, krow + k0 + 16);
            ldsm_x4(a2, qrow + k0 + 32); ldsm_x2(b2, krow + k0 + 32);
            ldsm_x4(a3, qrow + k0 + 48); ldsm_x2(b3, krow + k0 + 48);
            mma16816(s, a0, b0[0], b0[1]);
            mma16816(s1, a1, b1[0], b1[1]);
            mma16816(s2, a2, b2[0], b2[1]);
            mma16816(s3, a3, b3[0], b3[1]);
        }
        for (; k0 < mp.dkp; k0 += 16) {
            uint32_t a[4], bb[2];
            ldsm_x4(a, qrow + k0);
            ldsm_x2(bb, krow + k0);
            mma16816(s, a, bb[0], bb[1]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) s[e] += s1[e] + s2[e] + s3[e];
        const int jbase = lo + t * KT + w4 * 8 + cq;
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = jbase + (e & 1);
            s[e] = j < hi ? s[e] * L.scale : -INFINITY;
            tmax[e >> 1] = fmaxf(tmax[e >> 1], s[e]);
        }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            tmax[h2] = fmaxf(tmax[h2], __shfl_xor_sync(0xffffffffu, tmax[h2], 1));
            tmax[h2] = fmaxf(tmax[h2], __shfl_xor_sync(0xffffffffu, tmax[h2], 2));
        }
        if ((lane & 3) == 0) { smax[(ht * 4 + w4) * 16 + r0] = tmax[0]; smax[(ht * 4 + w4) * 16 + r0 + 8] = tmax[1]; }
        __syncthreads();
        float corr[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const int r = r0 + h2 * 8;
            float mx = smax[(ht * 4 + 0) * 16 + r];
            mx = fmaxf(mx, smax[(ht * 4 + 1) * 16 + r]);
            mx = fmaxf(mx, smax[(ht * 4 + 2) * 16 + r]);
            mx = fmaxf(mx, smax[(ht * 4 + 3) * 16 + r]);
            const float mn = fmaxf(m_run[h2], mx);                                // finite: key lo + t * KT exists in every tile
            corr[h2] = expf(m_run[h2] - mn);
            m_run[h2] = mn;
            const float p0 = expf(s[h2 * 2] - mn), p1 = expf(s[h2 * 2 + 1] - mn);
            l_run[h2] = l_run[h2] * corr[h2] + p0 + p1;
            __nv_bfloat162 pv = __floats2bfloat162_rn(p0, p1);
            *reinterpret_cast<__nv_bfloat162*>(Ps + (size_t)(ht * 16 + r) * (KT + 8) + w4 * 8 + cq) = pv;
        }
        __syncthreads();
        // ---- O[16 heads, this warp's quarter of the latent] = O * corr + P[16, 32] . C[32, quarter]
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { o[nt][0] *= corr[0]; o[nt][1] *= corr[0]; o[nt][2] *= corr[1]; o[nt][3] *= corr[1]; }
        const __nv_bfloat16* prow = Ps + (size_t)(ht * 16 + (lane & 15)) * (KT + 8) + (lane >> 4) * 8;
        const int ncol0 = w4 * NT * 8;
#pragma unroll
        for (int k0 = 0; k0 < KT; k0 += 16) {
            uint32_t a[4];
            ldsm_x4(a, prow + k0);
            const __nv_bfloat16* crow = Kt + (size_t)(k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * stride + ncol0 + (lane >> 4) * 8;
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                uint32_t bb[4];
                ldsm_x4_trans(bb, crow + nt * 8);
                mma16816(o[nt], a, bb[0], bb[1]);
                if (nt + 1 < NT) mma16816(o[nt + 1], a, bb[2], bb[3]);
            }
        }
    }
    // ---- row sums of the four warps meet; normalise (or hand the partial result to the merge)
    __syncthreads();
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
    }
    if ((lane & 3) == 0) { ssum[(ht * 4 + w4) * 16 + r0] = l_run[0]; ssum[(ht * 4 + w4) * 16 + r0 + 8] = l_run[1]; }
    __syncthreads();
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int r = r0 + h2 * 8, h = ht * 16 + r;
        if (h >= L.H) continue;
        const float lsum = ssum[(ht * 4 + 0) * 16 + r] + ssum[(ht * 4 + 1) * 16 + r] + ssum[(ht * 4 + 2) * 16 + r] + ssum[(ht * 4 + 3) * 16 + r];
        if (mp.splits == 1) {
            const float inv = 1.f / (L.sink ? lsum + expf(L.sink[h] - m_run[h2]) : lsum);      // the sink: a weight without a value
            __nv_bfloat16* dst = out + ((size_t)i * L.H + h) * L.R + w4 * NT * 8 + cq;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) = __floats2bfloat162_rn(o[nt][h2 * 2] * inv, o[nt][h2 * 2 + 1] * inv);
        } else {
            float* dst = mp.part + (((size_t)i * mp.splits + split) * L.H + h) * (L.R + 2);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) { dst[w4 * NT * 8 + cq + nt * 8] = o[nt][h2 * 2]; dst[w4 * NT * 8 + cq + nt * 8 + 1] = o[nt][h2 * 2 + 1]; }
            if (w4 == 0 && (lane & 3) == 0) { dst[L.R] = m_run[h2]; dst[L.R + 1] = lsum; }
        }
    }
}

// one block per (token, head): out = sum_s exp(m_s - m) O_s / sum_s exp(m_s - m) l_s
__global__ void latent_attn_merge_kernel(int H, int R, int splits, const float* __restrict__ part, __nv_bfloat16* __restrict__ out, const float* __restrict__ sink) {
    const int i = blockIdx.x, h = blockIdx.y;
    const float* p0 = part + (((size_t)i * splits) * H + h) * (R + 2);
    const size_t sstride = (size_t)H * (R + 2);
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, p0[s * sstride + R]);
    float l = 0.f;
    for (int s = 0; s < splits; ++s) { const float ms = p0[s * sstride + R]; if (ms != -INFINITY) l += expf(ms - m) * p0[s * sstride + R + 1]; }
    if (sink) l += expf(sink[h] - m);
    const float inv = 1.f / l;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; ++s) { const float ms = p0[s * sstride + R]; if (ms != -INFINITY) v += expf(ms - m) * p0[s * sstride + c]; }
        out[((size_t)i * H + h) * R + c] = __float2bfloat16_rn(v * inv);
    }
}


// ---- second form: keys as the M rows ---------------------------------------------------------------------------------------------
// S^T[key, head] = K[key, :] . Q[head, :]^T and O^T[dim, head] = C^T[dim, key] . P[key, head]: a cached row's fragment is loaded once
// for ALL heads (heads are 8-wide N tiles: H = 20 pads to 24, not 32), and the queries are the small operand.  8 warps per CTA:
//   scores: warp (m-tile of 16 keys, quarter of the feature dimension) -> partial S^T in shared memory (fp32);
//   softmax: warp w owns heads w, w + 8, ..., lanes = the tile's 32 keys; probabilities to shared memory as bf16, rescale factors beside;
//   values: warp w owns latent m-tiles w, w + 8, ... for all heads.
// 32-bit shared-memory addresses for the fragment loads (no generic-pointer arithmetic inside the tile loop)
__device__ __forceinline__ void ldsm_x4_a(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_a(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans_a(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_trans_a(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__host__ __device__ constexpr int kt_pt_stride(int NH) { return (NH & 1) ? NH * 8 + 16 : NH * 8 + 8; }   // 16-byte units per row odd: conflict-free ldmatrix

template <int NH, int MTW>
__global__ void __launch_bounds__(256) latent_attn_kt_kernel(Batch b, LatentDims L, const float* __restrict__ qa, const float* __restrict__ qr, PagedCache pc,
                                                             __nv_bfloat16* __restrict__ out, MmaParams mp) {
    extern __shared__ __align__(16) unsigned char smraw[];
    constexpr int HP = NH * 8, PS = HP + 1, PT = kt_pt_stride(NH);
    const int stride = mp.stride, width = L.R + L.r;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);                 // [HP][stride]
    __nv_bfloat16* Ks = Qs + (size_t)HP * stride;                                // [2][KT][stride]
    __nv_bfloat16* Pt = Ks + (size_t)2 * KT * stride;                            // [KT][PT] probabilities, bf16
    float* part = reinterpret_cast<float*>(Pt + KT * PT);                        // [4][KT][PS] partial scores of the four feature quarters
    float* corr_s = part + 4 * KT * PS;                                          // [HP] rescale factor of the running sums for this tile
    float* ml_s = corr_s + HP;                                                   // [2][HP] final max and sum
    const int i = blockIdx.x, split = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sq = b.tok_seq[i], pos = b.tok_pos[i];
    const int lo_all = pos - L.window + 1 > 0 ? pos - L.window + 1 : 0;
    const int cnt = pos + 1 - lo_all;
    int chunk = (cnt + mp.splits - 1) / mp.splits;
    chunk = (chunk + KT - 1) / KT * KT;
    const int lo = lo_all + split * chunk;
    const int hi = lo + chunk < pos + 1 ? lo + chunk : pos + 1;
    const int32_t* bt = pc.block_table + (size_t)b.seq_slot[sq] * pc.max_blocks;

    for (int h = warp; h < HP; h += 8) {
        __nv_bfloat16* qd = Qs + (size_t)h * stride;
        const float* a_src = qa + ((size_t)i * L.H + h) * L.R;
        const float* r_src = qr + ((size_t)i * L.H + h) * L.r;
        for (int c = lane; c < mp.dkp; c += 32) {
            float v = 0.f;
            if (h < L.H) {
                if (c < L.R) v = a_src[c];
                else if (c < width) v = r_src[c - L.R];
            }
            qd[c] = __float2bfloat16_rn(v);
        }
    }
    // staging: 8 threads per key row, 16-byte chunks.  The padding columns (width .. dkp) of both buffers are zeroed once; rows past
    // `hi` (last tile only) are zeroed when they occur.
    const int full_chunks = width / 8, chunks_per_row = mp.dkp / 8;
    const int st_row = tid >> 3, st_sub = tid & 7;
    for (int bf = 0; bf < 2; ++bf)
        for (int c = full_chunks + st_sub; c < chunks_per_row; c += 8)
            *reinterpret_cast<uint4*>(Ks + ((size_t)bf * KT + st_row) * stride + c * 8) = make_uint4(0u, 0u, 0u, 0u);
    const uint32_t ks_base = smem_u32(Ks);
    const uint32_t st_dst0 = ks_base + (uint32_t)(st_row * stride + st_sub * 8) * 2u;
    auto stage = [&](int buf, int j0) {
        const uint32_t d = st_dst0 + (uint32_t)buf * (uint32_t)(KT * stride * 2);
        const int j = j0 + st_row;
        if (j < hi) {
            const int page = bt[j / pc.page_size];
            const __nv_bfloat16* src = (const __nv_bfloat16*)pc.pool + (size_t)page * pc.page_stride + pc.layer_off + (size_t)(j % pc.page_size) * width + st_sub * 8;
            for (int c = st_sub; c < full_chunks; c += 8, src += 64)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d + (uint32_t)(c - st_sub) * 16u), "l"(src) : "memory");
        } else {
            for (int c = st_sub; c < full_chunks; c += 8)
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(d + (uint32_t)(c - st_sub) * 16u), "r"(0u) : "memory");
        }
        cp_async_commit();
    };
    float o[MTW][NH][4];
#pragma unroll
    for (int a = 0; a < MTW; ++a)
#pragma unroll
        for (int n = 0; n < NH; ++n) { o[a][n][0] = o[a][n][1] = o[a][n][2] = o[a][n][3] = 0.f; }
    float m_run[NH], l_run[NH];                                                  // softmax state of the heads this warp owns (uniform over its lanes)
#pragma unroll
    for (int k = 0; k < NH; ++k) { m_run[k] = -INFINITY; l_run[k] = 0.f; }
    const int mt = warp & 1, ks = warp >> 1;                                     // score phase: key m-tile, feature quarter
    const int ksteps = mp.dkp / 16;
    const int k_per = (ksteps + 3) / 4;
    const int k_lo = ks * k_per, k_hi = k_lo + k_per < ksteps ? k_lo + k_per : ksteps;
    const int r0 = lane >> 2, cq = (lane & 3) * 2;
    const int m_tiles = L.R / 16;
    const uint32_t tile_bytes = (uint32_t)(KT * stride * 2);
    // per-lane fragment addresses (bytes, shared window)
    const uint32_t k_frag = ks_base + (uint32_t)((mt * 16 + (lane & 15)) * stride + (lane >> 4) * 8 + k_lo * 16) * 2u;
    const uint32_t q_frag = smem_u32(Qs) + (uint32_t)((lane & 7) * stride + ((lane >> 3) & 1) * 8 + k_lo * 16) * 2u;
    const uint32_t c_frag = ks_base + (uint32_t)(((lane & 7) + (lane >> 4) * 8) * stride + ((lane >> 3) & 1) * 8) * 2u;
    const uint32_t p_frag = smem_u32(Pt) + (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * PT) * 2u;
    float* part_w = part + (size_t)ks * KT * PS + (mt * 16 + r0) * PS + cq;
    const int ntiles = hi > lo ? (hi - lo + KT - 1) / KT : 0;
    if (ntiles > 0) stage(0, lo);
    for (int t = 0; t < ntiles; ++t) {
        const int buf = t & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (t + 1 < ntiles) stage(buf ^ 1, lo + (t + 1) * KT);
        const uint32_t kt_off = (uint32_t)buf * tile_bytes;
        {   // ---- partial scores: 16 keys x all heads over this warp's quarter of the features
            float s[NH][4];
#pragma unroll
            for (int n = 0; n < NH; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
            uint32_t ka = k_frag + kt_off, qa_ = q_frag;
            for (int kk = k_lo; kk < k_hi; ++kk, ka += 32u, qa_ += 32u) {
                uint32_t a[4];
                ldsm_x4_a(a, ka);
#pragma unroll
                for (int n = 0; n < NH; ++n) {
                    uint32_t bb[2];
                    ldsm_x2_a(bb, qa_ + (uint32_t)(n * 8 * stride * 2));
                    mma16816(s[n], a, bb[0], bb[1]);
                }
            }
#pragma unroll
            for (int n = 0; n < NH; ++n) {
                part_w[n * 8] = s[n][0];
                part_w[n * 8 + 1] = s[n][1];
                part_w[8 * PS + n * 8] = s[n][2];
                part_w[8 * PS + n * 8 + 1] = s[n][3];
            }
        }
        __syncthreads();
        bool rescale = false;
        {   // ---- softmax of this warp's heads over the tile's 32 keys (lane = key)
            const int j = lo + t * KT + lane;
            const bool valid = j < hi;
            float sc[NH], mx[NH];
#pragma unroll
            for (int k = 0; k < NH; ++k) {
                const float* pp = part + lane * PS + warp + 8 * k;
                const float v = pp[0] + pp[KT * PS] + pp[2 * KT * PS] + pp[3 * KT * PS];
                sc[k] = valid ? v * L.scale : -INFINITY;
                mx[k] = sc[k];
            }
#pragma unroll
            for (int o_ = 16; o_ > 0; o_ >>= 1)
#pragma unroll
                for (int k = 0; k < NH; ++k) mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], o_));
            float p[NH], ps[NH], cr[NH];
#pragma unroll
            for (int k = 0; k < NH; ++k) {
                const float mn = fmaxf(m_run[k], mx[k]);                         // finite: the tile's first key exists
                cr[k] = expf(m_run[k] - mn);
                p[k] = expf(sc[k] - mn);
                ps[k] = p[k];
                m_run[k] = mn;
                Pt[lane * PT + warp + 8 * k] = __float2bfloat16_rn(p[k]);
            }
#pragma unroll
            for (int o_ = 16; o_ > 0; o_ >>= 1)
#pragma unroll
                for (int k = 0; k < NH; ++k) ps[k] += __shfl_xor_sync(0xffffffffu, ps[k], o_);
#pragma unroll
            for (int k = 0; k < NH; ++k) {
                l_run[k] = l_run[k] * cr[k] + ps[k];
                if (lane == 0) corr_s[warp + 8 * k] = cr[k];
            }
        }
        __syncthreads();
        {   // ---- O^T[dims of this warp's m-tiles, heads] = O^T * corr + C^T . P
            float cr[NH][2];
            bool one = true;
#pragma unroll
            for (int n = 0; n < NH; ++n) { cr[n][0] = corr_s[n * 8 + cq]; cr[n][1] = corr_s[n * 8 + cq + 1]; one = one && cr[n][0] == 1.f && cr[n][1] == 1.f; }
            rescale = !__all_sync(0xffffffffu, one);                             // once the running maxima have settled nothing is rescaled
            if (rescale) {
#pragma unroll
                for (int a = 0; a < MTW; ++a)
#pragma unroll
                    for (int n = 0; n < NH; ++n) { o[a][n][0] *= cr[n][0]; o[a][n][1] *= cr[n][1]; o[a][n][2] *= cr[n][0]; o[a][n][3] *= cr[n][1]; }
            }
#pragma unroll
            for (int k0 = 0; k0 < KT; k0 += 16) {
                uint32_t pb[NH][2];
#pragma unroll
                for (int n = 0; n < NH; ++n) ldsm_x2_trans_a(pb[n], p_frag + (uint32_t)((k0 * PT + n * 8) * 2));
#pragma unroll
                for (int a = 0; a < MTW; ++a) {
                    const int mtile = warp + 8 * a;
                    if (mtile < m_tiles) {
                        uint32_t af[4];
                        // A[m = dim][k = key] from rows stored [key][dim]: transposed 8x8 blocks (dims 0-7 | 8-15) x (keys 0-7 | 8-15)
                        ldsm_x4_trans_a(af, c_frag + kt_off + (uint32_t)((k0 * stride + mtile * 16) * 2));
#pragma unroll
                        for (int n = 0; n < NH; ++n) mma16816(o[a][n], af, pb[n][0], pb[n][1]);
                    }
                }
            }
        }
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < NH; ++k) {
            const int h = warp + 8 * k;
            ml_s[h] = m_run[k];
            // an unsplit key range normalises here, so the sink (a weight without a value) joins the sum here; key splits leave it to the merge
            ml_s[HP + h] = (L.sink && mp.splits == 1 && h < L.H) ? l_run[k] + expf(L.sink[h] - m_run[k]) : l_run[k];
        }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < MTW; ++a) {
        const int mtile = warp + 8 * a;
        if (mtile >= m_tiles) continue;
#pragma unroll
        for (int n = 0; n < NH; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = n * 8 + cq + (e & 1), dim = mtile * 16 + r0 + (e >> 1) * 8;
                if (h >= L.H) continue;
                if (mp.splits == 1) out[((size_t)i * L.H + h) * L.R + dim] = __float2bfloat16_rn(o[a][n][e] / ml_s[HP + h]);
                else mp.part[(((size_t)i * mp.splits + split) * L.H + h) * (L.R + 2) + dim] = o[a][n][e];
            }
    }
    if (mp.splits > 1)
        for (int h = tid; h < L.H; h += blockDim.x) {
            float* dst = mp.part + (((size_t)i * mp.splits + split) * L.H + h) * (L.R + 2);
            dst[L.R] = ml_s[h]; dst[L.R + 1] = ml_s[HP + h];
        }
}

size_t kt_smem(int NH, const LatentDims& L) {
    const int HP = NH * 8, dkp = (L.R + L.r + 15) / 16 * 16, stride = dkp + 8;
    return ((size_t)HP * stride + 2 * KT * stride + (size_t)KT * kt_pt_stride(NH)) * 2 + ((size_t)4 * KT * (HP + 1) + 3 * HP) * 4;
}

template <int NH, int MTW>
int launch_kt(const Batch& b, const LatentDims& L, const float* qa, const float* qr, const PagedCache& pc, void* out, const MmaParams& mp, cudaStream_t s) {
    static DevOnce once;
    if (once.need()) cudaFuncSetAttribute(latent_attn_kt_kernel<NH, MTW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    dim3 grid(b.n, mp.splits);
    latent_attn_kt_kernel<NH, MTW><<<grid, 256, kt_smem(NH, L), s>>>(b, L, qa, qr, pc, (__nv_bfloat16*)out, mp);
    return launch_check(cudaGetLastError(), "latent_attn_kt");
}

template <int NT>
int launch_nt(const Batch& b, const LatentDims& L, const float* qa, const float* qr, const PagedCache& pc, void* out, const MmaParams& mp, size_t smem,
              cudaStream_t s) {
    static DevOnce once;
    if (once.need()) cudaFuncSetAttribute(latent_attn_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const int HT = (L.H + 15) / 16;
    dim3 grid(b.n, mp.splits);
    latent_attn_mma_kernel<NT><<<grid, HT * 128, smem, s>>>(b, L, qa, qr, pc, (__nv_bfloat16*)out, mp);
    return launch_check(cudaGetLastError(), "latent_attn_mma");
}

}  // namespace

size_t latent_attn_mma_workspace(int token_splits, int H, int R) { return (size_t)token_splits * H * (R + 2) * sizeof(float); }

// the keys-as-rows form takes up to 32 heads and latents that are multiples of 16 up to 512
bool latent_attn_kt_usable(const LatentDims& L) {
    if (L.R % 16 || (L.R + L.r) % 8 || L.H > 32 || L.R > 512) return false;
    return kt_smem((L.H + 7) / 8, L) <= 200 * 1024;
}
int latent_attn_kt_ctas_per_sm(const LatentDims& L) {
    int k = (int)((227 * 1024) / (kt_smem((L.H + 7) / 8, L) + 1024));
    if (k > 8) k = 8;
    return k < 1 ? 1 : k;
}

int launch_latent_attn_kt(const Batch& b, const LatentDims& L, const float* qa, const float* qr, const PagedCache& pc, void* out, float* workspace,
                          int splits, cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    MmaParams mp;
    mp.splits = splits < 1 ? 1 : (splits > 16 ? 16 : splits);
    mp.part = workspace;
    mp.dkp = (L.R + L.r + 15) / 16 * 16;
    mp.stride = mp.dkp + 8;
    if (mp.splits > 1 && !workspace) mp.splits = 1;
    const int NH = (L.H + 7) / 8, mtw = (L.R / 16 + 7) / 8;
    int rc = WF_ERR_UNSUPPORTED;
#define KT_CASE(nh, mw) if (NH == nh && mtw == mw) rc = launch_kt<nh, mw>(b, L, qa, qr, pc, out, mp, s);
    KT_CASE(1, 1) KT_CASE(1, 2) KT_CASE(1, 3) KT_CASE(1, 4)
    KT_CASE(2, 1) KT_CASE(2, 2) KT_CASE(2, 3) KT_CASE(2, 4)
    KT_CASE(3, 1) KT_CASE(3, 2) KT_CASE(3, 3) KT_CASE(3, 4)
    KT_CASE(4, 1) KT_CASE(4, 2) KT_CASE(4, 3) KT_CASE(4, 4)
#undef KT_CASE
    if (rc == WF_ERR_UNSUPPORTED) set_error("latent_attn_kt: unsupported sizes (heads %d, latent %d)", L.H, L.R);
    if (rc) return rc;
    if (mp.splits > 1) {
        dim3 grid(b.n, L.H);
        latent_attn_merge_kernel<<<grid, 128, 0, s>>>(L.H, L.R, mp.splits, workspace, (__nv_bfloat16*)out, L.sink);
        return launch_check(cudaGetLastError(), "latent_attn_merge");
    }
    return WF_OK;
}

int latent_attn_mma_ctas_per_sm(const LatentDims& L) {
    const int HT = (L.H + 15) / 16, dkp = (L.R + L.r + 15) / 16 * 16, stride = dkp + 8;
    const size_t smem = ((size_t)HT * 16 * stride + 2 * KT * stride + (size_t)HT * 16 * (KT + 8)) * 2 + (size_t)HT * 128 * 4 + 1024;
    int k = (int)((227 * 1024) / smem);
    const int by_threads = 2048 / (HT * 128);
    if (k > by_threads) k = by_threads;
    return k < 1 ? 1 : k;
}

bool latent_attn_mma_usable(const LatentDims& L) {
    if (L.R % 32 || (L.R + L.r) % 8 || L.H > 128) return false;
    const int nt = L.R / 32;
    if (!(nt == 1 || nt == 2 || nt == 3 || nt == 4 || nt == 6 || nt == 8 || nt == 12 || nt == 16)) return false;
    const int HT = (L.H + 15) / 16, dkp = (L.R + L.r + 15) / 16 * 16, stride = dkp + 8;
    const size_t smem = ((size_t)HT * 16 * stride + 2 * KT * stride + (size_t)HT * 16 * (KT + 8)) * 2 + (size_t)HT * 128 * 4;
    return smem <= 200 * 1024 && HT * 128 <= 1024;
}

int launch_latent_attn_mma(const Batch& b, const LatentDims& L, const float* qa, const float* qr, const PagedCache& pc, void* out, float* workspace,
                           int splits, cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    MmaParams mp;
    mp.splits = splits < 1 ? 1 : (splits > 16 ? 16 : splits);
    mp.part = workspace;
    mp.dkp = (L.R + L.r + 15) / 16 * 16;
    mp.stride = mp.dkp + 8;
    if (mp.splits > 1 && !workspace) mp.splits = 1;
    const int HT = (L.H + 15) / 16;
    const size_t smem = ((size_t)HT * 16 * mp.stride + 2 * KT * mp.stride + (size_t)HT * 16 * (KT + 8)) * 2 + (size_t)HT * 128 * 4;
    int rc;
    switch (L.R / 32) {
        case 1: rc = launch_nt<1>(b, L, qa, qr, pc, out, mp, smem, s); break;
        case 2: rc = launch_nt<2>(b, L, qa, qr, pc, out, mp, smem, s); break;
        case 3: rc = launch_nt<3>(b, L, qa, qr, pc, out, mp, smem, s); break;
        case 4: rc = launch_nt<4>(b, L, qa, qr, pc, out, mp, smem, s); break;
        case 6: rc = launch_nt<6>(b, L, qa, qr, pc, out, mp, smem, s); break;
        case 8: rc = launch_nt<8>(b, L, qa, qr, pc, out, mp, smem, s); break;
        case 12: rc = launch_nt<12>(b, L, qa, qr, pc, out, mp, smem, s); break;
        case 16: rc = launch_nt<16>(b, L, qa, qr, pc, out, mp, smem, s); break;
        default: set_error("latent_attn_mma: unsupported latent size %d", L.R); return WF_ERR_UNSUPPORTED;
    }
    if (rc) return rc;
    if (mp.splits > 1) {
        dim3 grid(b.n, L.H);
        latent_attn_merge_kernel<<<grid, 128, 0, s>>>(L.H, L.R, mp.splits, workspace, (__nv_bfloat16*)out, L.sink);
        return launch_check(cudaGetLastError(), "latent_attn_merge");
    }
    return WF_OK;
}

}  // namespace seq
}  // namespace wf
