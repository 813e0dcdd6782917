// Grouped-query attention on tensor cores (bf16 mma.sync.m16n8k16, float softmax), for prompt portions and for decoding.
//
// A CTA of four warps owns one key/value head and a tile of query rows; a row is a (token, query head of that key/value head's group)
// pair, so one staged key / value tile serves every head of the group.  Keys and values are staged 64 at a time from the paged cache by
// cp.async into a ring of two (prompts) or three (decoding) buffers (rows padded by 16 bytes: conflict-free ldmatrix).  Scores S = Q K^T, then the distance penalty and the
// causal / window mask (skipped for tiles that every row of the warp sees whole), an online softmax in float in units of log 2 (scale and
// slopes carry log2 e, the exponentials are exp2), and O += P V with the weights entering the product as a TWO-term bf16 split
// (p = hi + lo, both products accumulated in float), so that the value sum sees the float weights to 2^-17 rather than rounded to bf16.
//
// Two forms of the same tile loop:
//   * prompt form: each warp has its own 16 rows and walks all 64 keys of a tile;
//   * decode form (every sequence brings one token): the four warps share the same 16 rows and each takes 16 keys of a tile; the key
//     range can also be cut over `splits` CTAs.  Partial (max, sum, weighted values) are merged through shared memory and, with splits,
//     through a float workspace and a merge kernel.
#include "seq_kernels.cuh"
#include <math.h>
#include <stdlib.h>

namespace wf {
namespace seq {

namespace {

constexpr int AM_THREADS = 128;
constexpr int AM_KT = 64;                 // keys per staged tile
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void am_ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void am_ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void am_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void am_cp16(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;          // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void am_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void am_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

struct AmParams {
    int rp2, rp2_log;        // rows per token: the group size rounded up to a power of two
    int tq;                  // tokens per CTA tile
    int splits;              // key splits (decode form)
    int ps_log;              // log2 of the page size when that is a power of two, else -1
    float* part;             // splits > 1: [n * H][splits][dv + 2] (weighted values unnormalised, max in units of log 2, sum)
};

// DKP / DVP: per-head key and value sizes rounded up to 64 or 128.  DECODE: the decode form.  NSTAGE: staged tiles (ring depth).
// EXT: the score of an element is formed in full (scale, tanh cap, bias by distance, distance penalty) instead of by the one-FMA form
// that scale and penalty alone allow.
template <int DKP, int DVP, bool DECODE, int NSTAGE, bool EXT>
__global__ void __launch_bounds__(AM_THREADS, 3) gqa_attn_mma_kernel(Batch b, GqaDims D, const __nv_bfloat16* __restrict__ qn, const float* __restrict__ gate,
                                                                    PagedCache pc, __nv_bfloat16* __restrict__ out, AmParams ap) {
    constexpr int KS = DKP + 8, VS = DVP + 8;              // shared-memory row strides in elements
    constexpr int NKS = DKP / 16;                          // k-steps of the score product
    constexpr int NVT = DVP / 8;                           // n-tiles of the value product
    constexpr int KW = DECODE ? 16 : AM_KT;                // keys of a tile that one warp consumes
    constexpr int NST = KW / 8;                            // score n-tiles per warp
    extern __shared__ __align__(16) unsigned char smraw[];
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smraw);           // [NSTAGE][AM_KT][KS]
    __nv_bfloat16* Vs = Ks + NSTAGE * AM_KT * KS;                          // [NSTAGE][AM_KT][VS]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g4 = lane >> 2, t4 = lane & 3;
    const int kvh = blockIdx.y, split = blockIdx.z;
    const int rep = D.H / D.G;
    // which sequence and which of its tokens this tile holds
    int sq = -1, tok0 = 0, ntok = 0;
    {
        // prompt form: the last tiles of a sequence see the most keys, so they are handed out first and the short ones fill the tail
        int t = DECODE ? (int)blockIdx.x : (int)(gridDim.x - 1 - blockIdx.x);
        for (int s = 0; s < b.nseq; ++s) {
            const int tiles = (b.seq_len[s] + ap.tq - 1) / ap.tq;
            if (t < tiles) { sq = s; tok0 = t * ap.tq; ntok = b.seq_len[s] - tok0 < ap.tq ? b.seq_len[s] - tok0 : ap.tq; break; }
            t -= tiles;
        }
    }
    if (sq < 0) return;
    const int flat0 = b.seq_start[sq] + tok0;              // index of the tile's first token in the flat batch
    const int pos0 = b.seq_pos0[sq] + tok0;                // its position
    const int pos_last = pos0 + ntok - 1;
    const int32_t* bt = pc.block_table + (size_t)b.seq_slot[sq] * pc.max_blocks;
    // rows of this warp: row r (0..15) of the warp's 16 -> token (row_base + r) >> rp2_log, head-in-group (row_base + r) & (rp2 - 1)
    const int row_base = DECODE ? 0 : warp * 16;
    int r_tok[2], r_head[2], r_pos[2], r_lo[2];          // r_lo: the first key the row sees (window and chunk)
    bool r_ok[2];
    float r_slope2[2];                                     // slope of the row's head times log2 e
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int r = row_base + g4 + 8 * k;
        const int tk = r >> ap.rp2_log, hg = r & (ap.rp2 - 1);
        r_ok[k] = tk < ntok && hg < rep;
        r_tok[k] = flat0 + tk; r_head[k] = kvh * rep + (hg < rep ? hg : 0); r_pos[k] = pos0 + tk;
        r_lo[k] = r_pos[k] - D.window + 1;
        if (D.chunk > 0) { const int c0 = r_pos[k] / D.chunk * D.chunk; if (c0 > r_lo[k]) r_lo[k] = c0; }
        r_slope2[k] = D.dist_exp > 0.f ? exp2f(-D.dist_exp * (float)(r_head[k] + 1) / (float)D.H) * LOG2E : 0.f;
    }
    const float scale2 = D.scale * LOG2E;
    const float cap2 = D.softcap > 0.f ? 2.f / D.softcap : 0.f;
    // first and last position among the rows of this warp that exist
    const int wpos_min = pos0 + (row_base >> ap.rp2_log);
    const int wpos_max = pos0 + ((row_base + 15) >> ap.rp2_log) < pos_last ? pos0 + ((row_base + 15) >> ap.rp2_log) : pos_last;
    // the latest "first visible key" among them (both bounds grow with the position)
    int wlo_max = wpos_max - D.window + 1;
    if (D.chunk > 0) { const int c0 = wpos_max / D.chunk * D.chunk; if (c0 > wlo_max) wlo_max = c0; }
    // query fragments (A operand), zero beyond d and for rows that do not exist
    uint32_t qf[NKS][4];
#pragma unroll
    for (int ks = 0; ks < NKS; ++ks)
#pragma unroll
        for (int k = 0; k < 2; ++k)
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                const int c = ks * 16 + hlf * 8 + 2 * t4;
                uint32_t v = 0u;
                if (r_ok[k] && c < D.d) v = *reinterpret_cast<const uint32_t*>(qn + ((size_t)r_tok[k] * D.H + r_head[k]) * D.d + c);
                qf[ks][k + 2 * hlf] = v;
            }
    // key range of the tile: every key some row of the tile may see, cut into AM_KT-key tiles aligned to multiples of AM_KT
    int lo_all = pos0 - D.window + 1 > 0 ? pos0 - D.window + 1 : 0;
    if (D.chunk > 0) { const int c0 = pos0 / D.chunk * D.chunk; if (c0 > lo_all) lo_all = c0; }
    int t_lo = lo_all / AM_KT, t_hi = pos_last / AM_KT;    // inclusive
    if (DECODE && ap.splits > 1) {
        const int nt = t_hi - t_lo + 1, per = (nt + ap.splits - 1) / ap.splits;
        t_lo += split * per;
        if (t_lo + per - 1 < t_hi) t_hi = t_lo + per - 1;
    }
    const size_t k_base = (size_t)kvh * pc.page_size * D.d, v_base = (size_t)D.G * pc.page_size * D.d + (size_t)kvh * pc.page_size * D.dv;
    const __nv_bfloat16* pool = (const __nv_bfloat16*)pc.pool + pc.layer_off;
    // a thread stages the same 16-byte column of every row it touches: 128 threads cover 128 / (row chunks) rows per pass
    constexpr int KC = DKP / 8, VC = DVP / 8;              // 16-byte chunks per row
    constexpr int KR = AM_THREADS / KC, VR = AM_THREADS / VC;
    const int kpart = tid % KC, krow = tid / KC, vpart = tid % VC, vrow = tid / VC;
    const bool kcol_ok = kpart * 8 < D.d, vcol_ok = vpart * 8 < D.dv;
    const size_t koff = k_base + kpart * 8, voff = v_base + vpart * 8;
    auto page_of = [&](int j, int& slot) -> const __nv_bfloat16* {      // the layer's part of the page that holds key j, and j's slot in it
        int pg;
        if (ap.ps_log >= 0) { pg = j >> ap.ps_log; slot = j & (pc.page_size - 1); } else { pg = j / pc.page_size; slot = j - pg * pc.page_size; }
        return pool + (size_t)bt[pg] * pc.page_stride;
    };
    auto stage = [&](int t, int buf) {
        const int j0 = t * AM_KT;
        const uint32_t kd = smem_u32(Ks + (size_t)buf * AM_KT * KS), vd = smem_u32(Vs + (size_t)buf * AM_KT * VS);
        if (KC == VC) {                                    // one page lookup per row serves the key and the value chunk
#pragma unroll
            for (int k = 0; k < AM_KT / KR; ++k) {
                const int key = krow + k * KR, j = j0 + key;
                const bool ok = j <= pos_last;
                int slot;
                const __nv_bfloat16* pg = page_of(ok ? j : 0, slot);
                am_cp16(kd + (uint32_t)(key * KS + kpart * 8) * 2u, pg + koff + (size_t)slot * D.d, ok && kcol_ok);
                if (!D.v_is_k) am_cp16(vd + (uint32_t)(key * VS + vpart * 8) * 2u, pg + voff + (size_t)slot * D.dv, ok && vcol_ok);
            }
        } else {
#pragma unroll
            for (int k = 0; k < AM_KT / KR; ++k) {
                const int key = krow + k * KR, j = j0 + key;
                const bool ok = j <= pos_last;
                int slot;
                const __nv_bfloat16* pg = page_of(ok ? j : 0, slot);
                am_cp16(kd + (uint32_t)(key * KS + kpart * 8) * 2u, pg + koff + (size_t)slot * D.d, ok && kcol_ok);
            }
#pragma unroll
            for (int k = 0; k < AM_KT / VR; ++k) {
                const int key = vrow + k * VR, j = j0 + key;
                const bool ok = j <= pos_last;
                int slot;
                const __nv_bfloat16* pg = page_of(ok ? j : 0, slot);
                am_cp16(vd + (uint32_t)(key * VS + vpart * 8) * 2u, pg + voff + (size_t)slot * D.dv, ok && vcol_ok);
            }
        }
        am_commit();
    };
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NVT][4];
#pragma unroll
    for (int j = 0; j < NVT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    const int kw0 = DECODE ? warp * 16 : 0;                // first key of the tile this warp consumes
#pragma unroll
    for (int i = 0; i < NSTAGE - 1; ++i) { if (t_lo + i <= t_hi) stage(t_lo + i, i); else am_commit(); }
    for (int t = t_lo; t <= t_hi; ++t) {
        const int buf = (t - t_lo) % NSTAGE;
        // the tile NSTAGE - 1 ahead goes into the buffer that the previous iteration finished reading (an empty group keeps the count uniform)
        if (t + NSTAGE - 1 <= t_hi) stage(t + NSTAGE - 1, (t - t_lo + NSTAGE - 1) % NSTAGE); else am_commit();
        am_wait<NSTAGE - 1>();
        __syncthreads();
        // values that are the keys are read from the staged key tile itself (same row stride: DKP == DVP then)
        const uint32_t kb = smem_u32(Ks + (size_t)buf * AM_KT * KS), vb = D.v_is_k ? kb : smem_u32(Vs + (size_t)buf * AM_KT * VS);
        // ---- scores
        float s[NST][4];
#pragma unroll
        for (int j = 0; j < NST; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < NKS; ++ks) {
#pragma unroll
            for (int jp = 0; jp < NST / 2; ++jp) {
                // matrices: (keys +0..7, dims +0), (keys +0..7, dims +8), (keys +8..15, dims +0), (keys +8..15, dims +8)
                const int mi = lane >> 3, rr = lane & 7;
                const int key = kw0 + jp * 16 + (mi >> 1) * 8 + rr, dim = ks * 16 + (mi & 1) * 8;
                uint32_t kf[4];
                am_ldsm_x4(kf, kb + (uint32_t)(key * KS + dim) * 2u);
                am_mma(s[2 * jp], qf[ks], kf[0], kf[1]);
                am_mma(s[2 * jp + 1], qf[ks], kf[2], kf[3]);
            }
        }
        // ---- distance penalty, mask, online softmax (rows g4 and g4 + 8 of the warp; a row's 4 lanes share it).  Scores are kept in
        // units of log 2 (scale and slope carry log2 e), so the exponentials are exp2.  The penalty of element (row, key) is
        // slope * (pos_row - key) = slope * (pos_row - jt0 - 2 t4) - slope * (column constant): one term per row and tile, one FMA per element.
        const int jt0 = t * AM_KT + kw0;
        float nb[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) nb[k] = -r_slope2[k] * (float)(r_pos[k] - jt0 - 2 * t4);
        float mx[2] = {-INFINITY, -INFINITY};
        // a tile every row of the warp sees whole needs no mask: its last key is not after the warp's first position, its first not before the window
        const bool whole = jt0 + KW - 1 <= wpos_min && jt0 >= wlo_max;
        if (EXT) {
#pragma unroll
            for (int j = 0; j < NST; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int k = e >> 1, key = jt0 + j * 8 + 2 * t4 + (e & 1);
                    const int dist = r_pos[k] - key;
                    const bool vis = whole || (r_ok[k] && dist >= 0 && key >= r_lo[k]);
                    float v = s[j][e] * D.scale;
                    // cap * tanh(v / cap) as cap * (1 - 2 / (exp(2 v / cap) + 1)): the hardware exponential and reciprocal keep the
                    // score to a few 1e-6 of the cap, well inside what the bf16 operands of the product leave
                    if (D.softcap > 0.f) v = D.softcap * (1.f - __fdividef(2.f, __expf(v * cap2) + 1.f));
                    if (D.rel) { const int dd = max(0, min(dist, D.rel_n - 1)); v += __ldg(D.rel + dd * D.H + r_head[k]); }
                    v = vis ? fmaf(v, LOG2E, -r_slope2[k] * (float)dist) : -INFINITY;
                    s[j][e] = v;
                    mx[k] = fmaxf(mx[k], v);
                }
        } else if (whole) {
#pragma unroll
            for (int j = 0; j < NST; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int k = e >> 1;
                    const float v = fmaf(s[j][e], scale2, fmaf(r_slope2[k], (float)(j * 8 + (e & 1)), nb[k]));
                    s[j][e] = v;
                    mx[k] = fmaxf(mx[k], v);
                }
        } else {
#pragma unroll
            for (int j = 0; j < NST; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int k = e >> 1, key = jt0 + j * 8 + 2 * t4 + (e & 1);
                    const int dist = r_pos[k] - key;
                    const bool vis = r_ok[k] && dist >= 0 && key >= r_lo[k];
                    const float v = vis ? fmaf(s[j][e], scale2, fmaf(r_slope2[k], (float)(j * 8 + (e & 1)), nb[k])) : -INFINITY;
                    s[j][e] = v;
                    mx[k] = fmaxf(mx[k], v);
                }
        }
        float corr[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 1));
            mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 2));
            const float mn = fmaxf(m_run[k], mx[k]);
            corr[k] = mn == -INFINITY ? 1.f : exp2f(m_run[k] - mn);     // nothing seen yet: keep the zeros
            m_run[k] = mn;
        }
        float ls[2] = {0.f, 0.f};
        const float msafe[2] = {m_run[0] == -INFINITY ? 0.f : m_run[0], m_run[1] == -INFINITY ? 0.f : m_run[1]};   // exp2(-inf - 0) = 0
#pragma unroll
        for (int j = 0; j < NST; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int k = e >> 1;
                const float p = exp2f(s[j][e] - msafe[k]);
                s[j][e] = p;
                ls[k] += p;
            }
#pragma unroll
        for (int k = 0; k < 2; ++k) l_run[k] = l_run[k] * corr[k] + ls[k];      // per-lane partial sums; the 4 lanes are added at the end
#pragma unroll
        for (int j = 0; j < NVT; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
        // ---- O += P V, P as hi + lo
#pragma unroll
        for (int kk = 0; kk < KW / 16; ++kk) {
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = 2 * kk + (q >> 1), e0 = (q & 1) * 2;
                const float a = s[j][e0], c = s[j][e0 + 1];
                const float ah = __bfloat162float(__float2bfloat16_rn(a)), ch = __bfloat162float(__float2bfloat16_rn(c));
                ph[q] = pack_bf16(ah, ch);
                pl[q] = pack_bf16(a - ah, c - ch);
            }
#pragma unroll
            for (int np = 0; np < NVT / 2; ++np) {
                // transposed matrices: (keys +0..7, cols +0), (keys +8..15, cols +0), (keys +0..7, cols +8), (keys +8..15, cols +8)
                const int mi = lane >> 3, rr = lane & 7;
                const int key = kw0 + kk * 16 + (mi & 1) * 8 + rr, col = np * 16 + (mi >> 1) * 8;
                uint32_t vf[4];
                am_ldsm_x4_trans(vf, vb + (uint32_t)(key * VS + col) * 2u);
                am_mma(o[2 * np], ph, vf[0], vf[1]);
                am_mma(o[2 * np], pl, vf[0], vf[1]);
                am_mma(o[2 * np + 1], ph, vf[2], vf[3]);
                am_mma(o[2 * np + 1], pl, vf[2], vf[3]);
            }
        }
        __syncthreads();                                   // the buffer is staged again in the next iteration
    }
    am_wait<0>();
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        l_run[k] += __shfl_xor_sync(0xffffffffu, l_run[k], 1);
        l_run[k] += __shfl_xor_sync(0xffffffffu, l_run[k], 2);
    }
    if (!DECODE) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if (!r_ok[k]) continue;
            const float lsum = D.sink ? l_run[k] + exp2f(-m_run[k]) : l_run[k];      // the extra key: score 0, no value
            const float mul = (gate && !D.gate_elem ? gate[(size_t)r_tok[k] * D.H + r_head[k]] : 1.f) / lsum;
            __nv_bfloat16* dst = out + ((size_t)r_tok[k] * D.H + r_head[k]) * D.dv;
            const float* ge = gate && D.gate_elem ? gate + ((size_t)r_tok[k] * D.H + r_head[k]) * D.dv : nullptr;
#pragma unroll
            for (int j = 0; j < NVT; ++j) {
                const int c = j * 8 + 2 * t4;
                if (c < D.dv) *reinterpret_cast<uint32_t*>(dst + c) = pack_bf16(o[j][2 * k] * mul * (ge ? ge[c] : 1.f), o[j][2 * k + 1] * mul * (ge ? ge[c + 1] : 1.f));
            }
        }
        return;
    }
    // ---- decode form: merge the four warps' partial results (same rows, disjoint keys) through shared memory
    float* sm_m = reinterpret_cast<float*>(smraw);         // [4][16]
    float* sm_l = sm_m + 64;                               // [4][16]
    float* sm_o = sm_l + 64;                               // [4][16][DVP]
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int r = g4 + 8 * k;
        if (t4 == 0) { sm_m[warp * 16 + r] = m_run[k]; sm_l[warp * 16 + r] = l_run[k]; }
#pragma unroll
        for (int j = 0; j < NVT; ++j) {
            const int c = j * 8 + 2 * t4;
            sm_o[((size_t)warp * 16 + r) * DVP + c] = o[j][2 * k];
            sm_o[((size_t)warp * 16 + r) * DVP + c + 1] = o[j][2 * k + 1];
        }
    }
    __syncthreads();
    for (int r = warp; r < 16; r += 4) {                   // a warp per row
        const int tk = r >> ap.rp2_log, hg = r & (ap.rp2 - 1);
        if (tk >= ntok || hg >= rep) continue;
        const int tok = flat0 + tk, head = kvh * rep + hg;
        float mg = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mg = fmaxf(mg, sm_m[w * 16 + r]);
        float sc[4], lg = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) { sc[w] = sm_m[w * 16 + r] == -INFINITY ? 0.f : exp2f(sm_m[w * 16 + r] - mg); lg += sm_l[w * 16 + r] * sc[w]; }
        if (ap.splits > 1) {
            float* dst = ap.part + (((size_t)tok * D.H + head) * ap.splits + split) * (D.dv + 2);
            for (int c = lane; c < D.dv; c += 32) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) v += sm_o[((size_t)w * 16 + r) * DVP + c] * sc[w];
                dst[c] = v;
            }
            if (lane == 0) { dst[D.dv] = mg; dst[D.dv + 1] = lg; }
        } else {
            if (D.sink) lg += exp2f(-mg);
            const float mul = (gate && !D.gate_elem ? gate[(size_t)tok * D.H + head] : 1.f) / lg;
            const float* ge = gate && D.gate_elem ? gate + ((size_t)tok * D.H + head) * D.dv : nullptr;
            for (int c = lane; c < D.dv; c += 32) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) v += sm_o[((size_t)w * 16 + r) * DVP + c] * sc[w];
                out[((size_t)tok * D.H + head) * D.dv + c] = __float2bfloat16_rn(v * mul * (ge ? ge[c] : 1.f));
            }
        }
    }
}

// one warp per (token, head): merge the key splits' partial results (maxima in units of log 2), apply the gate
__global__ void gqa_attn_merge_kernel(int rows, int splits, int dv, const float* __restrict__ part, const float* __restrict__ gate, __nv_bfloat16* __restrict__ out,
                                      int sink, int gate_elem) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* p = part + (size_t)row * splits * (dv + 2);
    float mg = -INFINITY;
    for (int z = 0; z < splits; ++z) mg = fmaxf(mg, p[(size_t)z * (dv + 2) + dv]);
    float lg = 0.f;
    for (int z = 0; z < splits; ++z) { const float m = p[(size_t)z * (dv + 2) + dv]; lg += m == -INFINITY ? 0.f : p[(size_t)z * (dv + 2) + dv + 1] * exp2f(m - mg); }
    if (sink) lg += exp2f(-mg);
    const float mul = (gate && !gate_elem ? gate[row] : 1.f) / lg;
    for (int c = lane; c < dv; c += 32) {
        float v = 0.f;
        for (int z = 0; z < splits; ++z) { const float m = p[(size_t)z * (dv + 2) + dv]; if (m != -INFINITY) v += p[(size_t)z * (dv + 2) + c] * exp2f(m - mg); }
        out[(size_t)row * dv + c] = __float2bfloat16_rn(v * mul * (gate && gate_elem ? gate[(size_t)row * dv + c] : 1.f));
    }
}

template <int DKP, int DVP, bool DECODE, int NSTAGE, bool EXT>
int am_launch(const Batch& b, const GqaDims& D, const void* qn, const float* gate, const PagedCache& pc, void* out, const AmParams& ap, int tiles, cudaStream_t s) {
    size_t smem = (size_t)NSTAGE * AM_KT * ((DKP + 8) + (DVP + 8)) * sizeof(__nv_bfloat16);
    const size_t merge = (size_t)(128 + 64 * DVP) * sizeof(float);
    if (DECODE && merge > smem) smem = merge;
    static bool attr_set = false;
    if (!attr_set) {
        if (cuda_check(cudaFuncSetAttribute(gqa_attn_mma_kernel<DKP, DVP, DECODE, NSTAGE, EXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "attention shared memory")) return WF_ERR_CUDA;
        attr_set = true;
    }
    dim3 grid(tiles, D.G, DECODE ? ap.splits : 1);
    gqa_attn_mma_kernel<DKP, DVP, DECODE, NSTAGE, EXT><<<grid, AM_THREADS, smem, s>>>(b, D, (const __nv_bfloat16*)qn, gate, pc, (__nv_bfloat16*)out, ap);
    return launch_check(cudaGetLastError(), "gqa_attn_mma");
}

template <bool DECODE, int NSTAGE>
int am_dispatch(const Batch& b, const GqaDims& D, const void* qn, const float* gate, const PagedCache& pc, void* out, const AmParams& ap, int tiles, cudaStream_t s) {
    const bool k64 = D.d <= 64, v64 = D.dv <= 64;
    if (D.softcap > 0.f || D.rel) {
        if (k64 && v64) return am_launch<64, 64, DECODE, NSTAGE, true>(b, D, qn, gate, pc, out, ap, tiles, s);
        if (k64) return am_launch<64, 128, DECODE, NSTAGE, true>(b, D, qn, gate, pc, out, ap, tiles, s);
        if (v64) return am_launch<128, 64, DECODE, NSTAGE, true>(b, D, qn, gate, pc, out, ap, tiles, s);
        return am_launch<128, 128, DECODE, NSTAGE, true>(b, D, qn, gate, pc, out, ap, tiles, s);
    }
    if (k64 && v64) return am_launch<64, 64, DECODE, NSTAGE, false>(b, D, qn, gate, pc, out, ap, tiles, s);
    if (k64) return am_launch<64, 128, DECODE, NSTAGE, false>(b, D, qn, gate, pc, out, ap, tiles, s);
    if (v64) return am_launch<128, 64, DECODE, NSTAGE, false>(b, D, qn, gate, pc, out, ap, tiles, s);
    return am_launch<128, 128, DECODE, NSTAGE, false>(b, D, qn, gate, pc, out, ap, tiles, s);
}

int g_decode_stages = -1;

}  // namespace

bool gqa_attn_mma_usable(const GqaDims& D, const PagedCache& pc) {
    const int rep = D.G > 0 ? D.H / D.G : 0;
    return rep >= 1 && rep <= 16 && D.d % 8 == 0 && D.dv % 8 == 0 && D.d <= 128 && D.dv <= 128 && (!D.v_is_k || D.d == D.dv) && pc.layer_off % 8 == 0 && pc.page_stride % 8 == 0 &&
           ((long long)pc.page_size * D.d) % 8 == 0 && D.G <= 65535;
}

bool gqa_attn_mma_takes(const GqaDims& D) { return D.chunk >= 0 && D.softcap >= 0.f; }

size_t gqa_attn_mma_workspace(int rows, int splits, int dv) { return (size_t)rows * splits * (dv + 2) * sizeof(float); }

int launch_gqa_attn_mma(const Batch& b, const GqaDims& D, const void* qn, const float* gate, const PagedCache& pc, void* out, float* workspace, int splits,
                        cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (!gqa_attn_mma_usable(D, pc)) { set_error("attention: the tensor-core form does not take these sizes"); return WF_ERR_UNSUPPORTED; }
    const int rep = D.H / D.G;
    AmParams ap;
    ap.rp2 = 1; ap.rp2_log = 0;
    while (ap.rp2 < rep) { ap.rp2 <<= 1; ++ap.rp2_log; }
    const bool decode = b.n == b.nseq;
    ap.tq = (decode ? 16 : 64) / ap.rp2;
    ap.splits = decode && workspace && splits > 1 ? splits : 1;
    ap.part = workspace;
    // every sequence's tokens are cut into tiles of tq; n / tq + nseq bounds their number (CTAs beyond the last tile return at once)
    const int tiles = decode ? b.n : b.n / ap.tq + b.nseq;
    ap.ps_log = -1;
    for (int k = 0; k < 30; ++k) if (pc.page_size == (1 << k)) ap.ps_log = k;
    if (g_decode_stages < 0) { const char* e = getenv("WF_SEQ_ATTN_STAGES"); g_decode_stages = e && atoi(e) == 3 ? 3 : 2; }
    int rc = !decode ? am_dispatch<false, 2>(b, D, qn, gate, pc, out, ap, tiles, s)
                     : (g_decode_stages == 3 ? am_dispatch<true, 3>(b, D, qn, gate, pc, out, ap, tiles, s) : am_dispatch<true, 2>(b, D, qn, gate, pc, out, ap, tiles, s));
    if (rc || ap.splits == 1) return rc;
    const int rows = b.n * D.H;
    gqa_attn_merge_kernel<<<(rows + 3) / 4, 128, 0, s>>>(rows, ap.splits, D.dv, workspace, gate, (__nv_bfloat16*)out, D.sink, D.gate_elem);
    return launch_check(cudaGetLastError(), "gqa_attn_merge");
}

}  // namespace seq
}  // namespace wf
